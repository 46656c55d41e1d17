"""One Swin stage (blocks of norm1 - window attention - residual - norm2 - MLP - residual,
sparse_swin/swin3d_base.py:741-782, 857-873): the one-pass add + LayerNorm kernel against torch,
and the block / stage modules against the CPU oracle's restatement of upstream's block."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from oracle import ssw_oracle as O
from tests.cases import make_case, rel_err

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("C", [16, 48, 96, 192, 384, 512])
def test_add_layernorm_against_torch(dtype, C):
    from sparseswin3d_b200 import stage

    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(C)
    for n in (1, 37, 5000):
        a = (torch.randn(n, C, generator=g) * 2 + 0.5).to(dtype).to(dev)
        b = torch.randn(n, C, generator=g).to(dtype).to(dev)
        ln = nn.LayerNorm(C).to(dev)
        with torch.no_grad():
            ln.weight.copy_(torch.randn(C, generator=g) * 0.5 + 1)
            ln.bias.copy_(torch.randn(C, generator=g) * 0.3)
        # sum and norm
        s, y = stage.add_layernorm(a, b, ln)
        s_ref = a + b                                              # rounded to dtype, as a separate add gives
        y_ref = F.layer_norm(s_ref.float(), (C,), ln.weight, ln.bias, ln.eps)
        assert torch.equal(s, s_ref)
        assert rel_err(y.float().cpu(), y_ref.cpu()) <= TOL[dtype]
        # norm only: the input is untouched and is what comes back as the sum
        s2, y2 = stage.add_layernorm(a, None, ln)
        assert s2 is a
        assert rel_err(y2.float().cpu(), F.layer_norm(a.float(), (C,), ln.weight, ln.bias, ln.eps).cpu()) <= TOL[dtype]
        # sum only, in place
        a2 = a.clone()
        s3, y3 = stage.add_layernorm(a2, b, None, sum_out=a2)
        assert y3 is None and s3.data_ptr() == a2.data_ptr() and torch.equal(s3, s_ref)


def test_add_layernorm_rejects_what_it_cannot_do():
    from sparseswin3d_b200 import _lib, stage

    dev = torch.device("cuda:0")
    a = torch.zeros(4, 10, device=dev)                      # 40-byte rows: not a multiple of 16
    with pytest.raises(_lib.SswError):
        stage.add_layernorm(a, None, nn.LayerNorm(10).to(dev))
    with pytest.raises(_lib.SswError):
        stage.add_layernorm(torch.zeros(4, 16), None, nn.LayerNorm(16))     # CPU tensor
    with pytest.raises(_lib.SswError):
        stage.add_layernorm(torch.zeros(4, 16, device=dev), torch.zeros(4, 32, device=dev), None)


def _block_params(blk):
    return {k: v.detach().cpu() for k, v in blk.state_dict().items()}


def _randomise(module, seed):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in module.named_parameters():
            if name.endswith("relative_position_bias_table"):
                p.copy_(torch.randn(p.shape, generator=g) * 0.5)
            elif name.endswith("norm1.weight") or name.endswith("norm2.weight"):
                p.copy_(1 + 0.3 * torch.randn(p.shape, generator=g))
            elif p.dim() == 1:
                p.copy_(0.2 * torch.randn(p.shape, generator=g))
            else:
                p.copy_(torch.randn(p.shape, generator=g) * (p.shape[1] ** -0.5))


@pytest.mark.parametrize("dims,win,batch", [((24, 24, 24), (7, 7, 7), 1), ((5, 30, 22), (5, 6, 7), 2)])
def test_stage_against_oracle_fp32(dims, win, batch):
    """Three blocks (W-MSA, SW-MSA, W-MSA) on a grid that needs padding; the second geometry clamps
    one axis of the window.  Fused shell (evaluation mode) against the float64 restatement."""
    from sparseswin3d_b200 import stage

    dev = torch.device("cuda:0")
    case = make_case(n_vox=900, dims=dims, window=win, batch=batch, seed=3)
    C, H = 96, 3
    layer = stage.BasicLayer(dim=C, depth=3, num_heads=H, window_size=win, drop_path=[0.0, 0.1, 0.2], qkv_bias=True).to(dev)
    _randomise(layer, 11)
    layer.eval()
    g = torch.Generator().manual_seed(5)
    feats = torch.randn(case["coords"].shape[0], C, generator=g)
    x = stage.SparseVoxels(feats.to(dev), case["coords"].to(dev), dims, batch)
    with torch.no_grad():
        y = layer(x)
    assert y.indices is x.indices and y.spatial_shape == list(dims)
    ref = O.basic_layer(feats, case["coords"], batch, dims, win, [_block_params(b) for b in layer.blocks], H)
    assert rel_err(y.features.cpu(), ref) <= 2e-4
    # a single block called on its own (its own plan) equals the first block of the stage
    with torch.no_grad():
        y0 = layer.blocks[0](x, None)
    ref0 = O.swin_block(feats, case["coords"], batch, dims, win, (0, 0, 0), _block_params(layer.blocks[0]), H)
    assert rel_err(y0.features.cpu(), ref0) <= 1e-4
    # the unfused shell (torch LayerNorm and adds: what runs under autograd) gives the same values
    layer.train()        # drop_path > 0 in training disables the one-pass shell; make it deterministic:
    for b in layer.blocks:
        b.drop_path = nn.Identity()
    y_t = layer(x)
    assert y_t.features.requires_grad
    assert rel_err(y_t.features.detach().cpu(), ref) <= 2e-4


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 6e-2), (torch.float16, 1e-2)])
def test_stage_16bit_against_oracle(dtype, tol):
    from sparseswin3d_b200 import stage

    dev = torch.device("cuda:0")
    case = make_case(n_vox=1500, grid=30, seed=4)
    C, H, win = 96, 3, (7, 7, 7)
    layer = stage.BasicLayer(dim=C, depth=2, num_heads=H, window_size=win, qkv_bias=True).to(dev)
    _randomise(layer, 12)
    layer = layer.to(dtype).eval()
    g = torch.Generator().manual_seed(6)
    feats = torch.randn(1500, C, generator=g).to(dtype)
    x = stage.SparseVoxels(feats.to(dev), case["coords"].to(dev), case["dims"], 1)
    with torch.no_grad():
        y = layer(x)
    prm = [{k: v.float() for k, v in _block_params(b).items()} for b in layer.blocks]
    ref = O.basic_layer(feats.float(), case["coords"], 1, case["dims"], win, prm, H)
    assert rel_err(y.features.float().cpu(), ref) <= tol


def test_stage_reuses_two_plans_and_captures_into_a_graph():
    """depth 4: two bucketing calls serve four blocks; with caller-held plans a forward launches no
    bucketing kernel at all and captures into a CUDA graph."""
    from sparseswin3d_b200 import _lib, stage

    dev = torch.device("cuda:0")
    case = make_case(n_vox=2500, grid=36, seed=9)
    C, H, win = 96, 3, (7, 7, 7)
    layer = stage.BasicLayer(dim=C, depth=4, num_heads=H, window_size=win, qkv_bias=True).to(dev).eval()
    _randomise(layer, 13)
    feats = torch.randn(2500, C, device=dev)
    x = stage.SparseVoxels(feats, case["coords"].to(dev), case["dims"], 1)
    with torch.no_grad():
        want = layer(x).features.clone()
        plans = layer.build_plans(x, feats.dtype)
        layer.strict = False
        layer(x, plans=plans)                     # warm-up outside capture
        torch.cuda.synchronize()
        side = torch.cuda.Stream(device=dev)
        g = torch.cuda.CUDAGraph(keep_graph=True)
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                out = layer(x, plans=plans).features
        info = _lib.graph_edges(g)
        g.instantiate()
        g.replay()
        torch.cuda.synchronize()
    assert torch.equal(out, want)
    names = " ".join(e[0] + " " + e[1] for e in info["edges"])
    assert "k_count" not in names and "k_scatter" not in names          # no bucketing inside the forward
    assert names.count("k_add_layernorm") > 0 and "k_attn_fused" in names
    assert all(p.stats()["error"] == 0 for p in plans)


@pytest.mark.parametrize("n_vox", [0, 1, 3])
def test_stage_on_almost_empty_scenes(n_vox):
    """No voxel, one voxel, three voxels: nothing to attend to but oneself (or nobody)."""
    from sparseswin3d_b200 import stage

    dev = torch.device("cuda:0")
    C, H, win, dims = 96, 3, (7, 7, 7), (10, 12, 9)
    layer = stage.BasicLayer(dim=C, depth=2, num_heads=H, window_size=win, qkv_bias=True).to(dev).eval()
    _randomise(layer, 21)
    coords = torch.tensor([[0, 1, 2, 3], [0, 9, 11, 8], [0, 1, 2, 4]][:n_vox], dtype=torch.int32).reshape(n_vox, 4)
    feats = torch.randn(n_vox, C, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        y = layer(stage.SparseVoxels(feats.to(dev), coords.to(dev), dims, 1))
    assert y.features.shape == (n_vox, C)
    if n_vox:
        ref = O.basic_layer(feats, coords, 1, dims, win, [_block_params(b) for b in layer.blocks], H)
        assert rel_err(y.features.cpu(), ref) <= 2e-4


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 3e-2)])
def test_stage_at_full_size_fused_and_unfused_shell_agree(dtype, tol):
    """The benchmark room (150 000 voxels), depth 2: the stage as built (two plans, one-pass shell)
    against upstream's structure on the same kernels (every block buckets for itself, torch
    LayerNorm and adds); both forms use the attention kernels the full-size parity tests pin."""
    from sparseswin3d_b200 import scenes, stage

    dev = torch.device("cuda:0")
    coords_np, dims = scenes.room_scene(150_000, seed=0)
    C, H, win = 96, 3, (7, 7, 7)
    layer = stage.BasicLayer(dim=C, depth=2, num_heads=H, window_size=win, qkv_bias=True).to(dev)
    _randomise(layer, 31)
    layer = layer.to(dtype).eval()
    feats = torch.randn(150_000, C, generator=torch.Generator().manual_seed(2)).to(dtype).to(dev)
    x = stage.SparseVoxels(feats, torch.from_numpy(coords_np).to(dev), dims, 1)
    with torch.no_grad():
        a = layer(x).features
        layer.reuse_plans, layer.fuse_shell = False, False
        b = layer(x).features
    assert rel_err(a.float().cpu(), b.float().cpu()) <= tol
