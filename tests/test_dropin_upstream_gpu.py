"""Drop-in test: upstream's OWN Python source runs on this library's operator module.

`sparse_swin/swin3d_base.py` is executed unmodified (read from an upstream checkout named by
SSW_REFERENCE, else from the copy `oracle/build_ref.py` stages in the untracked oracle/_ref/).  The
modules it imports but that are not installable here (spconv, pointcept) are replaced by empty
stand-ins, `torch.compile` by the identity, and `torch.utils.cpp_extension.load` - the call with
which upstream JIT-builds its CUDA extension (swin3d_base.py:22-26) - by a function that hands back
`sparseswin3d_b200.ops`.  Upstream's `WindowAttentionSparse.forward` (swin3d_base.py:654-677), its
`SparseTensor`, autograd Functions and helpers then run line by line as upstream wrote them, every
`ops.*` call landing in this library.  Results are held to the fixtures recorded from upstream's own
extension (tests/golden/) and to this package's module with the same weights."""
import sys
import types
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle.build_ref import upstream_python_source
from tests.cases import rel_err

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).resolve().parent / "golden"


def _load_upstream():
    src = upstream_python_source()
    if src is None:
        pytest.skip("upstream swin3d_base.py is neither in $SSW_REFERENCE nor staged under oracle/_ref/")
    from sparseswin3d_b200 import ops as our_ops

    class _Registry:
        def register_module(self, *a, **k):
            return lambda cls: cls

    sp = types.ModuleType("spconv.pytorch")
    from sparseswin3d_b200 import sparse_conv
    from sparseswin3d_b200.stage import SparseVoxels

    # the three spconv layers and two containers upstream's shell is written against
    sp.SubMConv3d, sp.SparseConv3d, sp.SparseInverseConv3d = (sparse_conv.SubMConv3d, sparse_conv.SparseConv3d,
                                                              sparse_conv.SparseInverseConv3d)
    sp.SparseModule, sp.SparseSequential = sparse_conv.SparseModule, sparse_conv.SparseSequential
    sp.SparseConvTensor = SparseVoxels      # the container upstream's blocks assert on (swin3d_base.py:338)
    spconv = types.ModuleType("spconv")
    spconv.pytorch = sp
    builder = types.ModuleType("pointcept.models.builder")
    builder.MODELS = _Registry()
    utils = types.ModuleType("pointcept.models.utils")
    utils.offset2batch = lambda offset: None
    stand_ins = {"spconv": spconv, "spconv.pytorch": sp, "pointcept": types.ModuleType("pointcept"),
                 "pointcept.models": types.ModuleType("pointcept.models"), "pointcept.models.builder": builder,
                 "pointcept.models.utils": utils}
    import torch.utils.cpp_extension as cpp_ext

    saved_modules = {k: sys.modules.get(k) for k in stand_ins}
    saved_load, saved_compile = cpp_ext.load, torch.compile
    mod = types.ModuleType("upstream_swin3d_base")
    mod.__file__ = str(src)
    try:
        sys.modules.update(stand_ins)
        cpp_ext.load = lambda *a, **k: our_ops
        torch.compile = lambda fn=None, *a, **k: fn if fn is not None else (lambda f: f)
        exec(compile(src.read_text(), str(src), "exec"), mod.__dict__)
    finally:
        cpp_ext.load, torch.compile = saved_load, saved_compile
        for k, v in saved_modules.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    assert mod.ops is our_ops
    return mod


class _GivenQkv(nn.Module):
    """Stands where the module's qkv Linear is: returns the fixture's qkv whatever the features."""

    def __init__(self, qkv):
        super().__init__()
        self.qkv = qkv

    def forward(self, features):
        return self.qkv.reshape(self.qkv.shape[0], -1)


@pytest.mark.parametrize("name", ["wmsa_h3_hd32", "swmsa_h3_hd32", "swmsa_h2_hd16_dense"])
def test_upstream_forward_on_this_library_matches_upstream_fixture(name):
    from sparseswin3d_b200.voxels import WindowedVoxels

    up = _load_upstream()
    dev = torch.device("cuda:0")
    z = np.load(GOLDEN / f"{name}.npz")
    qkv = torch.from_numpy(z["in_qkv"]).to(dev)
    N, _, H, hd = qkv.shape
    C = H * hd
    m = up.WindowAttentionSparse(C, H, (7, 7, 7)).to(dev)
    with torch.no_grad():
        m.relative_position_bias_table.copy_(torch.from_numpy(z["in_table"]))
    m.qkv, m.proj = _GivenQkv(qkv), nn.Identity()
    mask = torch.from_numpy(z["in_mask"]).to(dev) if z["in_mask"].size else None
    x = WindowedVoxels(torch.zeros(N, C, device=dev), torch.from_numpy(z["in_indices"]).to(dev),
                       int(z["in_n_windows"]), (int(z["in_n"]),))
    with torch.no_grad():
        y = m(x, mask)
    out = y.features.cpu()
    assert rel_err(out, torch.from_numpy(z["out"])) <= 1e-5          # what upstream's own extension gave


def test_upstream_module_and_this_module_agree_forward_and_backward():
    """Same weights in upstream's module (unfused chain on this library's operators, upstream's own
    autograd Functions) and in this package's module (fused kernels): outputs and gradients agree."""
    from sparseswin3d_b200.attention import WindowAttentionSparse
    from sparseswin3d_b200.voxels import WindowedVoxels
    from tests.cases import make_case

    up = _load_upstream()
    dev = torch.device("cuda:0")
    case = make_case(n_vox=700, grid=24, shift=(3, 3, 3), seed=21)
    C, H = 96, 3
    torch.manual_seed(5)
    ours = WindowAttentionSparse(C, H, (7, 7, 7), qkv_bias=True).to(dev)
    with torch.no_grad():
        ours.relative_position_bias_table.normal_(0, 0.5)
    theirs = up.WindowAttentionSparse(C, H, (7, 7, 7), qkv_bias=True).to(dev)
    theirs.load_state_dict(ours.state_dict())                        # state_dict compatible, strict
    feats = torch.randn(case["coords"].shape[0], C, device=dev)
    idx, mask = case["indices"].to(dev), case["mask"].to(dev)

    def run(module):
        f = feats.clone().requires_grad_(True)
        x = WindowedVoxels(f, idx, case["n_windows"], (case["n"],))
        y = module(x, mask).features
        (y * torch.linspace(-1, 1, y.numel(), device=dev).view_as(y)).sum().backward()
        return y.detach().cpu(), f.grad.cpu(), module.relative_position_bias_table.grad.cpu(), module.qkv.weight.grad.cpu()

    ya, fa, ta, wa = run(ours)
    yb, fb, tb, wb = run(theirs)
    assert rel_err(ya, yb) <= 1e-5
    assert rel_err(fa, fb) <= 1e-4 and rel_err(ta, tb) <= 1e-4 and rel_err(wa, wb) <= 1e-4


@pytest.mark.parametrize("depth", [2, 3])
def test_upstream_stage_and_this_stage_agree(depth):
    """Upstream's own BasicLayer / SwinTransformerBlock (swin3d_base.py:680-873: pad, roll, partition,
    attention, reverse, roll back, crop in every block, on this library's operators) against this
    package's stage (two plans per stage, one-pass add + LayerNorm shell) with the same weights."""
    from sparseswin3d_b200 import stage
    from tests.cases import make_case

    up = _load_upstream()
    dev = torch.device("cuda:0")
    dims, win = (20, 24, 22), (7, 7, 7)
    case = make_case(n_vox=1200, dims=dims, window=win, seed=31)
    C, H = 96, 3
    torch.manual_seed(7)
    ours = stage.BasicLayer(dim=C, depth=depth, num_heads=H, window_size=win, drop_path=[0.0] * depth, qkv_bias=True).to(dev)
    with torch.no_grad():
        for b in ours.blocks:
            b.attn.relative_position_bias_table.normal_(0, 0.5)
            b.norm1.weight.normal_(1, 0.2), b.norm1.bias.normal_(0, 0.2)
    theirs = up.BasicLayer(dim=C, depth=depth, num_heads=H, window_size=win, drop_path=[0.0] * depth, qkv_bias=True).to(dev)
    theirs.load_state_dict(ours.state_dict())                        # same parameter names, strict
    ours.eval(), theirs.eval()
    feats = torch.randn(1200, C, device=dev)
    coords = case["coords"].to(dev)
    with torch.no_grad():
        ya = ours(stage.SparseVoxels(feats, coords, dims, 1)).features
        yb_x = theirs(stage.SparseVoxels(feats.clone(), coords.clone(), dims, 1))
    assert list(yb_x.spatial_shape) == list(dims) and torch.equal(yb_x.indices.cpu(), coords.cpu())
    assert rel_err(ya.cpu(), yb_x.features.cpu()) <= 1e-4


def test_upstream_stage_with_patch_merging_and_patch_expand():
    """Upstream's BasicLayer with its own PatchMerging as `downsample`, then its PatchExpand
    (swin3d_base.py:950-1004), written against spconv's SparseConv3d / SparseInverseConv3d: here
    those names resolve to this library's layers.  Against this package's stage + PatchMerging +
    PatchExpand with the same weights, and against the dense operations of the oracle."""
    import contextlib
    import io

    from oracle import ssw_oracle as O
    from sparseswin3d_b200 import sparse_conv, stage
    from tests.cases import make_case

    up = _load_upstream()
    dev = torch.device("cuda:0")
    dims, win, C, H = (14, 16, 12), (7, 7, 7), 48, 3
    case = make_case(n_vox=900, dims=dims, window=win, heads=H, head_dim=C // H, seed=77)
    torch.manual_seed(3)
    with contextlib.redirect_stdout(io.StringIO()):      # upstream prints the indice_key when constructing
        theirs = up.BasicLayer(dim=C, depth=2, num_heads=H, window_size=win, drop_path=[0.0, 0.0], qkv_bias=True,
                               downsample=up.PatchMerging, indice_key="m0").to(dev).eval()
        theirs_up = up.PatchExpand(2 * C, indice_key="m0").to(dev).eval()
    ours = stage.BasicLayer(dim=C, depth=2, num_heads=H, window_size=win, drop_path=[0.0, 0.0], qkv_bias=True,
                            downsample=sparse_conv.PatchMerging, indice_key="m0").to(dev).eval()
    ours_up = sparse_conv.PatchExpand(2 * C, indice_key="m0").to(dev).eval()
    ours.load_state_dict(theirs.state_dict())
    ours_up.load_state_dict(theirs_up.state_dict())
    feats = torch.randn(900, C, device=dev)
    coords = case["coords"].to(dev)
    with torch.no_grad():
        ya = ours(stage.SparseVoxels(feats, coords, dims, 1))
        yb = theirs(stage.SparseVoxels(feats.clone(), coords, dims, 1))
        za, zb = ours_up(ya), theirs_up(yb)
    assert list(ya.spatial_shape) == [7, 8, 6] == list(yb.spatial_shape)
    assert torch.equal(ya.indices, yb.indices) and ya.features.shape[1] == 2 * C
    assert rel_err(ya.features.cpu(), yb.features.cpu()) <= 1e-4
    assert rel_err(za.features.cpu(), zb.features.cpu()) <= 1e-4 and torch.equal(za.indices.cpu(), case["coords"])
    # the downsampling itself against the dense convolution on the stage's output
    blocks_out = O.basic_layer(feats.cpu(), case["coords"], 1, dims, win,
                               [{k: v.detach().cpu() for k, v in b.state_dict().items()} for b in ours.blocks], H)
    normed = torch.nn.functional.layer_norm(blocks_out, (C,), ours.downsample.norm.weight.detach().cpu().double(),
                                            ours.downsample.norm.bias.detach().cpu().double(), 1e-5)
    ref, ref_idx, _ = O.strided_conv3d(normed, case["coords"], 1, dims, ours.downsample.reduction.weight.detach().cpu().double())
    assert torch.equal(ya.indices.cpu(), ref_idx) and rel_err(ya.features.cpu(), ref) <= 3e-4
