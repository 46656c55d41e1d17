"""Parity of the CUDA bucketing + fused attention path against the CPU oracle (through the C ABI)."""
import pytest
import torch

from oracle import ssw_oracle as O
from tests.cases import make_case, rel_err

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5   # |x-ref| <= tol * max(|ref|, rms(ref)), the fp32 bound of the task statement
BF16_TOL = 2e-2   # same form, bf16 inputs/outputs against the fp32 oracle


def _plan(case, dev, dtype, from_coords=True, tile=None):
    from sparseswin3d_b200 import attention, window

    pp = attention.plan_params(case["heads"], case["head_dim"], dtype, case["window"])
    if tile:
        pp["tile_rows"] = tile
    if from_coords:
        g = window.resolve_geometry(case["batch"], case["dims"], case["window"], case["shift"])
        return window.bucket_windows(coords=case["coords"].to(dev), geom=g, **pp)
    mask = case["mask"].to(dev) if case["mask"] is not None else None
    return window.bucket_windows(indices=case["indices"].to(dev), n_windows=case["n_windows"], n_per_window=case["n"],
                                 mask=mask, **pp)


def _check_plan(case, plan):
    idx = case["indices"].long()
    key = idx[:, 0] * case["n"] + idx[:, 1]
    order = torch.argsort(key)
    st = plan.stats()
    assert st["error"] == 0
    assert st["voxels"] == idx.shape[0]
    perm = plan.perm.cpu().long()
    assert torch.equal(perm, order)                      # sorted row -> voxel, bit exact
    arg_sort = O.return_inverse(O.flatten_indices(case["indices"].T.contiguous(), [case["n_windows"], case["n"]]), -1)[0]
    assert torch.equal(plan.inv_perm.cpu(), arg_sort)     # upstream's arg_sort (swin3d_base.py:674)
    wins, counts = torch.unique(idx[:, 0], return_counts=True)
    assert st["windows"] == wins.numel()
    assert torch.equal(plan.win_id[: wins.numel()].cpu().long(), wins)
    assert torch.equal(plan.occupancy().cpu().long(), counts)
    assert st["sum_c2"] == int((counts ** 2).sum())
    assert st["c_max"] == int(counts.max())
    # pack order is a permutation of the voxels
    assert torch.equal(torch.sort(plan.pack_perm.cpu().long())[0], torch.arange(idx.shape[0]))


@pytest.mark.parametrize("shift", [(0, 0, 0), (3, 3, 3)])
@pytest.mark.parametrize("from_coords", [True, False])
def test_bucket_and_fused_fp32(shift, from_coords):
    from sparseswin3d_b200 import attention

    dev = torch.device("cuda:0")
    case = make_case(n_vox=3000, grid=40, shift=shift, seed=3)
    plan = _plan(case, dev, torch.float32, from_coords)
    _check_plan(case, plan)
    ref, attn_ref = O.window_attention_core(case["qkv"], case["indices"], case["n_windows"], case["n"], case["scale"],
                                            case["table"], case["rpi"], case["mask"])
    out, attn = attention.window_attention_fused(case["qkv"].to(dev), plan, case["table"].to(dev), case["scale"],
                                                 use_mask=case["mask"] is not None, return_attn=True)
    torch.cuda.synchronize()
    assert plan.stats()["error"] == 0
    assert rel_err(out.cpu(), ref) <= FP32_TOL
    assert attn.numel() == attn_ref.values.numel()
    assert rel_err(attn.cpu(), attn_ref.values) <= FP32_TOL
    out2 = attention.window_attention_fused(case["qkv"].to(dev), plan, case["table"].to(dev), case["scale"],
                                            use_mask=case["mask"] is not None)
    # the emitting variant keeps a whole head per thread, the plain one splits it over a lane pair
    assert rel_err(out2.cpu(), out.cpu()) <= 2e-6


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, BF16_TOL), (torch.float16, 2e-3)])
def test_fused_half_types(dtype, tol):
    from sparseswin3d_b200 import attention

    dev = torch.device("cuda:0")
    case = make_case(n_vox=3000, grid=40, shift=(3, 3, 3), seed=4)
    plan = _plan(case, dev, dtype)
    qkv = case["qkv"].to(dtype)
    ref, _ = O.window_attention_core(qkv.float(), case["indices"], case["n_windows"], case["n"], case["scale"],
                                     case["table"], case["rpi"], case["mask"])
    out = attention.window_attention_fused(qkv.to(dev), plan, case["table"].to(dev), case["scale"], use_mask=True)
    assert out.dtype == dtype
    assert rel_err(out.float().cpu(), ref) <= tol


@pytest.mark.parametrize("n_vox,grid,heads,hd,window", [
    (1, 8, 3, 32, (7, 7, 7)),          # single voxel
    (40, 7, 3, 32, (7, 7, 7)),         # everything in one window
    (343, 7, 2, 16, (7, 7, 7)),        # one completely full window (c = 343 > tile)
    (2000, 14, 6, 16, (7, 7, 7)),      # dense-ish windows, several key tiles
    (500, 64, 12, 16, (7, 7, 7)),      # singletons mostly, many heads
    (3000, 18, 6, 32, (9, 9, 9)),      # window 9
    (600, 30, 3, 32, (5, 6, 7)),       # anisotropic window
])
@pytest.mark.parametrize("shift", [False, True])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, FP32_TOL), (torch.bfloat16, BF16_TOL), (torch.float16, 3e-3)])
def test_fused_shapes(n_vox, grid, heads, hd, window, shift, dtype, tol):
    """fp32 runs the CUDA-core kernel on a contiguous plan, the 16-bit types the tensor-core kernel
    on a padded plan (windows above one pack take that kernel's second phase: key tiles streamed past a resident query tile)."""
    from sparseswin3d_b200 import attention

    dev = torch.device("cuda:0")
    sh = tuple(w // 2 for w in window) if shift else (0, 0, 0)
    case = make_case(n_vox=n_vox, grid=grid, heads=heads, head_dim=hd, window=window, shift=sh, seed=n_vox)
    plan = _plan(case, dev, dtype)
    _check_plan(case, plan)
    qkv = case["qkv"].to(dtype)
    ref = O.dense_window_attention(qkv.float(), case["indices"], case["scale"], case["table"], case["rpi"], case["mask"])
    out = attention.window_attention_fused(qkv.to(dev), plan, case["table"].to(dev), case["scale"],
                                           use_mask=case["mask"] is not None)
    assert plan.stats()["error"] == 0
    assert out.dtype == dtype
    assert rel_err(out.float().cpu(), ref) <= tol


def test_padded_plan_is_rejected_for_fp32_and_coo_output():
    from sparseswin3d_b200 import _lib, attention, window

    dev = torch.device("cuda:0")
    case = make_case(n_vox=500, grid=20, seed=2)
    g = window.resolve_geometry(1, case["dims"], case["window"], case["shift"])
    plan = window.bucket_windows(coords=case["coords"].to(dev), geom=g, **attention.plan_params(3, 32, torch.bfloat16))
    assert plan.layout.padded == 1
    with pytest.raises(_lib.SswError):
        attention.window_attention_fused(case["qkv"].to(dev), plan, case["table"].to(dev), case["scale"])
    with pytest.raises(_lib.SswError):
        attention.window_attention_fused(case["qkv"].to(dev).bfloat16(), plan, case["table"].to(dev), case["scale"],
                                         return_attn=True)
    # a contiguous plan still serves 16-bit tensors (CUDA-core kernel, widened in shared memory)
    plan2 = window.bucket_windows(coords=case["coords"].to(dev), geom=g, **attention.plan_params(3, 32, torch.float32))
    a = attention.window_attention_fused(case["qkv"].to(dev).bfloat16(), plan, case["table"].to(dev), case["scale"])
    b = attention.window_attention_fused(case["qkv"].to(dev).bfloat16(), plan2, case["table"].to(dev), case["scale"])
    assert rel_err(a.float().cpu(), b.float().cpu()) <= BF16_TOL


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, BF16_TOL), (torch.float32, FP32_TOL)])
def test_skewed_occupancy_window9(dtype, tol):
    """The skewed-occupancy stress shape at reduced size: half the 9^3 windows are completely full
    (729 voxels, far above a tile), the rest hold 1-8 voxels; C = 192, 6 heads x 32, shifted and
    masked.  16-bit runs both phases of the tensor-core kernel with the bias table in global
    memory (17^3 x 6 entries do not fit next to the stages)."""
    import numpy as np

    from sparseswin3d_b200 import attention, scenes, window

    dev = torch.device("cuda:0")
    H, hd, W, shift = 6, 32, (9, 9, 9), (4, 4, 4)
    coords_np, dims = scenes.skewed_scene(grid=27, window=9, p_dense=0.5, seed=3)
    coords = torch.from_numpy(coords_np)
    N = coords.shape[0]
    idx, Bw, n, ws, ss, dp = O.window_keys(coords, 1, dims, W, shift)
    mask = O.compute_mask(dp, ws, ss)
    g = torch.Generator().manual_seed(7)
    qkv = torch.randn(N, 3, H, hd, generator=g).to(dtype)
    table = torch.randn(17 ** 3, H, generator=g) * 0.5
    ref = O.dense_window_attention(qkv.float(), idx, hd ** -0.5, table, O.relative_position_index(W), mask)
    geom = window.resolve_geometry(1, dims, W, shift)
    plan = window.bucket_windows(coords=coords.to(dev), geom=geom, **attention.plan_params(H, hd, dtype, W))
    out = attention.window_attention_fused(qkv.to(dev), plan, table.to(dev), hd ** -0.5, use_mask=True)
    st = plan.stats()
    assert st["error"] == 0 and st["c_max"] > 64 and st["voxels"] == N
    counts = np.unique(idx[:, 0].numpy(), return_counts=True)[1]
    assert st["sum_c2"] == int((counts.astype(np.int64) ** 2).sum())
    assert rel_err(out.float().cpu(), ref) <= tol


def test_plan_buffer_and_scratch_are_reused():
    """A caller that builds plans repeatedly passes its own scratch and plan buffers: the plan then
    lives in the caller's buffer and equals a freshly allocated one."""
    from sparseswin3d_b200 import attention, window

    dev = torch.device("cuda:0")
    case = make_case(n_vox=2000, grid=30, shift=(3, 3, 3), seed=9)
    g = window.resolve_geometry(1, case["dims"], case["window"], case["shift"])
    pp = attention.plan_params(3, 32, torch.float32)
    ref = window.bucket_windows(coords=case["coords"].to(dev), geom=g, **pp)
    buf = torch.empty(ref.layout.plan_ints + 100, dtype=torch.int32, device=dev)
    scratch = torch.empty(ref.layout.scratch_ints, dtype=torch.int32, device=dev)
    for _ in range(2):
        plan = window.bucket_windows(coords=case["coords"].to(dev), geom=g, scratch=scratch, plan_buffer=buf, **pp)
        assert plan.plan.data_ptr() == buf.data_ptr()
        assert torch.equal(plan.perm, ref.perm) and torch.equal(plan.inv_perm, ref.inv_perm)
        a = attention.window_attention_fused(case["qkv"].to(dev), plan, case["table"].to(dev), case["scale"], use_mask=True)
        b = attention.window_attention_fused(case["qkv"].to(dev), ref, case["table"].to(dev), case["scale"], use_mask=True)
        assert torch.equal(a, b)
