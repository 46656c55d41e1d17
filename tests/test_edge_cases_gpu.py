"""Edge cases of the CUDA path: empty inputs, collisions (duplicate voxels), voxels outside the
grid, a single voxel per window, every position of a window taken, batches of scenes."""
import numpy as np
import pytest
import torch

from oracle import ssw_oracle as O
from tests.cases import make_case, rel_err

pytestmark = pytest.mark.gpu


def test_empty_scene():
    from sparseswin3d_b200 import attention, window

    dev = torch.device("cuda:0")
    coords = torch.empty((0, 4), dtype=torch.int32, device=dev)
    geom = window.resolve_geometry(1, (20, 20, 20), (7, 7, 7), (3, 3, 3))
    for dtype in (torch.float32, torch.bfloat16):
        plan = window.bucket_windows(coords=coords, geom=geom, **attention.plan_params(3, 32, dtype))
        st = plan.stats()
        assert st["voxels"] == 0 and st["windows"] == 0 and st["error"] == 0
        qkv = torch.empty((0, 3, 3, 32), dtype=dtype, device=dev)
        table = torch.zeros(13 ** 3, 3, device=dev)
        out = attention.window_attention_fused(qkv, plan, table, 32 ** -0.5, use_mask=True)
        assert out.shape == (0, 96)
        dqkv, dtable = attention.window_attention_fused_backward(qkv, out, plan, table, 32 ** -0.5, True)
        assert dqkv.shape == qkv.shape and float(dtable.abs().sum()) == 0.0


def test_duplicate_voxel_is_reported_not_computed():
    from sparseswin3d_b200 import _lib, attention, window

    dev = torch.device("cuda:0")
    case = make_case(n_vox=300, grid=20, seed=1)
    coords = case["coords"].clone()
    coords[17] = coords[3]  # a collision: two voxels in the same cell
    geom = window.resolve_geometry(1, case["dims"], case["window"], case["shift"])
    plan = window.bucket_windows(coords=coords.to(dev), geom=geom, **attention.plan_params(3, 32, torch.float32))
    assert plan.stats()["error"] & _lib.DEV_DUPLICATE
    with pytest.raises(_lib.SswError):
        plan.raise_on_error()


def test_voxel_outside_the_grid_is_reported():
    from sparseswin3d_b200 import _lib, attention, window

    dev = torch.device("cuda:0")
    case = make_case(n_vox=300, grid=20, seed=2)
    geom = window.resolve_geometry(1, case["dims"], case["window"], case["shift"])
    for bad in ((0, 20, 0, 0), (0, 0, -1, 0), (1, 0, 0, 0)):  # beyond a dim, negative, batch index out of range
        coords = case["coords"].clone()
        coords[5] = torch.tensor(bad, dtype=torch.int32)
        plan = window.bucket_windows(coords=coords.to(dev), geom=geom, **attention.plan_params(3, 32, torch.float32))
        assert plan.stats()["error"] & _lib.DEV_BAD_COORD
        with pytest.raises(_lib.SswError):
            plan.raise_on_error()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_batch_of_scenes_with_full_and_singleton_windows(dtype, tol):
    """Two scenes in one call (the batch index is part of the window id): scene 0 is a completely
    full 14^3 block (eight windows with all 343 positions taken), scene 1 holds isolated voxels."""
    from sparseswin3d_b200 import attention, window

    dev = torch.device("cuda:0")
    dims, W, shift = (14, 14, 14), (7, 7, 7), (3, 3, 3)
    zz, yy, xx = np.meshgrid(np.arange(14), np.arange(14), np.arange(14), indexing="ij")
    full = np.stack([np.zeros(14 ** 3, int), zz.ravel(), yy.ravel(), xx.ravel()], 1)
    lone = np.array([[1, 0, 0, 0], [1, 13, 13, 13], [1, 7, 7, 7], [1, 3, 10, 6]])
    coords_np = np.concatenate([full, lone]).astype(np.int32)
    rng = np.random.default_rng(0)
    coords_np = coords_np[rng.permutation(coords_np.shape[0])]
    coords = torch.from_numpy(coords_np)
    N = coords.shape[0]
    idx, Bw, n, ws, ss, dp = O.window_keys(coords, 2, dims, W, shift)
    mask = O.compute_mask(dp, ws, ss)
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(N, 3, 3, 32, generator=g).to(dtype)
    table = torch.randn(13 ** 3, 3, generator=g) * 0.5
    ref = O.dense_window_attention(qkv.float(), idx, 32 ** -0.5, table, O.relative_position_index(W), mask)
    geom = window.resolve_geometry(2, dims, W, shift)
    plan = window.bucket_windows(coords=coords.to(dev), geom=geom, **attention.plan_params(3, 32, dtype))
    st = plan.stats()
    assert st["error"] == 0 and st["voxels"] == N
    counts = np.unique(idx[:, 0].numpy(), return_counts=True)[1]
    assert st["c_max"] == int(counts.max()) and st["windows"] == counts.size
    out = attention.window_attention_fused(qkv.to(dev), plan, table.to(dev), 32 ** -0.5, use_mask=True)
    assert rel_err(out.float().cpu(), ref) <= tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("what", ["voxel ids", "descriptors", "item count"])
def test_overwritten_plan_is_flagged_not_followed(dtype, what):
    """A plan buffer that was overwritten (a stale or recycled buffer): the attention kernels, forward
    and backward, must not turn its entries into addresses; they set SSW_DEV_BAD_PLAN and finish.

    The test is built so that even a missed check stays inside memory this process owns: qkv, out
    and the gradients are views into the middle third of allocations three times their size, and the
    bad voxel ids are only a little outside [0, N) (within one N on either side)."""
    from sparseswin3d_b200 import _lib, attention, window

    dev = torch.device("cuda:0")
    N = 1200
    case = make_case(n_vox=N, grid=24, seed=8)
    geom = window.resolve_geometry(1, case["dims"], case["window"], case["shift"])
    plan = window.bucket_windows(coords=case["coords"].to(dev), geom=geom, **attention.plan_params(3, 32, dtype))
    assert plan.stats()["error"] == 0

    def middle(rows_shape):
        big = torch.zeros((3 * N,) + rows_shape, dtype=dtype, device=dev)
        return big, big[N:2 * N]

    qkv_big, qkv = middle((3, 3, 32))
    qkv.copy_(case["qkv"].to(dtype))
    out_big, out = middle((96,))
    if what == "voxel ids":
        plan.pack_perm[::7] = N + 17           # just beyond [0, N): lands in the upper third if followed
        plan.pack_perm[3::11] = -5             # just below: lands in the lower third if followed
    elif what == "descriptors":
        d = plan.pack_desc
        d[::5, 0] = N + 3                      # first row beyond the voxel count
        d[1::5, 1] = 2000                      # occupancy beyond any window
        d[2::5, 2] = 70                        # more windows than a pack holds
    else:
        plan.header[_lib.H_PACKS] = plan.layout.pack_cap + 1000
    res = attention.window_attention_fused(qkv, plan, case["table"].to(dev), case["scale"], out=out)
    torch.cuda.synchronize()
    assert res.shape == (N, 96)
    assert plan.stats()["error"] & _lib.DEV_BAD_PLAN
    assert float(out_big[:N].abs().sum()) == 0.0 and float(out_big[2 * N:].abs().sum()) == 0.0  # nothing written outside
    with pytest.raises(_lib.SswError):
        plan.raise_on_error()
    # the backward follows the same plan long after the forward: same checks
    plan.header[_lib.H_ERROR] = 0
    go_big, go = middle((96,))
    go.fill_(0.01)
    dqkv, dtable = attention.window_attention_fused_backward(qkv, go, plan, case["table"].to(dev), case["scale"])
    torch.cuda.synchronize()
    assert dqkv.shape == qkv.shape
    assert plan.stats()["error"] & _lib.DEV_BAD_PLAN


def test_module_forward_raises_on_bad_indices_unless_told_not_to():
    """Upstream computes garbage silently on duplicate (window, pos) pairs; the module raises (one
    read-back of the plan's error word), and stays silent with strict=False."""
    from sparseswin3d_b200 import _lib, ops
    from sparseswin3d_b200.attention import WindowAttentionSparse
    from sparseswin3d_b200.voxels import WindowedVoxels

    dev = torch.device("cuda:0")
    case = make_case(n_vox=400, grid=20, seed=4)
    idx = case["indices"].clone()
    idx[9] = idx[2]                                   # two voxels in one cell
    m = WindowAttentionSparse(96, 3, (7, 7, 7)).to(dev)
    x = WindowedVoxels(torch.randn(400, 96, device=dev), idx.to(dev), case["n_windows"], (case["n"],))
    with torch.no_grad():
        with pytest.raises(_lib.SswError):
            m(x, None)
        y = m(x, None, strict=False)
        assert y.features.shape == (400, 96)
        with pytest.raises(_lib.SswError):           # the operator surface checks as well
            ops.qkv_sparse_indices(idx.to(dev), case["n_windows"], case["n"], 3, 32)
        idx[9, 0] = case["n_windows"]                 # a window id beyond batch_size
        with pytest.raises(_lib.SswError):
            m(WindowedVoxels(x.features, idx.to(dev), case["n_windows"], (case["n"],)), None)
