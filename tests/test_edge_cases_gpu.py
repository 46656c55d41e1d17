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
def test_overwritten_plan_is_flagged_not_followed(dtype):
    """A plan buffer whose voxel ids were overwritten (a stale or recycled buffer): the attention
    kernel must not use them as addresses; it sets SSW_DEV_BAD_PLAN and finishes."""
    from sparseswin3d_b200 import _lib, attention, window

    dev = torch.device("cuda:0")
    case = make_case(n_vox=1200, grid=24, seed=8)
    geom = window.resolve_geometry(1, case["dims"], case["window"], case["shift"])
    plan = window.bucket_windows(coords=case["coords"].to(dev), geom=geom, **attention.plan_params(3, 32, dtype))
    assert plan.stats()["error"] == 0
    plan.pack_perm[::7] = 2 ** 30          # far outside [0, N)
    plan.pack_perm[3::11] = -5
    out = attention.window_attention_fused(case["qkv"].to(dtype).to(dev), plan, case["table"].to(dev), case["scale"])
    torch.cuda.synchronize()
    assert out.shape == (1200, 96)
    assert plan.stats()["error"] & _lib.DEV_BAD_PLAN
    with pytest.raises(_lib.SswError):
        plan.raise_on_error()
