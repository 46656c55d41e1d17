"""Integer parity of the window geometry on the device, bit for bit against the CPU oracle:
(window, pos) of every voxel as upstream's pad + roll + window_partition_sparse leave them
(sparse_swin/swin3d_base.py:336-372, 501-554) and the shift-mask region id of every voxel as
compute_mask + sp_add_mask look it up (swin3d_base.py:436-452, 574-576: mask[w % nW, pos]).

Both places the library keeps a region id are checked: the int8 array `ssw_window_keys` returns and
the region bits of the plan's per-row metadata.  The cases mix clamped and shifted axes, because
get_window_size (swin3d_base.py:276-300) zeroes the shift of a clamped axis and the slice loops of
compute_mask then give that whole axis region 2."""
import numpy as np
import pytest
import torch

from oracle import ssw_oracle as O
from tests.cases import make_case, rel_err, room_crop_case

pytestmark = pytest.mark.gpu

# (dims, window, shift, batch, voxels per scene)
GEOMETRIES = [
    ((20, 21, 22), (5, 6, 7), (2, 3, 3), 1, 1500),   # nothing clamped, anisotropic window, padding on every axis
    ((5, 30, 22), (5, 6, 7), (2, 3, 3), 1, 900),     # one clamped axis (its shift collapses to 0), two shifted
    ((5, 30, 6), (5, 6, 7), (2, 3, 3), 1, 500),      # two clamped axes, one shifted; window shrinks to 5x6x6
    ((24, 24, 24), (7, 7, 7), (3, 0, 3), 1, 2000),   # shift 0 requested on one axis only
    ((24, 24, 24), (7, 7, 7), (0, 0, 3), 1, 2000),   # shifted along one axis only
    ((16, 18, 20), (7, 7, 7), (3, 3, 3), 2, 1200),   # a batch of two scenes: the batch index is part of the window id
]


def _oracle_regions(case):
    idx = case["indices"].long()
    mask = case["mask"]
    return mask[idx[:, 0] % mask.shape[0], idx[:, 1]]


def _check_geometry_ints(case, dev):
    from sparseswin3d_b200 import _lib, attention, window

    geom = window.resolve_geometry(case["batch"], case["dims"], case["window"], case["shift"])
    assert tuple(geom.ws) == tuple(case["ws"]) and tuple(geom.ss) == tuple(case["ss"])
    assert tuple(geom.dims_p) == tuple(case["dims_p"])
    assert geom.n_windows == case["n_windows"] and geom.n_per_window == case["n"]
    coords = case["coords"].to(dev)
    idx, region, err = window.window_keys(coords, geom, with_region=True)
    assert idx.dtype == torch.int32 and region.dtype == torch.int8
    assert int(err) == 0
    assert torch.equal(idx.cpu(), case["indices"])                 # window_partition_sparse, bit exact
    want = _oracle_regions(case)
    assert torch.equal(region.cpu(), want)                         # compute_mask[w % nW, pos], bit exact
    # the same ids as the fused kernels see them: region bits of the plan's row metadata
    for dtype in (torch.float32, torch.bfloat16):
        plan = window.bucket_windows(coords=coords, geom=geom, **attention.plan_params(3, 32, dtype, case["window"]))
        assert plan.stats()["error"] == 0
        vox = plan.pack_perm.cpu().long()
        meta = plan.pack_meta.cpu()
        assert torch.equal(meta & 1023, case["indices"][vox, 1])   # in-window position
        assert torch.equal(((meta >> 10) & 31).to(torch.int8), want[vox])
    return geom


@pytest.mark.parametrize("dims,win,shift,batch,n_vox", GEOMETRIES)
def test_window_keys_and_region_ids_bit_exact(dims, win, shift, batch, n_vox):
    dev = torch.device("cuda:0")
    case = make_case(n_vox=n_vox, dims=dims, window=win, shift=shift, batch=batch, seed=sum(dims))
    assert case["mask"] is not None
    _check_geometry_ints(case, dev)


def test_window_keys_room_crop_shift3():
    """The x,y < 200 corner of the benchmark room, shift 3: 36 000 voxels, padded grid on every axis."""
    dev = torch.device("cuda:0")
    case = room_crop_case(shift=(3, 3, 3))
    _check_geometry_ints(case, dev)


def test_unshifted_geometry_has_no_regions():
    from sparseswin3d_b200 import window

    dev = torch.device("cuda:0")
    case = make_case(n_vox=800, dims=(20, 21, 22), window=(5, 6, 7), shift=(0, 0, 0), seed=5)
    geom = window.resolve_geometry(1, case["dims"], case["window"], case["shift"])
    idx, region, err = window.window_keys(case["coords"].to(dev), geom, with_region=True)
    assert int(err) == 0 and torch.equal(idx.cpu(), case["indices"])
    assert int(region.abs().max()) == 0


@pytest.mark.parametrize("dims,win,shift,batch,n_vox", GEOMETRIES[:4])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_fused_attention_on_clamped_and_partly_shifted_grids(dims, win, shift, batch, n_vox, dtype, tol):
    """Values on the same geometries: a clamped window has fewer positions than the module's window,
    and upstream slices its relative_position_index to [:n, :n] (swin3d_base.py:662-664), which pairs
    positions of the *clamped* window with bias rows computed for the *module's* window."""
    from sparseswin3d_b200 import attention, window

    dev = torch.device("cuda:0")
    case = make_case(n_vox=n_vox, dims=dims, window=win, shift=shift, batch=batch, seed=sum(dims) + 1)
    geom = window.resolve_geometry(batch, dims, win, shift)
    plan = window.bucket_windows(coords=case["coords"].to(dev), geom=geom,
                                 **attention.plan_params(case["heads"], case["head_dim"], dtype, win))
    qkv = case["qkv"].to(dtype)
    ref = O.dense_window_attention(qkv.float(), case["indices"], case["scale"], case["table"], case["rpi"], case["mask"])
    out = attention.window_attention_fused(qkv.to(dev), plan, case["table"].to(dev), case["scale"], use_mask=True)
    assert plan.stats()["error"] == 0
    assert rel_err(out.float().cpu(), ref) <= tol
    if dtype == torch.float32:  # and the unfused chain on upstream's (indices, mask) interface agrees
        chain, _ = O.window_attention_core(case["qkv"], case["indices"], case["n_windows"], case["n"], case["scale"],
                                           case["table"], case["rpi"], case["mask"])
        assert rel_err(out.cpu(), chain) <= tol


def test_random_geometries_bit_exact():
    """A seeded sweep over random grids, windows, shifts and batch sizes: window keys, region ids and
    the sorted permutation against the oracle / a host sort of the same keys, bit for bit."""
    from sparseswin3d_b200 import attention, window

    dev = torch.device("cuda:0")
    rng = np.random.default_rng(2024)
    for trial in range(24):
        dims = tuple(int(v) for v in rng.integers(4, 36, 3))
        win = tuple(int(v) for v in rng.integers(3, 10, 3))
        shift = tuple(int(rng.integers(0, w // 2 + 1)) for w in win)
        batch = int(rng.integers(1, 4))
        n_vox = int(min(rng.integers(1, 1500), dims[0] * dims[1] * dims[2]))
        case = make_case(n_vox=n_vox, dims=dims, window=win, shift=shift, batch=batch, seed=1000 + trial)
        geom = window.resolve_geometry(batch, dims, win, shift)
        coords = case["coords"].to(dev)
        idx, region, err = window.window_keys(coords, geom, with_region=True)
        assert int(err) == 0 and torch.equal(idx.cpu(), case["indices"]), (dims, win, shift, batch)
        if case["mask"] is not None:
            assert torch.equal(region.cpu(), _oracle_regions(case)), (dims, win, shift, batch)
        else:
            assert int(region.abs().max()) == 0
        plan = window.bucket_windows(coords=coords, geom=geom, **attention.plan_params(3, 32, torch.float32, win))
        st = plan.stats()
        assert st["error"] == 0 and st["voxels"] == coords.shape[0]
        key = case["indices"][:, 0].long() * case["n"] + case["indices"][:, 1].long()
        want_perm = torch.argsort(key, stable=True)
        assert torch.equal(plan.perm.cpu().long(), want_perm), (dims, win, shift, batch)
        inv = torch.empty_like(want_perm)
        inv[want_perm] = torch.arange(want_perm.numel())
        assert torch.equal(plan.inv_perm.cpu().long(), inv)
        counts = torch.unique(case["indices"][:, 0], return_counts=True)[1]
        assert torch.equal(plan.occupancy().cpu().long(), counts) and st["windows"] == counts.numel()
