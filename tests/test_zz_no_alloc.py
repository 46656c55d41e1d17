"""ssw_bucket_windows_static: bucketing for callers that have no scratch buffer to give.

Hosts that run this library inside another framework's memory plan, or under a runtime that forbids
device allocation after start-up, cannot pass `scratch`; the library then uses a fixed array that is
part of its own image.  This test drives the entry point through the C ABI, twice in a row (the
array keeps whatever the previous call left in it), and checks every result against the regular
entry point.  It is collected last on purpose."""
import ctypes

import pytest
import torch

from tests.cases import make_case

pytestmark = pytest.mark.gpu


def _run_static(case, dev, tile, shift, plan=None):
    from sparseswin3d_b200 import _lib
    from sparseswin3d_b200 import window as W

    geom = W.resolve_geometry(case["batch"], case["dims"], case["window"], shift)
    coords = case["coords"].to(dev)
    L = _lib.PlanLayout()
    _lib.check(_lib.lib.ssw_plan_layout_init(L, coords.shape[0], geom.n_windows, geom.n_per_window, tile, 0), "layout")
    assert L.scratch_ints <= _lib.lib.ssw_bucket_windows_static_capacity()
    if plan is None:
        plan = torch.empty(L.plan_ints, dtype=torch.int32, device=dev)  # the caller's output buffer
    rw = (_lib.i32 * 3)(*case["window"])
    rc = _lib.lib.ssw_bucket_windows_static(coords.data_ptr(), geom, None, None, 0, rw, L, plan.data_ptr(),
                                            torch.cuda.current_stream(dev).cuda_stream)
    assert rc == 0, _lib.lib.ssw_status_string(rc)
    return W.WindowPlan(L, plan, tuple(case["window"]), bool(geom.shifted)), geom


def test_static_scratch_matches_regular_entry_point_twice():
    from sparseswin3d_b200 import attention
    from sparseswin3d_b200 import window as W

    dev = torch.device("cuda:0")
    tile = attention.default_tile_rows(3, 32, torch.float32, (7, 7, 7))
    # two calls in a row with different geometry and sizes: the second sees the first one's leftovers
    for seed, n_vox, shift in ((31, 3000, (0, 0, 0)), (32, 1800, (3, 3, 3))):
        case = make_case(n_vox=n_vox, grid=40, shift=shift, seed=seed)
        got, geom = _run_static(case, dev, tile, shift)
        # "allocates nothing": once its set-up call is behind it, a call leaves the device's free
        # memory exactly where it was (every tensor the second call touches exists before the reading)
        coords_dev = case["coords"].to(dev)
        case_dev = dict(case, coords=coords_dev)
        plan2 = torch.empty_like(got.plan)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        again, _ = _run_static(case_dev, dev, tile, shift, plan=plan2)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] == free_before
        assert torch.equal(again.perm, got.perm)
        ref = W.bucket_windows(coords=case["coords"].to(dev), geom=geom, rpb_window=case["window"], tile_rows=tile)
        torch.cuda.synchronize()
        sg, sr = got.stats(), ref.stats()
        assert sg == sr and sg["error"] == 0
        w = sg["windows"]
        assert torch.equal(got.perm, ref.perm) and torch.equal(got.inv_perm, ref.inv_perm)
        assert torch.equal(got.win_id[:w], ref.win_id[:w])
        assert torch.equal(got.win_start[: w + 1], ref.win_start[: w + 1])
        assert torch.equal(got.coo_start[: w + 1], ref.coo_start[: w + 1])
        # the order of equally occupied windows inside the work list is not fixed; its content is
        assert torch.equal(torch.sort(got.pack_perm)[0], torch.sort(ref.pack_perm)[0])
        qkv, table = case["qkv"].to(dev), case["table"].to(dev)
        a = attention.window_attention_fused(qkv, got, table, case["scale"], use_mask=bool(geom.shifted))
        b = attention.window_attention_fused(qkv, ref, table, case["scale"], use_mask=bool(geom.shifted))
        assert torch.equal(a, b)  # integer plan -> bit-identical attention output


def test_static_scratch_rejects_oversize():
    from sparseswin3d_b200 import _lib
    from sparseswin3d_b200 import window as W

    dev = torch.device("cuda:0")
    geom = W.resolve_geometry(1, (600, 600, 600), (7, 7, 7))  # 636 k windows x 12 ints: beyond the 16 MiB array
    L = _lib.PlanLayout()
    _lib.check(_lib.lib.ssw_plan_layout_init(L, 16, geom.n_windows, geom.n_per_window, 48, 0), "layout")
    assert L.scratch_ints > _lib.lib.ssw_bucket_windows_static_capacity()
    plan = torch.empty(L.plan_ints, dtype=torch.int32, device=dev)
    coords = torch.zeros((16, 4), dtype=torch.int32, device=dev)
    rw = (_lib.i32 * 3)(7, 7, 7)
    rc = _lib.lib.ssw_bucket_windows_static(coords.data_ptr(), geom, None, None, 0, rw, L, plan.data_ptr(), None)
    assert rc == -5
    assert b"built-in array" in _lib.lib.ssw_last_cuda_error()
