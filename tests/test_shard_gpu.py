"""Window-range sharding.  On one GPU: a scene bucketed range by range into one output buffer, and
the multi-destination store, equal the single pass bit for bit.  On two GPUs (skipped when the box
has one): ranks store their rows into each other's buffers and both end up with the single-GPU
output, bit for bit; so does the all-gather alternative."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("world", [2, 5])
def test_ranges_on_one_gpu_equal_single_pass(dtype, world):
    from sparseswin3d_b200 import attention, shard, window
    from tests.cases import make_case, skewed_case

    dev = torch.device("cuda:0")
    for case in (make_case(n_vox=6000, grid=48, shift=(3, 3, 3), seed=41), skewed_case()):
        geom = window.resolve_geometry(case["batch"], case["dims"], case["window"], case["shift"])
        coords, qkv, table = case["coords"].to(dev), case["qkv"].to(dtype).to(dev), case["table"].to(dev)
        pp = attention.plan_params(case["heads"], case["head_dim"], dtype, case["window"])
        use_mask = bool(geom.shifted)
        full = window.bucket_windows(coords=coords, geom=geom, **pp)
        ref = attention.window_attention_fused(qkv, full, table, case["scale"], use_mask=use_mask)
        bounds = shard.plan_window_ranges(coords, geom, world, **pp)
        assert bounds[0] == 0 and bounds[-1] == geom.n_windows and all(a <= b for a, b in zip(bounds, bounds[1:]))
        out = torch.full_like(ref, float("nan"))
        twin = torch.full_like(ref, float("nan"))          # stands for a peer's buffer
        taken = 0
        costs = []
        for r in range(world):
            plan = window.bucket_windows(coords=coords, geom=geom, window_range=(bounds[r], bounds[r + 1]), **pp)
            attention.window_attention_fused(qkv, plan, table, case["scale"], use_mask=use_mask, out=out,
                                             peer_out_ptrs=[twin.data_ptr()])
            st = plan.stats()
            assert st["error"] == 0
            taken += st["voxels"]
            costs.append(float(shard.window_cost(plan.occupancy().cpu()).sum()))
        assert taken == coords.shape[0]
        assert torch.equal(out, ref) and torch.equal(twin, ref)
        # the estimate the cuts balance: no range above its share by more than the largest window
        c_max = float(shard.window_cost(full.occupancy().cpu()).max())
        assert max(costs) <= sum(costs) / world + c_max + 1e-6


def _worker(rank, world, port, q):
    import torch.distributed as dist

    from sparseswin3d_b200 import attention, shard, window
    from tests.cases import make_case

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        ok = []
        for dtype in (torch.float32, torch.bfloat16):
            case = make_case(n_vox=6000, grid=48, shift=(3, 3, 3), seed=41)
            geom = window.resolve_geometry(1, case["dims"], case["window"], case["shift"])
            coords, qkv, table = case["coords"].to(dev), case["qkv"].to(dtype).to(dev), case["table"].to(dev)
            pp = attention.plan_params(3, 32, dtype, case["window"])
            ref = attention.window_attention_fused(qkv, window.bucket_windows(coords=coords, geom=geom, **pp), table,
                                                   case["scale"], use_mask=True)
            bounds = shard.plan_window_ranges(coords, geom, world, **pp)
            rows = shard.PeerRows(coords.shape[0], 96, dtype, dev)
            rows.local.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            for _ in range(2):   # a second pass over the same buffers
                res = shard.sharded_window_attention(coords, qkv, geom, table, case["scale"], case["window"], rank, world,
                                                     bounds, rows=rows)
            torch.cuda.synchronize()
            n_own = res.plan.stats()["voxels"]
            ok.append(bool(torch.equal(res.out, ref)) and res.plan.stats()["error"] == 0 and 1000 < n_own < 5000)
            gathered = shard.sharded_window_attention(coords, qkv, geom, table, case["scale"], case["window"], rank, world,
                                                      bounds)
            ok.append(bool(torch.equal(gathered.out, ref)))
            rows.close()
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sharded_pass_equals_single_gpu():
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    res = [q.get(timeout=10) for _ in range(2)]
    assert all(all(ok) for _, ok in res), res


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_one_process_two_devices_peer_store():
    """One process driving two devices: the second destination is an ordinary tensor on the other
    device, reachable after `ssw_enable_peer_access`."""
    from sparseswin3d_b200 import attention, window
    from sparseswin3d_b200._lib import check, lib
    from tests.cases import make_case

    dev, other = torch.device("cuda:0"), torch.device("cuda:1")
    case = make_case(n_vox=3000, grid=40, shift=(3, 3, 3), seed=8)
    geom = window.resolve_geometry(1, case["dims"], case["window"], case["shift"])
    with torch.cuda.device(dev):
        check(lib.ssw_enable_peer_access(1), "ssw_enable_peer_access")
        for dtype in (torch.float32, torch.bfloat16):
            qkv = case["qkv"].to(dtype).to(dev)
            plan = window.bucket_windows(coords=case["coords"].to(dev), geom=geom, **attention.plan_params(3, 32, dtype))
            twin = torch.zeros(3000, 96, dtype=dtype, device=other)
            torch.cuda.synchronize(other)
            out = attention.window_attention_fused(qkv, plan, case["table"].to(dev), case["scale"], use_mask=True,
                                                   peer_out_ptrs=[twin.data_ptr()])
            torch.cuda.synchronize(dev)
            assert plan.stats()["error"] == 0
            assert torch.equal(twin.cpu(), out.cpu())
