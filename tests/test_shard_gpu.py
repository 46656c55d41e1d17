"""Window-range sharding on real GPUs (needs 2): the sharded pass equals the single-GPU pass."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    import torch.distributed as dist

    from sparseswin3d_b200 import attention, shard, window
    from tests.cases import make_case

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        case = make_case(n_vox=6000, grid=48, shift=(3, 3, 3), seed=41)
        geom = window.resolve_geometry(1, case["dims"], case["window"], case["shift"])
        coords, qkv, table = case["coords"].to(dev), case["qkv"].to(dev), case["table"].to(dev)
        out, ids = shard.sharded_window_attention(coords, qkv, geom, table, case["scale"], case["window"], rank, world)
        plan = window.bucket_windows(coords=coords, geom=geom, **attention.plan_params(3, 32, torch.float32, case["window"]))
        ref = attention.window_attention_fused(qkv, plan, table, case["scale"], use_mask=True)
        torch.cuda.synchronize()
        q.put((rank, bool(torch.equal(out, ref)), int(ids.numel())))
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
    assert all(ok for _, ok, _ in res)
    assert sum(n for _, _, n in res) == 6000 and min(n for _, _, n in res) > 1000
