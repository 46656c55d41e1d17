"""CPU: the multi-GPU partitioning logic — window-range cuts and the output gather on two gloo
ranks (no GPU, no native calls)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sparseswin3d_b200 import shard


def test_scene_partition_covers_all():
    for world in (1, 2, 4, 8):
        got = sorted(s for r in range(world) for s in shard.scenes_of_rank(8, r, world))
        assert got == list(range(8))


def test_window_range_cuts_balance_and_cover():
    g = torch.Generator().manual_seed(0)
    counts = torch.cat([torch.randint(1, 9, (3000,), generator=g), torch.full((40,), 729), torch.randint(1, 9, (3000,), generator=g)])
    counts = counts[torch.randperm(counts.numel(), generator=g)]
    cost = shard.window_cost(counts)
    for world in (2, 4, 8):
        cuts = shard.window_range_cuts(counts, world)
        assert cuts[0] == 0 and cuts[-1] == counts.numel() and all(a <= b for a, b in zip(cuts, cuts[1:]))
        per = [float(cost[a:b].sum()) for a, b in zip(cuts, cuts[1:])]
        # no range exceeds its fair share by more than the largest single window
        assert max(per) <= float(cost.sum()) / world + float(cost.max()) + 1e-6
    assert shard.window_range_cuts(counts, 1) == [0, counts.numel()]
    assert shard.window_range_cuts(torch.zeros(0, dtype=torch.int64), 2) == [0, 0, 0]


def test_voxels_of_range():
    perm = torch.tensor([5, 3, 1, 0, 4, 2], dtype=torch.int32)
    win_start = torch.tensor([0, 2, 3, 6], dtype=torch.int32)
    assert shard.voxels_of_range(perm, win_start, 1, 3).tolist() == [1, 0, 4, 2]
    assert shard.voxels_of_range(perm, win_start, 0, 0).numel() == 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        N, C = 11, 4
        full = torch.arange(N * C, dtype=torch.float32).reshape(N, C)
        ids = torch.tensor([0, 3, 4, 9, 10] if rank == 0 else [1, 2, 5, 6, 7, 8])  # ragged shares
        out = shard.gather_rows(full[ids] * 1.0, ids, N)
        q.put((rank, bool(torch.equal(out, full))))
        # a rank with nothing to contribute
        ids2 = torch.arange(N) if rank == 0 else torch.zeros(0, dtype=torch.int64)
        out2 = shard.gather_rows(full[ids2], ids2, N)
        q.put((rank, bool(torch.equal(out2, full))))
    finally:
        dist.destroy_process_group()


def test_gather_rows_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    res = [q.get(timeout=10) for _ in range(4)]
    assert all(ok for _, ok in res)


def test_window_range_cuts_properties_on_random_occupancies():
    """Property test: for any occupancy list and rank count the cuts are monotone, cover every
    window once, and no range exceeds its fair share of the estimated cost by more than one window."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=150, deadline=None)
    @given(st.lists(st.integers(min_value=1, max_value=1023), min_size=0, max_size=400), st.integers(min_value=1, max_value=9),
           st.sampled_from([0.0, 8.0, 32.0, 500.0]))
    def check(occ, world, alpha):
        counts = torch.tensor(occ, dtype=torch.int64)
        cuts = shard.window_range_cuts(counts, world, alpha)
        assert len(cuts) == world + 1 and cuts[0] == 0 and cuts[-1] == len(occ)
        assert all(a <= b for a, b in zip(cuts, cuts[1:]))
        if occ:
            cost = shard.window_cost(counts, alpha)
            per = [float(cost[a:b].sum()) for a, b in zip(cuts, cuts[1:])]
            assert abs(sum(per) - float(cost.sum())) <= 1e-6 * float(cost.sum())
            assert max(per) <= float(cost.sum()) / world + float(cost.max()) + 1e-6

    check()
