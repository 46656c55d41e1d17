"""Multi-GPU partitioning of the attention path.

Windows never interact inside one attention call (the product is block diagonal by construction,
sparse_swin/ops.cu:359-377) and scenes never interact (the batch index is folded into the window
id, sparse_swin/swin3d_base.py:353), so the path shards without any exchange step:

* by scene: `scenes_of_rank` — rank r takes scenes r, r+world, ...;
* by contiguous window range for one huge scene: `window_range_cuts` splits the non-empty windows
  (in window-id order) into `world` contiguous ranges of equal estimated cost, `voxels_of_range`
  selects the voxels of a range, every rank runs bucketing + fused attention on its own voxels, and
  `gather_rows` (the only collective: an all-gather of finished output rows) rebuilds [N, C].

The collective goes through torch.distributed (NCCL on GPUs, gloo in the CPU tests)."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch


def scenes_of_rank(n_scenes: int, rank: int, world: int) -> List[int]:
    return list(range(rank, n_scenes, world))


def window_cost(counts: torch.Tensor, alpha: float = 32.0) -> torch.Tensor:
    """Estimated work of a window with c voxels: c^2 pair evaluations plus alpha * c of per-row
    work (gather, q load, store)."""
    c = counts.to(torch.float64)
    return c * c + alpha * c


def window_range_cuts(counts: torch.Tensor, world: int, alpha: float = 32.0) -> List[int]:
    """Cut points k_0 = 0 <= k_1 <= ... <= k_world = W over the non-empty windows (ascending window
    id) such that every range carries about 1/world of the total cost.  Cuts fall on window
    boundaries only, so no window is split and no halo is needed (the cyclic shift is applied to
    the coordinates before bucketing)."""
    W = counts.numel()
    if world <= 1 or W == 0:
        return [0] + [W] * max(world, 1)
    cum = torch.cumsum(window_cost(counts.cpu(), alpha), 0)
    total = float(cum[-1])
    cuts = [0]
    for r in range(1, world):
        k = int(torch.searchsorted(cum, torch.tensor(total * r / world, dtype=cum.dtype)))
        cuts.append(min(max(k + 1, cuts[-1]), W) if total > 0 else cuts[-1])
    cuts.append(W)
    return cuts


def voxels_of_range(perm: torch.Tensor, win_start: torch.Tensor, k0: int, k1: int) -> torch.Tensor:
    """Voxel ids (int64, for index_select on the caller's tensors) of windows [k0, k1): a
    contiguous slice of the (window, pos)-sorted permutation."""
    a, b = int(win_start[k0]), int(win_start[k1])
    return perm[a:b].to(torch.int64)


def gather_rows(local_rows: torch.Tensor, local_ids: torch.Tensor, n_total: int, group=None) -> torch.Tensor:
    """All-gather finished output rows.  `local_rows` [n_r, C] are this rank's rows, `local_ids`
    [n_r] their voxel ids in the full scene.  Ranks hold different numbers of rows, so both are
    padded to the largest count for the collective.  Returns [n_total, C] on every rank."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    dev = local_rows.device
    n_local = torch.tensor([local_rows.shape[0]], dtype=torch.int64, device=dev)
    counts = [torch.zeros_like(n_local) for _ in range(world)]
    dist.all_gather(counts, n_local, group=group)
    counts = [int(c) for c in counts]
    n_max = max(counts + [1])
    C = local_rows.shape[1]
    rows_pad = torch.zeros((n_max, C), dtype=local_rows.dtype, device=dev)
    ids_pad = torch.zeros(n_max, dtype=torch.int64, device=dev)
    rows_pad[: local_rows.shape[0]] = local_rows
    ids_pad[: local_ids.shape[0]] = local_ids.to(torch.int64)
    all_rows = [torch.empty_like(rows_pad) for _ in range(world)]
    all_ids = [torch.empty_like(ids_pad) for _ in range(world)]
    dist.all_gather(all_rows, rows_pad, group=group)
    dist.all_gather(all_ids, ids_pad, group=group)
    out = torch.empty((n_total, C), dtype=local_rows.dtype, device=dev)
    for r in range(world):
        out.index_copy_(0, all_ids[r][: counts[r]], all_rows[r][: counts[r]])
    return out


def sharded_window_attention(coords: torch.Tensor, qkv: torch.Tensor, geom, table: torch.Tensor, scale: float,
                             rpb_window: Sequence[int], rank: int, world: int, group=None,
                             alpha: float = 32.0, gather: bool = True):
    """One attention pass over a single scene sharded by contiguous window ranges.

    Every rank buckets the whole coordinate set (N int32 keys: cheap, replicated, and it keeps the
    cut points identical everywhere without communication), takes its window range, runs the fused
    kernel on its own voxels' qkv rows and, if `gather`, all-gathers the output rows.
    Returns (out, ids): the full [N, C] output (or this rank's rows) and this rank's voxel ids."""
    from . import attention, window

    H, hd = qkv.shape[2], qkv.shape[3]
    pp = attention.plan_params(H, hd, qkv.dtype, rpb_window)
    full = window.bucket_windows(coords=coords, geom=geom, **pp)
    counts = full.occupancy()
    cuts = window_range_cuts(counts, world, alpha)
    ids = voxels_of_range(full.perm, full.win_start, cuts[rank], cuts[rank + 1])
    if ids.numel():
        sub_coords = coords.index_select(0, ids).contiguous()
        sub_qkv = qkv.index_select(0, ids).contiguous()
        plan = window.bucket_windows(coords=sub_coords, geom=geom, **pp)
        local = attention.window_attention_fused(sub_qkv, plan, table, scale, use_mask=bool(geom.shifted))
    else:
        local = torch.empty((0, H * hd), dtype=qkv.dtype, device=qkv.device)
    if not gather or world == 1:
        return (local if world > 1 or not gather else _place(local, ids, coords.shape[0])), ids
    return gather_rows(local, ids, coords.shape[0], group), ids


def _place(rows: torch.Tensor, ids: torch.Tensor, n_total: int) -> torch.Tensor:
    out = torch.empty((n_total, rows.shape[1]), dtype=rows.dtype, device=rows.device)
    out.index_copy_(0, ids, rows)
    return out
