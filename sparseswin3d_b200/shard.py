"""Multi-GPU partitioning of the attention path.

Windows never interact inside one attention call (the product is block diagonal by construction,
sparse_swin/ops.cu:359-377) and scenes never interact (the batch index is folded into the window
id, sparse_swin/swin3d_base.py:353), so the path shards without any exchange step on its inputs:

* by scene: `scenes_of_rank` - rank r takes scenes r, r+world, ...;
* by contiguous window range for one huge scene.  `plan_window_ranges` looks at the scene once (one
  bucketing, one read-back) and cuts the dense window-id axis into `world` ranges of equal estimated
  cost.  After that a pass needs no host synchronisation: every rank buckets the coordinates
  restricted to its range (`bucket_windows(window_range=...)`: the N int32 keys are read by every
  rank, only its own are sorted), runs the fused kernels on its windows, and the kernels store every
  finished output row into the [N, C] buffer of EVERY rank (`PeerRows`: the same buffer mapped
  across processes with CUDA IPC, plain stores over NVLink).  A barrier ends the pass; there is no
  gather.  `gather_rows` is the collective alternative (an NCCL / gloo all-gather of finished rows)
  for callers that cannot map peer memory.

No TMA access to peer memory and no multicast is used: peer memory is only ever the target of
ordinary stores issued by this library's own kernels."""
from __future__ import annotations

from dataclasses import dataclass
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


def plan_window_ranges(coords: torch.Tensor, geom, world: int, alpha: float = 32.0, **plan_params) -> List[int]:
    """Boundaries in DENSE window-id space, [b_0 = 0, b_1, ..., b_world = geom.n_windows]: rank r
    works on the windows with ids in [b_r, b_{r+1}).  Looks at the scene once (one bucketing and one
    read-back of the occupancies) - call it when the coordinates change, not per pass.  Every rank
    computes the same boundaries from the same coordinates, so nothing is communicated."""
    from . import window

    full = window.bucket_windows(coords=coords, geom=geom, **plan_params)
    counts = full.occupancy().cpu()
    win_id = full.win_id[: counts.numel()].cpu()
    cuts = window_range_cuts(counts, world, alpha)
    bounds = [0]
    for k in cuts[1:-1]:
        bounds.append(int(win_id[k]) if k < win_id.numel() else int(geom.n_windows))
    bounds.append(int(geom.n_windows))
    return bounds


class _DeviceBytes:
    """Lets torch view raw device memory (no copy, no ownership) through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class PeerRows:
    """An [N, C] output buffer that exists on every rank and that the kernels of every rank can
    store to.  Each rank allocates its own (`ssw_peer_buffer_create`), the CUDA IPC handles go round
    once through the process group, and every rank maps the others' buffers into the context of ITS
    OWN device (`ssw_peer_buffer_open`) - the device whose kernels will store to them.  (A mapping
    made under the owner's device index, as `torch.multiprocessing`'s tensor rebuilding does, is
    not reachable from kernels of this rank's device: they fault.)  `local` is this rank's buffer as
    a tensor; `ptrs` are the device addresses of the peers' buffers, for
    `window_attention_fused(..., out=local, peer_out_ptrs=ptrs)`.  Peer memory is only ever the
    target of plain stores from this library's kernels; nothing else is given these addresses.

    Call `close()` on every rank (it is collective) before the process group goes away."""

    def __init__(self, n: int, c: int, dtype: torch.dtype, device: torch.device, group=None):
        import ctypes

        import torch.distributed as dist

        from ._lib import check, lib

        self.group = group
        self.ptrs: List[int] = []
        self._own = ctypes.c_void_p()
        self._multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        nbytes = max(n * c * torch.empty((), dtype=dtype).element_size(), 16)
        handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(device):
            check(lib.ssw_peer_buffer_create(nbytes, ctypes.byref(self._own), handle), "ssw_peer_buffer_create")
            self.local = torch.as_tensor(_DeviceBytes(self._own.value, nbytes), device=device)[: n * c *
                                         torch.empty((), dtype=dtype).element_size()].view(dtype).view(n, c)
            if not self._multi:
                return
            world, rank = dist.get_world_size(group), dist.get_rank(group)
            handles: list = [None] * world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            for r, h in enumerate(handles):
                if r == rank:
                    continue
                p = ctypes.c_void_p()
                check(lib.ssw_peer_buffer_open(h, ctypes.byref(p)), "ssw_peer_buffer_open")
                self.ptrs.append(p.value)
        dist.barrier(group=group)       # nobody stores before everyone has mapped

    def close(self):
        """Collective: every rank unmaps its peers' buffers, then every rank frees its own."""
        from ._lib import check, lib

        if self._own.value is None:
            return
        torch.cuda.synchronize(self.local.device)
        with torch.cuda.device(self.local.device):
            if self._multi:
                import torch.distributed as dist

                dist.barrier(group=self.group)      # no kernel of any rank still stores
                for p in self.ptrs:
                    check(lib.ssw_peer_buffer_close(p), "ssw_peer_buffer_close")
                self.ptrs = []
                dist.barrier(group=self.group)      # every mapping is gone before an owner frees
            check(lib.ssw_peer_buffer_destroy(self._own), "ssw_peer_buffer_destroy")
        self._own.value = None
        self.local = None


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


@dataclass
class ShardedPass:
    """What `sharded_window_attention` leaves behind: this rank's plan, the buffer that holds the
    complete output once the closing collective has passed, and `error` - a one-element int32 device
    tensor, non-zero when ANY rank's plan or kernels recorded an error bit (the closing collective
    carries it, so no rank has to be asked)."""
    plan: object
    out: torch.Tensor
    error: Optional[torch.Tensor] = None


def sharded_window_attention(coords: torch.Tensor, qkv: torch.Tensor, geom, table: torch.Tensor, scale: float,
                             rpb_window: Sequence[int], rank: int, world: int, bounds: Sequence[int],
                             rows: Optional[PeerRows] = None, group=None, scratch: Optional[torch.Tensor] = None,
                             plan_buffer: Optional[torch.Tensor] = None) -> ShardedPass:
    """One attention pass over a single scene sharded by contiguous window ranges.

    `bounds` come from `plan_window_ranges` (once per scene).  With `rows` (a `PeerRows`) the
    kernels store each finished row on every rank, and the pass ends with a one-word all-reduce on
    the stream (the maximum of the ranks' error words): it orders every rank's stores before
    whatever the caller enqueues next and costs no host synchronisation; `rows.local` is then the
    full [N, C] output.  A caller whose consumer of one pass may still run while the next pass
    stores should alternate two `PeerRows`.  Without `rows` the finished rows are all-gathered with
    `gather_rows` (which reads the row counts back: one host synchronisation)."""
    from . import _lib, attention, window

    H, hd = qkv.shape[2], qkv.shape[3]
    pp = attention.plan_params(H, hd, qkv.dtype, rpb_window)
    plan = window.bucket_windows(coords=coords, geom=geom, scratch=scratch, plan_buffer=plan_buffer,
                                 window_range=(bounds[rank], bounds[rank + 1]), **pp)
    if rows is not None:
        attention.window_attention_fused(qkv, plan, table, scale, use_mask=bool(geom.shifted), out=rows.local,
                                         peer_out_ptrs=rows.ptrs)
        error = plan.header[_lib.H_ERROR:_lib.H_ERROR + 1].clone()
        if world > 1:
            import torch.distributed as dist

            dist.all_reduce(error, op=dist.ReduceOp.MAX, group=group)
        return ShardedPass(plan, rows.local, error)
    out = torch.empty((coords.shape[0], H * hd), dtype=qkv.dtype, device=qkv.device)
    attention.window_attention_fused(qkv, plan, table, scale, use_mask=bool(geom.shifted), out=out)
    if world == 1:
        return ShardedPass(plan, out, plan.header[_lib.H_ERROR:_lib.H_ERROR + 1].clone())
    n_own = int(plan.header[_lib.H_N])
    ids = plan.perm[:n_own].to(torch.int64)
    return ShardedPass(plan, gather_rows(out.index_select(0, ids), ids, coords.shape[0], group))
