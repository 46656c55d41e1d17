"""Window geometry and bucketing: the host-side mirror of upstream's ``get_window_size``,
``pad_sparse_tensor``, ``roll_sparse_tensor``, ``window_partition_sparse`` and ``compute_mask``
(sparse_swin/swin3d_base.py:276-300, 336-372, 436-452, 501-554), collapsed into one geometry
record plus one device-side counting sort (``bucket_windows``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import Geometry, PlanLayout, check, lib, ptr, stream_ptr


def resolve_geometry(batch: int, dims: Sequence[int], window: Sequence[int], shift: Sequence[int] = (0, 0, 0)) -> Geometry:
    """Clamp window/shift to the grid (swin3d_base.py:276-300), pad dims up to a window
    multiple (:745-751) and count windows (:345-347, :371)."""
    g = Geometry()
    g.batch = int(batch)
    g.dims[:] = [int(d) for d in dims]
    g.window[:] = [int(w) for w in window]
    g.shift[:] = [int(s) for s in shift]
    check(lib.ssw_geometry_resolve(g), "ssw_geometry_resolve")
    return g


def window_keys(coords: torch.Tensor, geom: Geometry, with_region: bool = False):
    """coords [N,4] int32 (b,z,y,x) -> indices [N,2] int32 (window, pos) exactly as
    window_partition_sparse leaves them after pad + roll(-shift) (swin3d_base.py:749-759);
    optionally also the compute_mask region id of each voxel."""
    _require_cuda_i32(coords, "coords", 4)
    n = coords.shape[0]
    idx = torch.empty((n, 2), dtype=torch.int32, device=coords.device)
    region = torch.empty((n,), dtype=torch.int8, device=coords.device) if with_region else None
    err = torch.zeros(1, dtype=torch.int32, device=coords.device)
    check(lib.ssw_window_keys(ptr(coords), n, geom, ptr(idx), ptr(region), ptr(err), stream_ptr(coords.device)),
          "ssw_window_keys")
    return (idx, region, err) if with_region else (idx, err)


def _require_cuda_i32(t: torch.Tensor, name: str, cols: int):
    if not t.is_cuda:
        raise _lib.SswError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != torch.int32 or t.dim() != 2 or t.shape[1] != cols or not t.is_contiguous():
        raise _lib.SswError(f"{name} must be a contiguous int32 [N,{cols}] tensor")


@dataclass
class WindowPlan:
    """Result of `bucket_windows`: one int32 device array plus typed views into it.  Every view
    has its *capacity* length; the live lengths (non-empty windows W, work items) are device
    values in `header` so that building a plan never synchronises the host."""

    layout: PlanLayout
    plan: torch.Tensor
    rpb_window: tuple
    has_regions: bool

    def _view(self, off: int, n: int) -> torch.Tensor:
        return self.plan[off:off + n]

    @property
    def header(self):
        return self._view(self.layout.off_header, _lib.HEADER_INTS)

    @property
    def perm(self):
        return self._view(self.layout.off_perm, self.layout.n_vox)

    @property
    def inv_perm(self):
        return self._view(self.layout.off_inv_perm, self.layout.n_vox)

    @property
    def win_id(self):
        return self._view(self.layout.off_win_id, self.layout.w_cap)

    @property
    def win_start(self):
        return self._view(self.layout.off_win_start, self.layout.w_cap + 1)

    @property
    def coo_start(self):
        return self._view(self.layout.off_coo_start, self.layout.w_cap + 1)

    @property
    def pack_perm(self):
        return self._view(self.layout.off_pack_perm, self.layout.n_vox)

    @property
    def pack_meta(self):
        return self._view(self.layout.off_pack_meta, self.layout.n_vox)

    @property
    def pack_desc(self):
        return self._view(self.layout.off_pack_desc, 4 * self.layout.pack_cap).view(-1, 4)

    def stats(self) -> dict:
        """Synchronises: reads the header back."""
        h = self.header.cpu().tolist()
        return {"voxels": h[_lib.H_N], "windows": h[_lib.H_W], "work_items": h[_lib.H_PACKS], "error": h[_lib.H_ERROR],
                "c_max": h[_lib.H_CMAX], "sum_c2": (h[_lib.H_SUMC2_HI] << 32) | (h[_lib.H_SUMC2_LO] & 0xFFFFFFFF),
                "tile_rows": h[_lib.H_TILE]}

    def raise_on_error(self):
        """Synchronises.  Upstream silently mis-computes on duplicate or out-of-range voxels;
        this raises instead."""
        e = int(self.header[_lib.H_ERROR])
        if e & _lib.DEV_BAD_COORD:
            raise _lib.SswError("a voxel lies outside the grid / window table")
        if e & _lib.DEV_DUPLICATE:
            raise _lib.SswError("two voxels share (window, pos): coordinates must be unique")
        if e & _lib.DEV_TIMEOUT:
            raise _lib.SswError("device-side wait on an async copy timed out")
        if e & _lib.DEV_BAD_PLAN:
            raise _lib.SswError("an attention kernel was handed an inconsistent plan (stale or overwritten buffer)")

    def occupancy(self) -> torch.Tensor:
        """`_c` of upstream at window granularity (int32 [W]).  Synchronises."""
        w = int(self.header[_lib.H_W])
        s = self.win_start[: w + 1]
        return s[1:] - s[:-1]


def bucket_windows(*, coords: Optional[torch.Tensor] = None, geom: Optional[Geometry] = None,
                   indices: Optional[torch.Tensor] = None, n_windows: Optional[int] = None,
                   n_per_window: Optional[int] = None, mask: Optional[torch.Tensor] = None,
                   rpb_window: Sequence[int] = (7, 7, 7), tile_rows: int = 64, padded: bool = False,
                   scratch: Optional[torch.Tensor] = None, plan_buffer: Optional[torch.Tensor] = None,
                   window_range: Optional[Sequence[int]] = None) -> WindowPlan:
    """Sort voxels by (window, pos) on the device and build the fused kernel's work list.

    Give either ``coords`` [N,4] + ``geom`` (pad, cyclic shift, partition and region ids are
    computed on the fly) or ``indices`` [N,2] + ``n_windows`` + ``n_per_window`` (the tensor and
    sizes upstream's WindowAttentionSparse.forward receives as x.indices, x.batch_size,
    x.spatial_shape[0]) with an optional ``mask`` [nW, n] int8 from compute_mask.

    ``tile_rows`` and ``padded`` shape the fused kernel's work list; take them from
    ``attention.plan_params(heads, head_dim, dtype, window)`` for the tensor the plan will serve.
    ``scratch`` and ``plan_buffer`` (int32 device tensors, reused when large enough) let a caller
    that builds plans repeatedly keep the call free of allocations.

    ``window_range`` = (lo, hi) buckets only the voxels whose window id lies in [lo, hi) - one GPU's
    share of a scene that is split by contiguous window ranges (see ``shard``).  Voxel ids in the plan
    still refer to the full arrays; ``inv_perm`` is defined for the voxels taken only."""
    if (coords is None) == (indices is None):
        raise _lib.SswError("give exactly one of coords= or indices=")
    if coords is not None:
        _require_cuda_i32(coords, "coords", 4)
        if geom is None:
            raise _lib.SswError("coords= needs geom=")
        n_windows, n_per_window, src = geom.n_windows, geom.n_per_window, coords
    else:
        _require_cuda_i32(indices, "indices", 2)
        if n_windows is None or n_per_window is None:
            raise _lib.SswError("indices= needs n_windows= and n_per_window=")
        src = indices
    if mask is not None:
        if coords is not None:
            raise _lib.SswError("mask= is only used with indices=; with coords= regions come from geom")
        if mask.dtype != torch.int8 or mask.dim() != 2 or mask.shape[1] != n_per_window or not mask.is_contiguous() \
                or mask.device != src.device:
            raise _lib.SswError("mask must be a contiguous int8 [nW, n_per_window] tensor on the same device")
    L = PlanLayout()
    check(lib.ssw_plan_layout_init(L, src.shape[0], int(n_windows), int(n_per_window), int(tile_rows), int(bool(padded))),
          "ssw_plan_layout_init")
    dev = src.device
    if plan_buffer is not None and plan_buffer.numel() >= L.plan_ints:
        if plan_buffer.dtype != torch.int32 or plan_buffer.device != dev or not plan_buffer.is_contiguous():
            raise _lib.SswError("plan_buffer must be a contiguous int32 tensor on the same device")
        plan = plan_buffer[: L.plan_ints]
    else:
        plan = torch.empty(L.plan_ints, dtype=torch.int32, device=dev)
    if scratch is None or scratch.numel() < L.scratch_ints:
        scratch = torch.empty(max(L.scratch_ints, 1), dtype=torch.int32, device=dev)
    rw = (_lib.i32 * 3)(*[int(x) for x in rpb_window])
    lo, hi = (0, 0x7FFFFFFF) if window_range is None else (int(window_range[0]), int(window_range[1]))
    check(lib.ssw_bucket_windows_range(ptr(coords), geom, ptr(indices), ptr(mask), 0 if mask is None else mask.shape[0],
                                       rw, L, ptr(plan), ptr(scratch), lo, hi, stream_ptr(dev)), "ssw_bucket_windows")
    has_regions = mask is not None or (coords is not None and bool(geom.shifted))
    return WindowPlan(L, plan, tuple(int(x) for x in rpb_window), has_regions)
