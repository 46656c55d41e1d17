"""Sparse 3-D convolutions over voxel sets: stand-ins for the three spconv layers upstream's model
shell is built from (sparse_swin/swin3d_base.py: `SubMConv3d` :915-923, 1039-1059; `SparseConv3d`
:932-935, 965-970; `SparseInverseConv3d` :989-994) with the constructor arguments upstream passes,
operating on `stage.SparseVoxels` (or any object with `features`, `indices` [N,4] int32 (b,z,y,x),
`spatial_shape`, `batch_size`, `indice_dict`, `replace_feature`).

A convolution is a rulebook (which input voxel feeds which output voxel through which kernel tap,
built once per `indice_key` and kept in `x.indice_dict`), a gathered operand (this library's
kernels) and one dense GEMM (torch).  A submanifold convolution over a sparse neighbourhood takes
the pair form instead: the existing (input, output) pairs grouped by tap, one batched GEMM over the
taps, and a gather-reduce on the output side.  Semantics are those of the dense operation restricted to the
active sites:

* `SubMConv3d(k, padding=k//2)`: output sites = input sites in the same order;
  out[i] = sum_t W[t] x[voxel at coords[i] + offset(t)], absent neighbours contribute nothing.
* `SparseConv3d(k, stride=k)`: output grid = (D - k) // k + 1 per axis; an output cell is active when
  at least one of its k^3 input cells is; active outputs are listed in (b, z, y, x) order.  Input
  voxels beyond k * output grid (an odd last plane) have no output cell, as in the dense operation.
* `SparseInverseConv3d(k, indice_key)`: the transposed operation of the `SparseConv3d` that
  registered `indice_key`: output sites = that convolution's input sites, each fed by its one
  parent cell through the tap it occupies.

Weights are stored as [k^3, Cin, Cout] (tap (dz, dy, dx) at index (dz * k + dy) * k + dx).  spconv is
not available here and upstream pins no version of it, so neither its weight layout nor the order
in which it lists output voxels is reproduced; `weight_from_dense` converts a dense
`[Cout, Cin, k, k, k]` kernel.  With autograd recording the gathers run as torch indexing (which
differentiates); otherwise as this library's kernels."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.nn as nn

from . import _lib, ops
from ._lib import check, dtype_code, lib, ptr, stream_ptr
from .stage import SparseVoxels

I32 = torch.int32
# the pair form of a submanifold convolution is used when its padded pair slots are at most this
# fraction of the dense operand's k^3 N rows
PAIR_FORM_MAX_FILL = 0.5


@dataclass
class Rulebook:
    kind: str                     # "subm" or "strided"
    ksize: int
    in_indices: torch.Tensor      # [N, 4]
    in_shape: list
    out_indices: torch.Tensor     # [M, 4]
    out_shape: list
    nbr: torch.Tensor             # [M, k^3] int32: input voxel per (output voxel, tap), -1 = none
    parent: Optional[torch.Tensor] = None   # strided: [N] output voxel of every input voxel, -1 = none
    tap: Optional[torch.Tensor] = None      # strided: [N] tap through which it feeds its parent
    # subm, pair form (only when the scene is sparse enough for it to pay): the off-centre taps'
    # (input, output) pairs grouped by tap, every tap's run padded to `seg` slots
    seg: int = 0
    pair_in: Optional[torch.Tensor] = None  # [(k^3 - 1) * seg, 1] input voxel of every pair slot, -1 = padding
    row_start: Optional[torch.Tensor] = None   # [N + 1] output i's pair slots are row_slots[row_start[i] : row_start[i + 1]]
    row_slots: Optional[torch.Tensor] = None   # [pairs] in tap order within a row


def _dims3(d: Sequence[int]):
    return (_lib.i32 * 3)(*[int(v) for v in d])


def voxel_grid(indices: torch.Tensor, batch_size: int, spatial_shape: Sequence[int], strict: bool = True) -> torch.Tensor:
    """Dense cell -> voxel id table (int32 [B, D, H, W], -1 = empty)."""
    if not indices.is_cuda or indices.dtype != I32 or indices.dim() != 2 or indices.shape[1] != 4 or not indices.is_contiguous():
        raise _lib.SswError("indices must be a contiguous CUDA int32 [N, 4] tensor (b, z, y, x)")
    D, H, W = (int(v) for v in spatial_shape)
    grid = torch.empty((int(batch_size), D, H, W), dtype=I32, device=indices.device)
    err = torch.zeros(1, dtype=I32, device=indices.device)
    check(lib.ssw_voxel_grid_build(ptr(indices), indices.shape[0], int(batch_size), _dims3((D, H, W)), ptr(grid), ptr(err),
                                   stream_ptr(indices.device)), "ssw_voxel_grid_build")
    if strict and not torch.cuda.is_current_stream_capturing():
        e = int(err)
        if e & _lib.DEV_BAD_COORD:
            raise _lib.SswError("a voxel lies outside the grid")
        if e & _lib.DEV_DUPLICATE:
            raise _lib.SswError("two voxels share a cell: coordinates must be unique")
    return grid


def subm_rulebook(x, ksize: int) -> Rulebook:
    if ksize % 2 != 1:
        raise _lib.SswError("a submanifold convolution needs an odd kernel size")
    grid = voxel_grid(x.indices, x.batch_size, x.spatial_shape)
    n = x.indices.shape[0]
    nbr = torch.empty((n, ksize ** 3), dtype=I32, device=x.indices.device)
    check(lib.ssw_subm_neighbors(ptr(x.indices), n, int(x.batch_size), _dims3(x.spatial_shape), ptr(grid), int(ksize), ptr(nbr),
                                 stream_ptr(x.indices.device)), "ssw_subm_neighbors")
    rb = Rulebook("subm", ksize, x.indices, list(x.spatial_shape), x.indices, list(x.spatial_shape), nbr)
    # Pair form.  On a surface-sparse scene a voxel has a few of its k^3 neighbours, and the gathered
    # operand [N, k^3 Cin] would be mostly zeros.  Group the existing (input, output) pairs by tap
    # instead, pad every off-centre tap's run to the longest one (so that one batched GEMM serves
    # them all) and let the output side pick its pairs up (`ssw_gather_reduce`).  One read-back.
    k3 = ksize ** 3
    if n > 0 and k3 > 1:
        centre = k3 // 2
        off = torch.cat([nbr[:, :centre], nbr[:, centre + 1:]], 1).t().contiguous()   # [k^3 - 1, N], tap-major
        has = off >= 0
        rank = torch.cumsum(has, 1, dtype=torch.int32) - 1                   # position inside its tap's run
        seg = int(rank[:, -1].max()) + 1
        seg = (seg + 7) // 8 * 8
        if 0 < (k3 - 1) * seg <= PAIR_FORM_MAX_FILL * k3 * n:
            taps = torch.arange(k3 - 1, dtype=torch.int32, device=nbr.device).unsqueeze(1)
            slot = taps * seg + rank
            pair_in = torch.full(((k3 - 1) * seg,), -1, dtype=I32, device=nbr.device)
            pair_in[slot[has].long()] = off[has]
            rb.pair_in = pair_in.view(-1, 1)
            # the same pairs seen from the output side: per output row the list of its slots, in tap order
            has_rt = has.t().contiguous()                                     # [N, k^3 - 1]
            rb.row_slots = slot.t()[has_rt].to(I32).contiguous()
            row_start = torch.zeros(n + 1, dtype=I32, device=nbr.device)
            row_start[1:] = torch.cumsum(has_rt.sum(1, dtype=torch.int32), 0, dtype=torch.int32)
            rb.row_start = row_start
            rb.seg = seg
    return rb


def strided_rulebook(x, ksize: int) -> Rulebook:
    """kernel = stride = ksize, no padding.  One host synchronisation (the number of output voxels)."""
    k = int(ksize)
    idx = x.indices
    dev = idx.device
    n = idx.shape[0]
    dims = [int(v) for v in x.spatial_shape]
    od = [(d - k) // k + 1 if d >= k else 0 for d in dims]
    n_cells = int(x.batch_size) * od[0] * od[1] * od[2]
    if n_cells >= 2 ** 31 - 1:
        raise _lib.SswError("the output grid leaves the int32 domain")
    b, z, y, xx = idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]
    valid = (z < od[0] * k) & (y < od[1] * k) & (xx < od[2] * k)
    cell = ((b * od[0] + z // k) * od[1] + y // k) * od[2] + xx // k
    tap = ((z % k) * k + y % k) * k + xx % k
    if n == 0 or n_cells == 0:
        out_idx = torch.zeros((0, 4), dtype=I32, device=dev)
        return Rulebook("strided", k, idx, dims, out_idx, od, torch.zeros((0, k ** 3), dtype=I32, device=dev),
                        torch.full((n,), -1, dtype=I32, device=dev), tap.to(I32))
    # rank of every voxel's output cell among the occupied cells (ascending cell id = (b, z, y, x) order);
    # voxels without an output cell go to one extra bin behind all cells
    keyed = torch.where(valid, cell, torch.full_like(cell, n_cells)).to(I32).contiguous()
    rank, count = ops.return_inverse(keyed, n_cells + 1)
    n_invalid = int((~valid).sum())
    m = count - (1 if n_invalid else 0)
    parent = torch.where(valid, rank, torch.full_like(rank, -1))
    vi = valid.nonzero().squeeze(1)
    cell_of = torch.empty(m, dtype=torch.int64, device=dev)
    cell_of[parent[vi].long()] = cell[vi].long()
    out_idx = torch.stack([cell_of // (od[0] * od[1] * od[2]), (cell_of // (od[1] * od[2])) % od[0], (cell_of // od[2]) % od[1],
                           cell_of % od[2]], 1).to(I32).contiguous()
    nbr = torch.full((m, k ** 3), -1, dtype=I32, device=dev)
    nbr[parent[vi].long(), tap[vi].long()] = vi.to(I32)
    return Rulebook("strided", k, idx, dims, out_idx, od, nbr, parent.to(I32).contiguous(), tap.to(I32).contiguous())


def gather_cols(x: torch.Tensor, nbr: torch.Tensor) -> torch.Tensor:
    """cols[m, t * C + c] = x[nbr[m, t], c], zero where nbr < 0."""
    m, taps = nbr.shape
    c = x.shape[1]
    if torch.is_grad_enabled() and x.requires_grad:
        g = x.index_select(0, nbr.clamp(min=0).reshape(-1).long()) * (nbr.reshape(-1, 1) >= 0).to(x.dtype)
        return g.reshape(m, taps * c)
    x = x.contiguous()
    cols = torch.empty((m, taps * c), dtype=x.dtype, device=x.device)
    check(lib.ssw_gather_cols(ptr(x), dtype_code(x.dtype), x.shape[0], m, taps, c, ptr(nbr), ptr(cols), stream_ptr(x.device)),
          "ssw_gather_cols")
    return cols


def gather_slices(z: torch.Tensor, parent: torch.Tensor, tap: torch.Tensor, taps: int) -> torch.Tensor:
    """out[i] = z[parent[i], tap[i] * C : (tap[i] + 1) * C] with C = z.shape[1] / taps; zero where parent < 0."""
    n = parent.shape[0]
    c = z.shape[1] // taps
    if torch.is_grad_enabled() and z.requires_grad:
        rows = z.reshape(-1, c).index_select(0, (parent.clamp(min=0).long() * taps + tap.long()))
        return rows * (parent.reshape(-1, 1) >= 0).to(z.dtype)
    z = z.contiguous()
    out = torch.empty((n, c), dtype=z.dtype, device=z.device)
    check(lib.ssw_gather_slices(ptr(z), dtype_code(z.dtype), z.shape[0], taps, c, n, ptr(parent), ptr(tap), ptr(out),
                                stream_ptr(z.device)), "ssw_gather_slices")
    return out


def weight_from_dense(w: torch.Tensor) -> torch.Tensor:
    """A dense convolution kernel [Cout, Cin, k, k, k] in this module's [k^3, Cin, Cout] layout."""
    co, ci, k = w.shape[0], w.shape[1], w.shape[2]
    return w.permute(2, 3, 4, 1, 0).reshape(k ** 3, ci, co).contiguous()


def _same3(v) -> int:
    if isinstance(v, (tuple, list)):
        if len(set(int(a) for a in v)) != 1:
            raise ValueError("only cubic kernels and strides are built")
        return int(v[0])
    return int(v)


class _ConvBase(nn.Module):
    def __init__(self, in_channels: int, out_channels: int, kernel_size, bias: bool, indice_key):
        super().__init__()
        self.in_channels, self.out_channels = int(in_channels), int(out_channels)
        self.kernel_size = _same3(kernel_size)
        self.indice_key = indice_key
        k3 = self.kernel_size ** 3
        self.weight = nn.Parameter(torch.empty(k3, self.in_channels, self.out_channels))
        self.bias = nn.Parameter(torch.zeros(self.out_channels)) if bias else None
        nn.init.kaiming_uniform_(self.weight.view(k3 * self.in_channels, self.out_channels).t(), a=math.sqrt(5))
        if self.bias is not None:
            bound = 1.0 / math.sqrt(k3 * self.in_channels)
            nn.init.uniform_(self.bias, -bound, bound)

    def _rulebook(self, x, kind: str, build):
        d = getattr(x, "indice_dict", None)
        if d is None:
            d = x.indice_dict = {}
        rb = d.get(self.indice_key) if self.indice_key is not None else None
        if rb is None or rb.kind != kind or rb.ksize != self.kernel_size or rb.in_indices is not x.indices:
            with torch.no_grad():
                rb = build(x, self.kernel_size)
            if self.indice_key is not None:
                d[self.indice_key] = rb
        return rb

    def _affine(self, cols: torch.Tensor, w2d: torch.Tensor) -> torch.Tensor:
        out = cols @ w2d.to(cols.dtype)
        return out if self.bias is None else out + self.bias.to(out.dtype)


class SubMConv3d(_ConvBase):
    """spconv.SubMConv3d(in_channels, out_channels, kernel_size, stride=1, padding=k//2, bias, indice_key)."""

    def __init__(self, in_channels, out_channels, kernel_size=3, stride=1, padding=None, bias=True, indice_key=None, **unused):
        super().__init__(in_channels, out_channels, kernel_size, bias, indice_key)
        if _same3(stride) != 1:
            raise ValueError("a submanifold convolution has stride 1")
        if padding is not None and _same3(padding) != self.kernel_size // 2:
            raise ValueError("a submanifold convolution pads by kernel_size // 2")

    def forward(self, x):
        rb = self._rulebook(x, "subm", subm_rulebook)
        f = x.features
        pairs_ok = (rb.seg > 0 and not (torch.is_grad_enabled() and (f.requires_grad or self.weight.requires_grad))
                    and (self.out_channels * f.element_size()) % 16 == 0)
        if not pairs_ok:
            cols = gather_cols(f, rb.nbr)
            return x.replace_feature(self._affine(cols, self.weight.reshape(-1, self.out_channels)))
        k3 = self.kernel_size ** 3
        centre = k3 // 2
        w = self.weight.to(f.dtype)
        base = f @ w[centre]                                                 # the voxel itself
        if self.bias is not None:
            base = base + self.bias.to(base.dtype)
        xp = gather_cols(f, rb.pair_in).view(k3 - 1, rb.seg, self.in_channels)
        yp = torch.bmm(xp, torch.cat([w[:centre], w[centre + 1:]], 0)).view(-1, self.out_channels)
        out = torch.empty_like(base)
        check(lib.ssw_gather_reduce(ptr(base), ptr(yp), dtype_code(f.dtype), yp.shape[0], ptr(rb.row_start), ptr(rb.row_slots),
                                    rb.row_slots.shape[0], f.shape[0], self.out_channels, ptr(out), stream_ptr(f.device)),
              "ssw_gather_reduce")
        return x.replace_feature(out)


class SparseConv3d(_ConvBase):
    """spconv.SparseConv3d(in_channels, out_channels, kernel_size, stride, bias, indice_key) with
    stride = kernel_size and no padding (patch embedding and patch merging)."""

    def __init__(self, in_channels, out_channels, kernel_size=2, stride=None, padding=0, bias=True, indice_key=None, **unused):
        super().__init__(in_channels, out_channels, kernel_size, bias, indice_key)
        if stride is not None and _same3(stride) != self.kernel_size:
            raise ValueError("only stride = kernel_size is built")
        if _same3(padding) != 0:
            raise ValueError("only padding 0 is built")

    def forward(self, x):
        rb = self._rulebook(x, "strided", strided_rulebook)
        cols = gather_cols(x.features, rb.nbr)
        out = self._affine(cols, self.weight.reshape(-1, self.out_channels))
        y = SparseVoxels(out, rb.out_indices, rb.out_shape, x.batch_size)
        y.indice_dict = x.indice_dict
        return y


class SparseInverseConv3d(_ConvBase):
    """spconv.SparseInverseConv3d(in_channels, out_channels, kernel_size, indice_key, bias): undoes the
    geometry of the SparseConv3d that registered `indice_key` on this tensor's ancestors."""

    def __init__(self, in_channels, out_channels, kernel_size=2, indice_key=None, bias=True, **unused):
        super().__init__(in_channels, out_channels, kernel_size, bias, indice_key)

    def forward(self, x):
        rb = getattr(x, "indice_dict", {}).get(self.indice_key)
        if rb is None or rb.kind != "strided" or rb.ksize != self.kernel_size:
            raise _lib.SswError(f"no strided convolution has registered indice_key {self.indice_key!r} on this tensor")
        if rb.out_indices.shape[0] != x.features.shape[0]:
            raise _lib.SswError("this tensor does not live on the output sites of that convolution")
        k3 = self.kernel_size ** 3
        # all taps of every coarse voxel in one GEMM: z[m, t * Cout + o] = sum_c y[m, c] W[t, c, o]
        w2d = self.weight.permute(1, 0, 2).reshape(self.in_channels, k3 * self.out_channels)
        z = x.features @ w2d.to(x.features.dtype)
        out = gather_slices(z, rb.parent, rb.tap, k3)
        if self.bias is not None:
            out = out + self.bias.to(out.dtype)
        y = SparseVoxels(out, rb.in_indices, rb.in_shape, x.batch_size)
        y.indice_dict = x.indice_dict
        return y


class SparseModule(nn.Module):
    """Marker base class (spconv.SparseModule)."""


class SparseSequential(nn.Sequential):
    """spconv.SparseSequential: modules that take the voxel container get it; plain feature modules
    (normalisations, activations) are applied to `features`."""

    def forward(self, x):
        for m in self:
            if isinstance(m, (SparseModule, _ConvBase, SparseSequential)) or hasattr(m, "forward_voxels"):
                x = m(x)
            else:
                x = x.replace_feature(m(x.features))
        return x


class PatchMerging(SparseModule):
    """LayerNorm then a 2x2x2 stride-2 convolution doubling the channels (swin3d_base.py:950-976)."""

    def __init__(self, dim: int, norm_layer=nn.LayerNorm, spatial_dims: int = 3, indice_key=None):
        super().__init__()
        self.dim = dim
        self.reduction = SparseConv3d(dim, 2 * dim, kernel_size=2, stride=2, bias=False, indice_key=indice_key)
        self.norm = norm_layer(dim)

    def forward(self, x):
        return self.reduction(x.replace_feature(self.norm(x.features)))


class PatchExpand(SparseModule):
    """The inverse 2x2x2 convolution halving the channels, then LayerNorm (swin3d_base.py:979-1004)."""

    def __init__(self, dim: int, norm_layer=nn.LayerNorm, spatial_dims: int = 3, indice_key=None):
        super().__init__()
        self.expansion = SparseInverseConv3d(dim, dim // 2, kernel_size=2, bias=False, indice_key=indice_key)
        self.norm = norm_layer(dim // 2)

    def forward(self, x):
        y = self.expansion(x)
        return y.replace_feature(self.norm(y.features))
