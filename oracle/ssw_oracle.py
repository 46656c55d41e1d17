"""CPU restatement of SparseSwin3D's sparse window-attention path.  TEST INFRASTRUCTURE ONLY.

This module is the *checker*, never the product: only the test-suite, the smoke test and the
benchmark's CPU-baseline / reference legs may import it.  It restates, with plain PyTorch CPU
ops (multi-threaded, so it doubles as "the reference's PyTorch CPU path" when timed), what the
upstream project computes with CUDA-only code.  Every function cites the upstream lines it
follows (paths relative to the upstream repository root).

Parity status: the upstream project has no tests, golden vectors or CPU path.  The restatement
is pinned by fixtures under ``tests/golden/`` that were produced by running the *unmodified*
upstream extension (``oracle/_ref/custom_ops.so``, built by ``oracle/build_ref.py``) on a B200
with seeded inputs inside the upstream validity domain (``B_w*H*n*hd < 2**31``); the script
that generated them, ``tests/golden/make_golden.py``, is committed next to them.

Conventions kept from upstream:
  * all index tensors are int32, and index arithmetic wraps like int32 (ops.cu:264-268);
  * a "sparse tensor" is (indices[4, nnz] int32, values[nnz], shape list[4])
    (swin3d_base.py:29-65);
  * softmax quirks: row maximum starts from 0 (ops.cu:137), the denominator gets +1e-8
    (ops.cu:164), the shift mask adds -100 (swin3d_base.py:578).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

I32 = torch.int32


# --------------------------------------------------------------------------------------------
# containers
# --------------------------------------------------------------------------------------------
@dataclass
class SparseTensor:
    """swin3d_base.py:29-65 (container only; `permute` below)."""

    indices: torch.Tensor  # [4, nnz] int32
    values: torch.Tensor  # [nnz]
    shape: List[int]

    def __mul__(self, other):  # swin3d_base.py:61-65
        return SparseTensor(self.indices, self.values * other, self.shape)

    def permute(self, dims):  # swin3d_base.py:47-59
        shape = [self.shape[d] for d in dims]
        idx = self.indices[list(dims), :].contiguous()
        order = sort_indices(flatten_indices(idx, shape))
        return SparseTensor(idx.index_select(1, order), self.values.index_select(0, order), shape)


def _wrap_i32(x: torch.Tensor) -> torch.Tensor:
    """int64 -> int32 with two's-complement wrap, the arithmetic of ops.cu:264-268."""
    return ((x + 2**31) % 2**32 - 2**31).to(I32)


# --------------------------------------------------------------------------------------------
# window geometry (swin3d_base.py:276-300, 336-372, 436-452, 501-554, 741-759)
# --------------------------------------------------------------------------------------------
def get_window_size(x_size, window_size, shift_size=None):
    """swin3d_base.py:276-300: clamp the window (and drop the shift) on axes that fit in it."""
    ws = list(window_size)
    ss = list(shift_size) if shift_size is not None else None
    for i in range(len(x_size)):
        if x_size[i] <= window_size[i]:
            ws[i] = x_size[i]
            if ss is not None:
                ss[i] = 0
    return tuple(ws) if ss is None else (tuple(ws), tuple(ss))


def resolve_geometry(dims, window_size, shift_size):
    """Pad-right amounts and padded dims as in SwinTransformerBlock.forward_part1
    (swin3d_base.py:743-751)."""
    ws, ss = get_window_size(tuple(dims), tuple(window_size), tuple(shift_size))
    dims_p = tuple(d + (w - d % w) % w for d, w in zip(dims, ws))
    return ws, ss, dims_p


def window_keys(coords: torch.Tensor, batch: int, dims, window_size, shift_size):
    """pad -> cyclic roll by -shift -> window partition.

    coords [N,4] int32 (b,z,y,x).  Returns (indices [N,2] int32 = (window,pos), B_w, n, ws, ss, dims_p).
    pad_sparse_tensor only grows the shape (swin3d_base.py:514-526, pads are right-side only at
    :745-748); roll is ``(idx + shift) % dim`` with shift = -s (swin3d_base.py:551,754);
    partition is swin3d_base.py:351-371.
    """
    ws, ss, dp = resolve_geometry(dims, window_size, shift_size)
    c = coords.to(torch.int64)
    z, y, x = c[:, 1], c[:, 2], c[:, 3]
    if any(s > 0 for s in ss):
        z = (z - ss[0]) % dp[0]
        y = (y - ss[1]) % dp[1]
        x = (x - ss[2]) % dp[2]
    nd, nh, nw = dp[0] // ws[0], dp[1] // ws[1], dp[2] // ws[2]
    win = c[:, 0] * nd * nh * nw + (z // ws[0]) * nh * nw + (y // ws[1]) * nw + (x // ws[2])
    pos = (z % ws[0]) * ws[1] * ws[2] + (y % ws[1]) * ws[2] + (x % ws[2])
    idx = torch.stack([_wrap_i32(win), _wrap_i32(pos)], dim=1).contiguous()
    return idx, batch * nd * nh * nw, ws[0] * ws[1] * ws[2], ws, ss, dp


def window_partition_dense(x: torch.Tensor, ws) -> torch.Tensor:
    """swin3d_base.py:416-433 (dense [b,d,h,w,c] -> [windows, n, c])."""
    b, d, h, w, c = x.shape
    x = x.view(b, d // ws[0], ws[0], h // ws[1], ws[1], w // ws[2], ws[2], c)
    return x.permute(0, 1, 3, 5, 2, 4, 6, 7).contiguous().view(-1, ws[0] * ws[1] * ws[2], c)


def compute_mask(dims_p, ws, ss) -> torch.Tensor:
    """swin3d_base.py:436-452: region id per cell of the padded grid, as [nW, n] int8.
    Follows the slice loops literally, including the ``slice(-0, None)`` behaviour on an
    axis whose shift is 0."""
    d, h, w = dims_p
    img = torch.zeros((1, d, h, w, 1), dtype=torch.int8)
    cnt = 0
    for sd in (slice(-ws[0]), slice(-ws[0], -ss[0]), slice(-ss[0], None)):
        for sh in (slice(-ws[1]), slice(-ws[1], -ss[1]), slice(-ss[1], None)):
            for sw in (slice(-ws[2]), slice(-ws[2], -ss[2]), slice(-ss[2], None)):
                img[:, sd, sh, sw, :] = cnt
                cnt += 1
    return window_partition_dense(img, ws).squeeze(-1)


def region_ids_closed_form(coords_shifted_zyx: torch.Tensor, dims_p, ws, ss) -> torch.Tensor:
    """Closed form of `compute_mask` evaluated at shifted-frame cells [N,3] (z,y,x):
    per axis r = 2 if s == 0 else (0 if p < Dp-ws else 1 if p < Dp-s else 2); id = 9 r_z + 3 r_y + r_x."""
    out = torch.zeros(coords_shifted_zyx.shape[0], dtype=torch.int64)
    for a, mul in zip(range(3), (9, 3, 1)):
        p = coords_shifted_zyx[:, a].to(torch.int64)
        if ss[a] == 0:
            r = torch.full_like(p, 2)
        else:
            r = (p >= dims_p[a] - ws[a]).to(torch.int64) + (p >= dims_p[a] - ss[a]).to(torch.int64)
        out += mul * r
    return out.to(torch.int8)


# --------------------------------------------------------------------------------------------
# the ten exported ops (sparse_swin/ops.cpp:7-18)
# --------------------------------------------------------------------------------------------
def flatten_indices(indices: torch.Tensor, sizes: Sequence[int]) -> torch.Tensor:
    """ops.cu:232-273: row-major hash with strides = products of the trailing sizes; sizes[0]
    is never used; the sum is accumulated in int32 and wraps."""
    D = len(sizes)
    assert indices.shape[0] == D
    strides = [1] * D
    for i in range(D - 2, -1, -1):
        strides[i] = strides[i + 1] * int(sizes[i + 1])
    strides = [int(_wrap_i32(torch.tensor(s))) for s in strides]  # strides are int32 too (ops.cu:237-245)
    acc = torch.zeros(indices.shape[1], dtype=torch.int64)
    for i in range(D):
        acc = _wrap_i32(acc + indices[i].to(torch.int64) * strides[i]).to(torch.int64)
    return acc.to(I32)


def sort_indices(flat: torch.Tensor) -> torch.Tensor:
    """ops.cu:276-289: argsort of int32 keys (thrust sort_by_key over a 0..n-1 sequence)."""
    return torch.sort(flat.to(torch.int64), stable=True)[1].to(I32)


def return_inverse(x: torch.Tensor, maxnum: int = -1) -> Tuple[torch.Tensor, int]:
    """ops.cu:718-730: rank of every element among the distinct values present; count."""
    if maxnum == -1:
        maxnum = int(x.max()) + 1
    present = torch.zeros(maxnum, dtype=torch.bool)
    present[x.to(torch.int64)] = True
    c = int(present.sum())
    rank = torch.empty(maxnum, dtype=I32)
    rank[present.nonzero().squeeze(1)] = torch.arange(c, dtype=I32)
    return rank.index_select(0, x.to(torch.int64)), c


def unique_consecutive_indices(nums: torch.Tensor) -> torch.Tensor:
    """ops.cu:32-103: inverse of unique_consecutive = inclusive scan of (x[i] != x[i-1])."""
    if nums.numel() == 0:
        return torch.zeros(0, dtype=I32)
    d = torch.zeros_like(nums, dtype=torch.int64)
    d[1:] = (nums[1:] != nums[:-1]).to(torch.int64)
    return torch.cumsum(d, 0).to(I32)


def qkv_sparse_indices(indices: torch.Tensor, batch_size: int, spatial_dim: int, num_heads: int, c: int):
    """ops.cu:206-227, 293-335.  indices [N,2] int32 (window,pos) -> (idx_qv[4,N*H*c],
    perm_qv, idx_k[4,N*H*c], perm_k).  Index blocks are UNSORTED, in (voxel, head, channel)
    order; q/v rows are (window, head, pos, ch); k rows are (window, head, ch, pos)."""
    N = indices.shape[0]
    win = indices[:, 0].repeat_interleave(num_heads * c)
    pos = indices[:, 1].repeat_interleave(num_heads * c)
    head = torch.arange(num_heads, dtype=I32).repeat_interleave(c).repeat(N)
    ch = torch.arange(c, dtype=I32).repeat(N * num_heads)
    idx_qv = torch.stack([win, head, pos, ch]).contiguous()
    idx_k = torch.stack([win, head, ch, pos]).contiguous()
    perm_qv = sort_indices(flatten_indices(idx_qv, [batch_size, num_heads, spatial_dim, c]))
    perm_k = sort_indices(flatten_indices(idx_k, [batch_size, num_heads, c, spatial_dim]))
    return idx_qv, perm_qv, idx_k, perm_k


def _excl_cumsum(x: torch.Tensor) -> torch.Tensor:
    out = torch.zeros_like(x)
    out[1:] = torch.cumsum(x[:-1], 0)
    return out


def _blocked(vals: torch.Tensor, starts: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """Gather `len(starts)` row-major [rows, cols] blocks beginning at `starts` into [nb, rows, cols]."""
    ar = torch.arange(rows * cols, dtype=torch.int64)
    return vals[(starts[:, None] + ar[None, :]).reshape(-1)].reshape(-1, rows, cols)


def _scatter_blocks(out: torch.Tensor, blocks: torch.Tensor, starts: torch.Tensor):
    nb, r, c = blocks.shape
    ar = torch.arange(r * c, dtype=torch.int64)
    out[(starts[:, None] + ar[None, :]).reshape(-1)] = blocks.reshape(-1)


def _bincount_nonzero(a: torch.Tensor) -> torch.Tensor:
    """ops.cu:781-784."""
    y = torch.bincount(a.to(torch.int64))
    return y[y.nonzero().squeeze(1)].to(torch.int64)


def matmul_cuda_naive(mat1_v, mat1_idx, mat1_shape, mat2_v, mat2_idx, mat2_shape, mul_type: str):
    """ops.cu:1034-1088 -> 788-943 (+ reshape_sparse 732-779, csr2csc transpose 560-660,
    kernels 344-418).  Returns (idx[4,nnz3] int32, vals[nnz3], shape, _c[int32])."""
    if mul_type not in ("q_k", "qk_v"):
        raise RuntimeError(f"Invalid mul_type: {mul_type}. Expected 'q_k' or 'qk_v'.")
    if mat1_v.dtype != mat2_v.dtype:
        raise RuntimeError("mat1 dtype does not match mat2 dtype")
    if not (len(mat1_shape) == 4 and len(mat2_shape) == 4 and mat1_shape[0] == mat2_shape[0]
            and mat1_shape[1] == mat2_shape[1] and mat1_shape[3] == mat2_shape[2]):
        raise RuntimeError("Invalid shapes")
    x2, x3a, x4a = mat1_shape[1], mat1_shape[2], mat1_shape[3]
    x3b, x4b = mat2_shape[2], mat2_shape[3]
    i1 = mat1_idx.to(torch.int64)
    i2 = mat2_idx.to(torch.int64)
    row1 = i1[0] * x2 * x3a + i1[1] * x3a + i1[2]  # ops.cu:762
    col1 = i1[0] * x2 * x4a + i1[1] * x4a + i1[3]  # ops.cu:764
    row2 = i2[0] * x2 * x3b + i2[1] * x3b + i2[2]
    col2 = i2[0] * x2 * x4b + i2[1] * x4b + i2[3]
    # csr2csc of the RHS (ops.cu:804-829): values re-ordered by (col, row), rows already ascending.
    m2t = mat2_v[torch.sort(col2, stable=True)[1]]
    key_rows = torch.unique_consecutive(row1)  # ops.cu:813
    acc_t = torch.float32 if mat1_v.dtype in (torch.float16, torch.bfloat16) else mat1_v.dtype
    if mul_type == "q_k":
        C = mat1_shape[3]
        c = _bincount_nonzero(col1.reshape(-1, C)[:, 0])  # ops.cu:836
        key_cols = key_rows
        idx_starts = _excl_cumsum(c)
        out_starts = _excl_cumsum(c * c)
        mat_starts = _excl_cumsum(c * C)
        total = int((c * c).sum())
        out = torch.empty(total, dtype=mat1_v.dtype)
        row_c = torch.empty(total, dtype=torch.int64)
        col_c = torch.empty(total, dtype=torch.int64)
        for cv in torch.unique(c).tolist():
            sel = (c == cv).nonzero().squeeze(1)
            A = _blocked(mat1_v, mat_starts[sel], cv, C).to(acc_t)
            B = _blocked(m2t, mat_starts[sel], cv, C).to(acc_t)
            _scatter_blocks(out, torch.bmm(A, B.transpose(1, 2)).to(mat1_v.dtype), out_starts[sel])
            ii = torch.arange(cv).repeat_interleave(cv)[None, :] + idx_starts[sel][:, None]
            jj = torch.arange(cv).repeat(cv)[None, :] + idx_starts[sel][:, None]
            _scatter_blocks(row_c, ii.reshape(-1, cv, cv), out_starts[sel])
            _scatter_blocks(col_c, jj.reshape(-1, cv, cv), out_starts[sel])
    else:
        C = mat2_shape[3]
        c = _bincount_nonzero(col2.reshape(-1, C)[:, 0])  # ops.cu:870
        key_cols = torch.unique(col2)  # ops.cu:818
        idx_starts = _excl_cumsum(c)
        out_starts = _excl_cumsum(c * C)
        m1_starts = _excl_cumsum(c * c)
        m2_starts = _excl_cumsum(c * C)
        total = int((c * C).sum())
        out = torch.empty(total, dtype=mat1_v.dtype)
        row_c = torch.empty(total, dtype=torch.int64)
        col_c = torch.empty(total, dtype=torch.int64)
        blk = torch.arange(c.numel(), dtype=torch.int64)
        for cv in torch.unique(c).tolist():
            sel = (c == cv).nonzero().squeeze(1)
            A = _blocked(mat1_v, m1_starts[sel], cv, cv).to(acc_t)  # [nb, c, c]
            Bt = _blocked(m2t, m2_starts[sel], C, cv).to(acc_t)  # [nb, C, c]
            _scatter_blocks(out, torch.bmm(A, Bt.transpose(1, 2)).to(mat1_v.dtype), out_starts[sel])
            ii = torch.arange(cv).repeat_interleave(C)[None, :] + idx_starts[sel][:, None]
            jj = torch.arange(C).repeat(cv)[None, :] + (blk[sel] * C)[:, None]
            _scatter_blocks(row_c, ii.reshape(-1, cv, C), out_starts[sel])
            _scatter_blocks(col_c, jj.reshape(-1, cv, C), out_starts[sel])
    rows = key_rows[row_c]  # ops.cu:909-912
    cols = key_cols[col_c]
    x3, x4 = mat1_shape[2], mat2_shape[3]
    rem = rows % (x2 * x3)
    idx = torch.stack([rows // (x2 * x3), rem // x3, rem % x3, cols % x4]).to(I32)  # ops.cu:930-940
    return idx, out, [mat1_shape[0], x2, x3, x4], c.to(I32)


def _starts(c: torch.Tensor, m: torch.Tensor) -> torch.Tensor:
    return _excl_cumsum(c.to(torch.int64) * m)


def matmul_grad_cuda_naive(mat1_v, mat2_v, _c, C: int, mul_type: str) -> torch.Tensor:
    """ops.cu:945-1031 with kernels 422-515.  Blocks are keyed by `_c` only."""
    c = _c.to(torch.int64)
    acc_t = torch.float32 if mat1_v.dtype in (torch.float16, torch.bfloat16) else mat1_v.dtype
    if mul_type == "rc_cr":  # out[c,c] = m1[c,C] . m2[c,C]^T
        so, s1, s2 = _starts(c, c), _starts(c, torch.tensor(C)), _starts(c, torch.tensor(C))
        shp = lambda cv: ((cv, C), (cv, C), (cv, cv))
        total = int((c * c).sum())
    elif mul_type == "rr_rc":  # out[c,C] = m1[c,c] . m2[C,c]^T
        so, s1, s2 = _starts(c, torch.tensor(C)), _starts(c, c), _starts(c, torch.tensor(C))
        shp = lambda cv: ((cv, cv), (C, cv), (cv, C))
        total = int((c * C).sum())
    elif mul_type == "cr_rr":  # out[C,c] = m1[C,c] . m2[c,c]^T
        so, s1, s2 = _starts(c, torch.tensor(C)), _starts(c, torch.tensor(C)), _starts(c, c)
        shp = lambda cv: ((C, cv), (cv, cv), (C, cv))
        total = int((c * C).sum())
    else:
        raise RuntimeError(f"Invalid mul_type: {mul_type}. Expected 'rc_cr', 'rr_rc' or 'cr_rr'.")
    out = torch.empty(total, dtype=mat1_v.dtype)
    for cv in torch.unique(c).tolist():
        sel = (c == cv).nonzero().squeeze(1)
        (r1, k1), (r2, k2), (ro, co) = shp(cv)
        A = _blocked(mat1_v, s1[sel], r1, k1).to(acc_t)
        B = _blocked(mat2_v, s2[sel], r2, k2).to(acc_t)
        _scatter_blocks(out, torch.bmm(A, B.transpose(1, 2)).to(mat1_v.dtype), so[sel])
    return out


def qkv_transpose(mat1_v, _c, C: int, mul_type: str) -> torch.Tensor:
    """ops.cu:663-715 with kernels 518-557: per block, [c,C] -> [C,c] ("rc") or [c,c]^T ("rr")."""
    c = _c.to(torch.int64)
    out = torch.empty_like(mat1_v)
    if mul_type == "rc":
        st = _starts(c, torch.tensor(C))
    elif mul_type == "rr":
        st = _starts(c, c)
    else:
        raise RuntimeError(f"Invalid mul_type: {mul_type}. Expected 'rc', or 'rr'.")
    for cv in torch.unique(c).tolist():
        sel = (c == cv).nonzero().squeeze(1)
        cols = C if mul_type == "rc" else cv
        A = _blocked(mat1_v, st[sel], cv, cols)
        _scatter_blocks(out, A.transpose(1, 2).contiguous(), st[sel])
    return out


def softmax_last_dim_forward(row_ids: torch.Tensor, values: torch.Tensor) -> torch.Tensor:
    """ops.cu:128-167: m = max(0, rowmax) (zero-initialised atomicMax), p = exp(v-m),
    out = p / (sum p + 1e-8)."""
    ids = row_ids.to(torch.int64)
    if values.numel() == 0:
        return values.clone()
    N = int(ids[-1]) + 1
    m = torch.zeros(N, dtype=values.dtype)
    m.scatter_reduce_(0, ids, values, reduce="amax", include_self=True)
    out = (values - m.index_select(0, ids)).exp()
    s = torch.zeros(N, dtype=out.dtype)
    s.scatter_add_(0, ids, out)
    s += 1e-8
    return out / s.index_select(0, ids)


def softmax_last_dim_backward(row_ids, values, grad_values) -> torch.Tensor:
    """ops.cu:169-194: g*y - y * sum_row(g*y)."""
    ids = row_ids.to(torch.int64)
    gi = grad_values * values
    s = torch.zeros_like(values)  # upstream allocates nnz entries and uses the first N rows
    s.scatter_add_(0, ids, gi)
    return gi - values * s.index_select(0, ids)


# --------------------------------------------------------------------------------------------
# Python layer of the path (swin3d_base.py:141-197, 483-498, 557-581, 589-677)
# --------------------------------------------------------------------------------------------
def qkv_sparse(qkv: torch.Tensor, indices: torch.Tensor, batch_size: int, spatial_dim: int):
    """swin3d_base.py:483-498.  qkv [N,3,H,hd] -> coalesced COO q, k (pre-transposed), v."""
    H, c = qkv.shape[2:]
    idx_qv, perm_qv, idx_k, perm_k = qkv_sparse_indices(indices, batch_size, spatial_dim, H, c)
    pq, pk = perm_qv.to(torch.int64), perm_k.to(torch.int64)
    iq, ik = idx_qv.index_select(1, pq), idx_k.index_select(1, pk)
    q = SparseTensor(iq, qkv[:, 0].reshape(-1).index_select(0, pq), [batch_size, H, spatial_dim, c])
    kt = SparseTensor(ik, qkv[:, 1].reshape(-1).index_select(0, pk), [batch_size, H, c, spatial_dim])
    v = SparseTensor(iq, qkv[:, 2].reshape(-1).index_select(0, pq), [batch_size, H, spatial_dim, c])
    return q, kt, v


def spspmm_block_naive(m1: SparseTensor, m2: SparseTensor, mul_type="q_k") -> SparseTensor:
    """swin3d_base.py:141-158."""
    if mul_type not in ("q_k", "qk_v"):
        raise ValueError(f"Invalid value for 'mul': {mul_type}. Must be 'q_k' or 'qk_v'.")
    idx, v, shape, _ = matmul_cuda_naive(m1.values, m1.indices, m1.shape, m2.values, m2.indices, m2.shape, mul_type)
    return SparseTensor(idx, v, shape)


def softmax_last_dim(mat: SparseTensor) -> SparseTensor:
    """swin3d_base.py:161-197: always computed in fp32, cast back."""
    rows = unique_consecutive_indices(flatten_indices(mat.indices[:3].contiguous(), mat.shape[:-1]))
    out = softmax_last_dim_forward(rows, mat.values.float())
    return SparseTensor(mat.indices, out.to(mat.values.dtype), mat.shape)


def relative_position_index(window_size) -> torch.Tensor:
    """swin3d_base.py:630-647: [n, n] int64 index into the bias table."""
    cd, ch, cw = (torch.arange(w) for w in window_size)
    coords = torch.stack(torch.meshgrid(cd, ch, cw, indexing="ij"))
    cf = torch.flatten(coords, 1)
    rel = (cf[:, :, None] - cf[:, None, :]).permute(1, 2, 0).contiguous()
    rel[:, :, 0] += window_size[0] - 1
    rel[:, :, 1] += window_size[1] - 1
    rel[:, :, 2] += window_size[2] - 1
    rel[:, :, 0] *= (2 * window_size[1] - 1) * (2 * window_size[2] - 1)
    rel[:, :, 1] *= 2 * window_size[2] - 1
    return rel.sum(-1)


def dense_bias(table: torch.Tensor, rpi: torch.Tensor, n: int, dtype) -> torch.Tensor:
    """swin3d_base.py:662-665: table[rpi[:n,:n]] as [H, n, n]."""
    b = table[rpi[:n, :n].reshape(-1)].reshape(n, n, -1)
    return b.permute(2, 0, 1).contiguous().to(dtype)


def sp_add_rpb(sp: SparseTensor, dense: torch.Tensor) -> SparseTensor:
    """swin3d_base.py:557-566."""
    i = sp.indices.to(torch.int64)
    g = dense.reshape(-1).index_select(0, i[1] * dense.shape[1] * dense.shape[2] + i[2] * dense.shape[2] + i[3])
    return SparseTensor(sp.indices, sp.values + g, sp.shape)


def sp_add_mask(sp: SparseTensor, mask: torch.Tensor) -> SparseTensor:
    """swin3d_base.py:569-581: -100 where the two positions lie in different regions."""
    i = sp.indices.to(torch.int64)
    w = i[0] % mask.shape[0]
    a = mask.reshape(-1).index_select(0, w * mask.shape[1] + i[2])
    b = mask.reshape(-1).index_select(0, w * mask.shape[1] + i[3])
    m = (b - a).to(sp.values.dtype)
    m = torch.where(m != 0, torch.full_like(m, -100.0), m)
    return SparseTensor(sp.indices, sp.values + m, sp.shape)


def window_attention_core(qkv, indices, batch_size, n, scale, table, rpi, mask=None):
    """WindowAttentionSparse.forward between the two Linears (swin3d_base.py:659-675).

    qkv [N,3,H,hd]; indices [N,2] int32.  Returns (out [N, H*hd] in the caller's voxel order,
    attn SparseTensor after softmax)."""
    q, kt, v = qkv_sparse(qkv, indices, batch_size, n)
    q = q * scale
    attn = spspmm_block_naive(q, kt, "q_k")
    attn = sp_add_rpb(attn, dense_bias(table, rpi, n, attn.values.dtype))
    if mask is not None:
        attn = sp_add_mask(attn, mask)
    attn = softmax_last_dim(attn)
    x = spspmm_block_naive(attn, v, "qk_v").permute((0, 2, 1, 3))
    arg_sort = return_inverse(flatten_indices(indices.T.contiguous(), [batch_size, n]), -1)[0]
    out = x.values.reshape(qkv.shape[0], -1).index_select(0, arg_sort.to(torch.int64))
    return out, attn


def window_attention_forward(features, indices, batch_size, n, num_heads, w_qkv, b_qkv, w_proj, b_proj,
                             table, rpi, mask=None):
    """WindowAttentionSparse.forward, whole (swin3d_base.py:654-677); dropout layers are
    identity at inference and `attn_drop` is never applied upstream."""
    C = features.shape[-1]
    hd = C // num_heads
    qkv = torch.nn.functional.linear(features, w_qkv, b_qkv).reshape(-1, 3, num_heads, hd)
    core, attn = window_attention_core(qkv, indices, batch_size, n, hd ** -0.5, table, rpi, mask)
    return torch.nn.functional.linear(core, w_proj, b_proj), core, attn


# --------------------------------------------------------------------------------------------
# independent cross-check: dense attention per window, no COO machinery at all
# --------------------------------------------------------------------------------------------
def dense_window_attention(qkv, indices, scale, table, rpi, mask=None, acc_dtype=torch.float64):
    """Per-window dense attention with the same quirks; loops in Python, for small cases and as
    an independent check of `window_attention_core`."""
    N, _, H, hd = qkv.shape
    out = torch.zeros(N, H * hd, dtype=acc_dtype)
    win = indices[:, 0].to(torch.int64)
    pos = indices[:, 1].to(torch.int64)
    order = torch.argsort(win * (int(pos.max()) + 1 if N else 1) + pos)
    ws, ps = win[order], pos[order]
    bounds = torch.cat([torch.tensor([0]), (ws[1:] != ws[:-1]).nonzero().squeeze(1) + 1, torch.tensor([N])])
    x = qkv.to(acc_dtype)
    for a, b in zip(bounds[:-1].tolist(), bounds[1:].tolist()):
        vox = order[a:b]
        p = ps[a:b]
        q = x[vox, 0].permute(1, 0, 2) * scale  # [H,c,hd]
        k = x[vox, 1].permute(1, 0, 2)
        v = x[vox, 2].permute(1, 0, 2)
        s = q @ k.transpose(1, 2)
        s = s + table[rpi[p][:, p].reshape(-1)].reshape(len(p), len(p), H).permute(2, 0, 1).to(acc_dtype)
        if mask is not None:
            r = mask[int(ws[a]) % mask.shape[0]][p].to(torch.int64)
            s = s + torch.where(r[:, None] != r[None, :], -100.0, 0.0).to(acc_dtype)[None]
        m = torch.clamp(s.amax(-1, keepdim=True), min=0.0)
        e = (s - m).exp()
        pr = e / (e.sum(-1, keepdim=True) + 1e-8)
        out[vox] = (pr @ v).permute(1, 0, 2).reshape(len(p), H * hd)
    return out


# --------------------------------------------------------------------------------------------------
# One Swin block / one stage (sparse_swin/swin3d_base.py:741-782, 857-873), on plain CPU tensors
# --------------------------------------------------------------------------------------------------
def swin_block(feats, coords, batch, dims, window_size, shift_size, prm, num_heads, eps=1e-5, acc_dtype=torch.float64):
    """SwinTransformerBlock.forward (swin3d_base.py:777-782): x + attn(norm1(x)) (forward_part1,
    :741-769: pad, roll by -shift, partition, WindowAttentionSparse, reverse, roll back - the window
    keys of `window_keys` are that chain's indices and the output order is the input's), then
    x + mlp(norm2(x)) (forward_part2, :771-775; MLP :1144-1149 with exact GELU).  `prm` maps
    upstream's parameter names inside the block (norm1.weight, attn.qkv.weight, ...) to tensors.
    Dropout and stochastic depth are the identity (evaluation mode)."""
    F = torch.nn.functional
    x = feats.to(acc_dtype)
    g = lambda k: prm[k].to(acc_dtype) if k in prm and prm[k] is not None else None
    C = x.shape[1]
    hd = C // num_heads
    idx, _, n, ws, ss, dp = window_keys(coords, batch, dims, window_size, shift_size)
    mask = compute_mask(dp, ws, ss) if any(s > 0 for s in ss) else None   # :755-760: mask only when shifted
    h = F.layer_norm(x, (C,), g("norm1.weight"), g("norm1.bias"), eps)
    qkv = F.linear(h, g("attn.qkv.weight"), g("attn.qkv.bias")).reshape(-1, 3, num_heads, hd)
    core = dense_window_attention(qkv, idx, hd ** -0.5, g("attn.relative_position_bias_table"),
                                  relative_position_index(window_size), mask, acc_dtype=acc_dtype)
    x = x + F.linear(core, g("attn.proj.weight"), g("attn.proj.bias"))
    h = F.layer_norm(x, (C,), g("norm2.weight"), g("norm2.bias"), eps)
    m = F.linear(F.gelu(F.linear(h, g("mlp.linear1.weight"), g("mlp.linear1.bias"))), g("mlp.linear2.weight"),
                 g("mlp.linear2.bias"))
    return x + m


def basic_layer(feats, coords, batch, dims, window_size, block_params, num_heads, eps=1e-5, acc_dtype=torch.float64):
    """BasicLayer.forward without downsampling (swin3d_base.py:857-873): blocks alternate shift 0
    and shift window // 2 (:835-836, :846)."""
    shift = tuple(w // 2 for w in window_size)
    x = feats
    for i, prm in enumerate(block_params):
        x = swin_block(x, coords, batch, dims, window_size, (0, 0, 0) if i % 2 == 0 else shift, prm, num_heads, eps, acc_dtype)
    return x


# --------------------------------------------------------------------------------------------------
# Sparse convolutions as the dense operation restricted to the active sites (the layers upstream
# takes from spconv: swin3d_base.py:915-935, 965-970, 989-994, 1039-1059).  Small grids only.
# Weights in the layout of sparseswin3d_b200.sparse_conv: [k^3, Cin, Cout], tap (dz, dy, dx) at
# (dz * k + dy) * k + dx.
# --------------------------------------------------------------------------------------------------
def _densify(feats, coords, batch, dims):
    C = feats.shape[1]
    dense = torch.zeros(batch, C, *dims, dtype=feats.dtype)
    c = coords.long()
    dense[c[:, 0], :, c[:, 1], c[:, 2], c[:, 3]] = feats
    return dense


def _dense_kernel(weight, k):
    k3, ci, co = weight.shape
    return weight.reshape(k, k, k, ci, co).permute(4, 3, 0, 1, 2).contiguous()   # [Cout, Cin, kz, ky, kx]


def subm_conv3d(feats, coords, batch, dims, weight, bias=None):
    """Submanifold convolution: conv3d with padding k // 2 on the densified scene, read at the input sites."""
    k = round(weight.shape[0] ** (1 / 3))
    out = torch.nn.functional.conv3d(_densify(feats, coords, batch, dims), _dense_kernel(weight, k), bias, padding=k // 2)
    c = coords.long()
    return out[c[:, 0], :, c[:, 1], c[:, 2], c[:, 3]]


def strided_conv3d(feats, coords, batch, dims, weight, bias=None):
    """kernel = stride = k, no padding: (features, coords [M,4] in (b,z,y,x) order, output dims).
    An output cell is active when any of its k^3 input cells is."""
    k = round(weight.shape[0] ** (1 / 3))
    F = torch.nn.functional
    out = F.conv3d(_densify(feats, coords, batch, dims), _dense_kernel(weight, k), bias, stride=k)
    occ = F.max_pool3d(_densify(torch.ones(coords.shape[0], 1, dtype=feats.dtype), coords, batch, dims), k, stride=k)
    idx = (occ[:, 0] > 0).nonzero()                       # lexicographic in (b, z, y, x)
    return out[idx[:, 0], :, idx[:, 1], idx[:, 2], idx[:, 3]], idx.to(I32), list(out.shape[2:])


def inverse_conv3d(feats_coarse, coords_coarse, batch, dims_coarse, coords_fine, weight, bias=None):
    """The transposed operation of `strided_conv3d`, read at the fine sites (zero, plus bias, for a
    fine voxel beyond the coarse grid)."""
    k = round(weight.shape[0] ** (1 / 3))
    k3, ci, co = weight.shape
    wt = weight.reshape(k, k, k, ci, co).permute(3, 4, 0, 1, 2).contiguous()     # [Cin, Cout, kz, ky, kx]
    out = torch.nn.functional.conv_transpose3d(_densify(feats_coarse, coords_coarse, batch, dims_coarse), wt, None, stride=k)
    c = coords_fine.long()
    res = torch.zeros(c.shape[0], co, dtype=feats_coarse.dtype)
    ok = (c[:, 1] < out.shape[2]) & (c[:, 2] < out.shape[3]) & (c[:, 3] < out.shape[4])
    res[ok] = out[c[ok, 0], :, c[ok, 1], c[ok, 2], c[ok, 3]]
    return res if bias is None else res + bias
