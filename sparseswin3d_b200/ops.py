"""The ten operators upstream's pybind module exports (sparse_swin/ops.cpp:7-18), with the same
names, argument order and return tuples, implemented on the B200 library.  Every index tensor is
int32 and is returned as int32 (upstream avoids ``tensor[idx]`` because it promotes to int64,
README.md:20-23; the same convention holds here: only ``index_select`` style gathers).

Errors are ``RuntimeError`` (upstream: TORCH_CHECK -> c10::Error -> RuntimeError)."""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from . import _lib
from ._lib import PlanLayout, SswError, check, dtype_code, lib, ptr, stream_ptr

I32 = torch.int32
# qkv_sparse_indices raises on duplicate / out-of-range indices (one host read-back); set to False
# to skip the check, e.g. to keep that call free of synchronisation.
STRICT = True


def _ws(nbytes: int, device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)


def _need(cond: bool, msg: str):
    if not cond:
        raise SswError(msg)


def _i32(t: torch.Tensor, name: str):
    _need(t.is_cuda, f"{name} must be a CUDA tensor (there is no CPU path)")
    _need(t.dtype == I32, f"{name} dtype is not int32, but {t.dtype}")


def flatten_indices(indices: torch.Tensor, sizes: Sequence[int]) -> torch.Tensor:
    """ops.cpp:11 — row-major int32 hash of [D, nnz] indices; sizes[0] is never used."""
    _i32(indices, "indices")
    _need(indices.dim() == 2 and indices.shape[0] == len(sizes), "indices must be [len(sizes), nnz]")
    indices = indices.contiguous()
    out = torch.empty(indices.shape[1], dtype=I32, device=indices.device)
    sz = (_lib.i32 * len(sizes))(*[int(s) for s in sizes])
    check(lib.ssw_flatten_indices(ptr(indices), len(sizes), indices.shape[1], sz, ptr(out), stream_ptr(indices.device)),
          "flatten_indices")
    return out


def sort_indices(flattened_indices: torch.Tensor) -> torch.Tensor:
    """ops.cpp:12 — argsort of int32 keys, returned as int32."""
    _i32(flattened_indices, "flattened_indices")
    k = flattened_indices.contiguous().view(-1)
    n = k.numel()
    out = torch.empty(n, dtype=I32, device=k.device)
    nb = lib.ssw_argsort_workspace_bytes(n)
    ws = _ws(nb, k.device)
    check(lib.ssw_argsort_i32(ptr(k), n, ptr(out), ptr(ws), nb, stream_ptr(k.device)), "sort_indices")
    return out


def return_inverse(x: torch.Tensor, maxnum: int = -1) -> Tuple[torch.Tensor, int]:
    """ops.cpp:13 — (rank of every element among the distinct values present, their count).
    maxnum = -1 means max(x) + 1.  Synchronises (as upstream does) to return the count."""
    _i32(x, "x")
    x = x.contiguous().view(-1)
    n = x.numel()
    if maxnum == -1:
        _need(n > 0, "return_inverse of an empty tensor needs maxnum")
        maxnum = int(x.max()) + 1
    out = torch.empty(n, dtype=I32, device=x.device)
    cnt = torch.zeros(2, dtype=I32, device=x.device)
    nb = lib.ssw_return_inverse_workspace_bytes(maxnum)
    ws = _ws(nb, x.device)
    check(lib.ssw_return_inverse(ptr(x), n, int(maxnum), ptr(out), ptr(cnt), ptr(cnt[1:]), ptr(ws), nb,
                                 stream_ptr(x.device)), "return_inverse")
    c, err = cnt.tolist()
    _need(err == 0, "return_inverse: a value lies outside [0, maxnum)")
    return out, int(c)


def unique_consecutive_indices(nums: torch.Tensor) -> torch.Tensor:
    """ops.cpp:14 — inverse indices of unique_consecutive, int32."""
    _need(nums.dim() == 1, "nums must be 1-D")
    if nums.dtype != I32:
        _need(nums.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8), f"unsupported dtype {nums.dtype}")
        _need(nums.numel() == 0 or int(nums.abs().max()) < 2 ** 31, "values do not fit int32")
        nums = nums.to(I32)
    _i32(nums, "nums")
    nums = nums.contiguous()
    n = nums.numel()
    out = torch.empty(n, dtype=I32, device=nums.device)
    nb = lib.ssw_scan_workspace_bytes(n)
    ws = _ws(nb, nums.device)
    check(lib.ssw_unique_consecutive_inverse(ptr(nums), n, ptr(out), ptr(ws), nb, stream_ptr(nums.device)),
          "unique_consecutive_indices")
    return out


def qkv_sparse_indices(indices: torch.Tensor, batch_size: int, spatial_dim: int, num_heads: int, c: int):
    """ops.cpp:10 — (idx_qv [4, N*H*c], perm_qv, idx_k, perm_k), all int32.  idx_* are the unsorted
    index blocks; perm_* sort them (and the matching value vectors) into coalesced order."""
    from .window import bucket_windows

    _i32(indices, "indices")
    _need(indices.dim() == 2 and indices.shape[1] == 2, "indices must be [N, 2] (window, pos)")
    indices = indices.contiguous()
    N = indices.shape[0]
    M = N * num_heads * c
    dev = indices.device
    iqv = torch.empty((4, M), dtype=I32, device=dev)
    ik = torch.empty((4, M), dtype=I32, device=dev)
    pqv = torch.empty(M, dtype=I32, device=dev)
    pk = torch.empty(M, dtype=I32, device=dev)
    if N == 0:
        return iqv, pqv, ik, pk
    plan = bucket_windows(indices=indices, n_windows=int(batch_size), n_per_window=int(spatial_dim))
    check(lib.ssw_qkv_sparse_indices(ptr(indices), N, int(num_heads), int(c), plan.layout, ptr(plan.plan), ptr(iqv),
                                     ptr(pqv), ptr(ik), ptr(pk), stream_ptr(dev)), "qkv_sparse_indices")
    # Upstream silently mis-sorts on duplicate or out-of-range (window, pos); this operator chain
    # synchronises a few calls later anyway (matmul_cuda_naive reads its block counts back), so the
    # device-side error word is read here, unless a CUDA graph is being captured.
    if STRICT and not torch.cuda.is_current_stream_capturing():
        plan.raise_on_error()
    return iqv, pqv, ik, pk


def matmul_cuda_naive(mat1_v, mat1_idx, mat1_shape: List[int], mat2_v, mat2_idx, mat2_shape: List[int], mul_type: str):
    """ops.cpp:8 — blocked per-(window, head) product of two coalesced COO operands.
    'q_k': q [B,H,n,hd] x k_t [B,H,hd,n] -> attn [B,H,n,n];  'qk_v': attn x v [B,H,n,hd] -> [B,H,n,hd].
    Returns (idx [4, nnz] int32, vals, shape, _c int32)."""
    _need(mat1_idx.dim() == 2 and mat2_idx.dim() == 2, "index tensors must be 2-D")
    _need(mat1_v.dim() == 1 and mat2_v.dim() == 1, "value tensors must be 1-D")
    _need(mul_type in ("q_k", "qk_v"), f"Invalid mul_type: {mul_type}. Expected 'q_k' or 'qk_v'.")
    _need(mat1_v.dtype == mat2_v.dtype, f"mat1 dtype {mat1_v.dtype} does not match mat2 dtype {mat2_v.dtype}")
    _need(mat1_idx.dtype == mat2_idx.dtype, "mat1 index dtype does not match mat2 index dtype")
    _i32(mat1_idx, "mat1 index")
    _need(len(mat1_shape) == 4 and len(mat2_shape) == 4 and mat1_shape[0] == mat2_shape[0]
          and mat1_shape[1] == mat2_shape[1] and mat1_shape[3] == mat2_shape[2],
          f"Invalid shapes: mat1_shape {list(mat1_shape)} and mat2_shape {list(mat2_shape)}")
    dev = mat1_v.device
    dt = dtype_code(mat1_v.dtype)
    mat1_v, mat2_v = mat1_v.contiguous(), mat2_v.contiguous()
    mat1_idx, mat2_idx = mat1_idx.contiguous(), mat2_idx.contiguous()
    is_pv = mul_type == "qk_v"
    C = int(mat2_shape[3] if is_pv else mat1_shape[3])
    blk_idx = mat2_idx if is_pv else mat1_idx
    nnz_blk = blk_idx.shape[1]
    _need(C > 0 and nnz_blk % C == 0, "operand rows are not dense in the channel dimension")
    R = nnz_blk // C
    blk_start = torch.empty(R + 1, dtype=I32, device=dev)
    sq_start = torch.empty(R + 1, dtype=I32, device=dev)
    counts = torch.zeros(2, dtype=torch.int64, device=dev)
    nb_ws = lib.ssw_coo_plan_workspace_bytes(R)
    ws = _ws(nb_ws, dev)
    st = stream_ptr(dev)
    check(lib.ssw_coo_block_plan(ptr(blk_idx), nnz_blk, C, ptr(blk_start), ptr(sq_start), ptr(counts), ptr(ws), nb_ws,
                                 st), "matmul_cuda_naive (plan)")
    n_blocks, sum_sq = counts.tolist()  # the one synchronisation; upstream has ~10 .item() calls here
    total = nnz_blk if is_pv else sum_sq
    _need(sum_sq < 2 ** 31, "sum of c^2 leaves the int32 domain of the COO layout")
    if is_pv:
        _need(mat1_v.numel() == sum_sq, "attention operand does not match the block structure of v")
    else:
        _need(mat2_v.numel() == mat1_v.numel(), "q and k_t must have the same number of values")
    out_idx = torch.empty((4, total), dtype=I32, device=dev)
    out_v = torch.empty(total, dtype=mat1_v.dtype, device=dev)
    c_out = torch.empty(n_blocks, dtype=I32, device=dev)
    check(lib.ssw_coo_matmul(int(is_pv), dt, ptr(mat1_v), ptr(mat1_idx), mat1_idx.shape[1], ptr(mat2_v), C,
                             ptr(blk_start), ptr(sq_start), n_blocks, total, ptr(out_v), ptr(out_idx), ptr(c_out),
                             ptr(counts), st), "matmul_cuda_naive")
    shape = [int(mat1_shape[0]), int(mat1_shape[1]), int(mat1_shape[2]), int(mat2_shape[3])]
    return out_idx, out_v, shape, c_out


def _offsets(_c: torch.Tensor):
    _i32(_c, "_c")
    _c = _c.contiguous()
    nb = _c.numel()
    cstart = torch.empty(nb + 1, dtype=I32, device=_c.device)
    sqstart = torch.empty(nb + 1, dtype=I32, device=_c.device)
    nbytes = lib.ssw_coo_plan_workspace_bytes(nb)
    ws = _ws(nbytes, _c.device)
    check(lib.ssw_coo_offsets_from_counts(ptr(_c), nb, ptr(cstart), ptr(sqstart), ptr(ws), nbytes,
                                          stream_ptr(_c.device)), "block offsets")
    return cstart, sqstart, nb


_GRAD_MODES = {"rc_cr": 0, "rr_rc": 1, "cr_rr": 2}


def matmul_grad_cuda_naive(mat1_v, mat2_v, _c, C: int, mul_type: str) -> torch.Tensor:
    """ops.cpp:9 — the three blocked products of the backward pass, keyed by `_c` only."""
    _need(mul_type in _GRAD_MODES, f"Invalid mul_type: {mul_type}. Expected 'rc_cr', 'rr_rc' or 'cr_rr'.")
    _need(mat1_v.dtype == mat2_v.dtype, "mat1 dtype does not match mat2 dtype")
    mat1_v, mat2_v = mat1_v.contiguous(), mat2_v.contiguous()
    cstart, sqstart, nb = _offsets(_c)
    total = int((_c.long() * _c.long()).sum()) if mul_type == "rc_cr" else int(_c.long().sum()) * int(C)
    out = torch.empty(total, dtype=mat1_v.dtype, device=mat1_v.device)
    check(lib.ssw_coo_matmul_grad(_GRAD_MODES[mul_type], dtype_code(mat1_v.dtype), ptr(mat1_v), ptr(mat2_v), ptr(cstart),
                                  ptr(sqstart), nb, int(C), ptr(out), stream_ptr(mat1_v.device)), "matmul_grad_cuda_naive")
    return out


def qkv_transpose(mat1_v, _c, C: int, mul_type: str) -> torch.Tensor:
    """ops.cpp:17 — per-block transposes: 'rc' [c,C] -> [C,c], 'rr' [c,c] -> transposed."""
    _need(mul_type in ("rc", "rr"), f"Invalid mul_type: {mul_type}. Expected 'rc', or 'rr'.")
    mat1_v = mat1_v.contiguous()
    cstart, sqstart, nb = _offsets(_c)
    out = torch.empty_like(mat1_v)
    check(lib.ssw_coo_block_transpose(int(mul_type == "rr"), dtype_code(mat1_v.dtype), ptr(mat1_v), ptr(cstart),
                                      ptr(sqstart), nb, int(C), ptr(out), stream_ptr(mat1_v.device)), "qkv_transpose")
    return out


def _softmax_common(indices, values):
    _i32(indices, "indices")
    _need(values.dtype == torch.float32, "softmax runs in float32 (upstream casts before the call)")
    indices, values = indices.contiguous(), values.contiguous()
    nnz = values.numel()
    n_rows = int(indices[-1]) + 1 if nnz else 0  # assumes sorted row ids, as upstream (ops.cu:135)
    row_start = torch.empty(n_rows + 1, dtype=I32, device=values.device)
    return indices, values, nnz, n_rows, row_start


def softmax_last_dim_forward(indices: torch.Tensor, values: torch.Tensor) -> torch.Tensor:
    """ops.cpp:15 — row-wise softmax over sorted row ids with upstream's max(0, .) and +1e-8."""
    indices, values, nnz, n_rows, row_start = _softmax_common(indices, values)
    out = torch.empty_like(values)
    check(lib.ssw_softmax_rows_fwd(ptr(indices), nnz, n_rows, ptr(values), ptr(out), ptr(row_start),
                                   stream_ptr(values.device)), "softmax_last_dim_forward")
    return out


def softmax_last_dim_backward(indices: torch.Tensor, values: torch.Tensor, grad_values: torch.Tensor) -> torch.Tensor:
    """ops.cpp:16 — g*y - y*sum_row(g*y)."""
    indices, values, nnz, n_rows, row_start = _softmax_common(indices, values)
    grad_values = grad_values.contiguous().float()
    out = torch.empty_like(values)
    check(lib.ssw_softmax_rows_bwd(ptr(indices), nnz, n_rows, ptr(values), ptr(grad_values), ptr(out), ptr(row_start),
                                   stream_ptr(values.device)), "softmax_last_dim_backward")
    return out
