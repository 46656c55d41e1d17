"""Python layer of upstream's unfused path (sparse_swin/swin3d_base.py:29-198, 483-498, 557-581) on
top of `ops`: the int32 COO container, the two autograd Functions, qkv_sparse_cuda and the bias /
mask adds.  Same names and call signatures as upstream, so code written against upstream's helpers
runs unchanged; only the module it imports them from differs."""
from __future__ import annotations

from typing import List

import torch
from torch.autograd import Function
from torch.autograd.function import once_differentiable

from . import ops
from ._lib import check, dtype_code, lib, ptr, stream_ptr


class SparseTensor:
    """indices [4, nnz] int32, values [nnz], shape list[4] (swin3d_base.py:29-65)."""

    def __init__(self, indices, values, shape):
        assert indices.ndim == 2 and indices.shape[0] == 4, "Invalid shape"
        assert values.ndim == 1, "Invalid shape"
        assert len(shape) == 4, "Invalid shape"
        self.indices, self.values, self.shape = indices, values, list(shape)

    def __repr__(self):
        return f"SparseTensor(indices={self.indices}, values={self.values}, shape={self.shape})"

    def coalesce(self):
        order = ops.sort_indices(ops.flatten_indices(self.indices, self.shape))
        return SparseTensor(self.indices.index_select(1, order), self.values.index_select(0, order), self.shape)

    def permute(self, dims):
        if len(dims) != len(self.shape):
            raise ValueError(f"The length of dims {dims} must match the number of dimensions in shape {self.shape}.")
        if sorted(dims) != list(range(len(self.shape))):
            raise ValueError(f"dims {dims} must be a permutation of the dimensions [0, {len(self.shape) - 1}].")
        shape = [self.shape[d] for d in dims]
        idx = self.indices.index_select(0, torch.tensor(list(dims), dtype=torch.int32, device=self.indices.device))
        order = ops.sort_indices(ops.flatten_indices(idx, shape))
        return SparseTensor(idx.index_select(1, order), self.values.index_select(0, order), shape)

    def __mul__(self, other):
        if isinstance(other, (int, float)):
            return SparseTensor(self.indices, self.values * other, self.shape)
        raise NotImplementedError


class _spspmm_block_naive(Function):
    """swin3d_base.py:68-138."""

    @staticmethod
    def forward(ctx, mat1_v, mat1_idx, mat1_shape, mat2_v, mat2_idx, mat2_shape, mul_type):
        if mul_type not in ("q_k", "qk_v"):
            raise ValueError(f"Invalid value for 'mul': {mul_type}. Must be 'q_k' or 'qk_v'.")
        idx, v, shape, _c = ops.matmul_cuda_naive(mat1_v, mat1_idx, mat1_shape, mat2_v, mat2_idx, mat2_shape, mul_type)
        ctx.save_for_backward(mat2_v, mat1_v, _c)
        ctx.mul_type = mul_type
        ctx.C = mat1_shape[-1] if mul_type == "q_k" else mat2_shape[-1]
        ctx.mark_non_differentiable(idx)
        ctx.shape = shape
        return idx, v

    @staticmethod
    @once_differentiable
    def backward(ctx, _g_idx, g):
        g = g.contiguous()
        mat2_v, mat1_v, _c = ctx.saved_tensors
        C = ctx.C
        if ctx.mul_type == "q_k":
            g1 = ops.matmul_grad_cuda_naive(g, mat2_v, _c, C, "rr_rc")
            g2 = ops.matmul_grad_cuda_naive(ops.qkv_transpose(mat1_v, _c, C, "rc"), ops.qkv_transpose(g, _c, C, "rr"),
                                            _c, C, "cr_rr")
        else:
            g1 = ops.matmul_grad_cuda_naive(g, mat2_v, _c, C, "rc_cr")
            g2 = ops.matmul_grad_cuda_naive(ops.qkv_transpose(mat1_v, _c, C, "rr"), ops.qkv_transpose(g, _c, C, "rc"),
                                            _c, C, "rr_rc")
        return g1, None, None, g2, None, None, None


def spspmm_block_naive(mat1: SparseTensor, mat2: SparseTensor, mul_type: str = "q_k") -> SparseTensor:
    """swin3d_base.py:141-158."""
    if mul_type not in ("q_k", "qk_v"):
        raise ValueError(f"Invalid value for 'mul': {mul_type}. Must be 'q_k' or 'qk_v'.")
    shape = [mat1.shape[0], mat1.shape[1], mat1.shape[2], mat2.shape[3]]
    idx, v = _spspmm_block_naive.apply(mat1.values, mat1.indices, mat1.shape, mat2.values, mat2.indices, mat2.shape,
                                       mul_type)
    return SparseTensor(idx, v, shape)


class _softmax_last_dim(Function):
    """swin3d_base.py:161-188."""

    @staticmethod
    def forward(ctx, mat_v, mat_idx, mat_shape):
        rows = ops.unique_consecutive_indices(ops.flatten_indices(mat_idx, mat_shape))
        out = ops.softmax_last_dim_forward(rows, mat_v)
        ctx.save_for_backward(out, rows)
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        out, rows = ctx.saved_tensors
        return ops.softmax_last_dim_backward(rows, out, grad), None, None


def softmax_last_dim(mat: SparseTensor) -> SparseTensor:
    """swin3d_base.py:191-197: always in fp32, cast back."""
    dtype = mat.values.dtype
    out = _softmax_last_dim.apply(mat.values.float(), mat.indices[:3].contiguous(), mat.shape[:-1])
    return SparseTensor(mat.indices, out.to(dtype), mat.shape)


def qkv_sparse_cuda(qkv: torch.Tensor, indices: torch.Tensor, batch_size: int, spatial_shape: int):
    """swin3d_base.py:483-498: qkv [N,3,H,hd] -> coalesced COO q, k (already transposed), v."""
    H, c = qkv.shape[2:]
    iqv, pqv, ik, pk = ops.qkv_sparse_indices(indices, batch_size, spatial_shape, H, c)
    iq = iqv.index_select(1, pqv)
    ikk = ik.index_select(1, pk)
    q = SparseTensor(iq, qkv[:, 0].reshape(-1).index_select(0, pqv), [batch_size, H, spatial_shape, c])
    kt = SparseTensor(ikk, qkv[:, 1].reshape(-1).index_select(0, pk), [batch_size, H, c, spatial_shape])
    v = SparseTensor(iq, qkv[:, 2].reshape(-1).index_select(0, pqv), [batch_size, H, spatial_shape, c])
    return q, kt, v


class _add_bias_mask(Function):
    @staticmethod
    def forward(ctx, vals, idx, dense, mask):
        vals = vals.contiguous()
        out = torch.empty_like(vals)
        d = None if dense is None else dense.to(vals.dtype).contiguous()
        check(lib.ssw_coo_add_bias_mask(dtype_code(vals.dtype), ptr(vals), ptr(idx), vals.numel(), ptr(d),
                                        0 if d is None else d.shape[1], ptr(mask), 0 if mask is None else mask.shape[0],
                                        0 if mask is None else mask.shape[1], ptr(out), stream_ptr(vals.device)),
              "sp_add_rpb / sp_add_mask")
        ctx.save_for_backward(idx)
        ctx.dense_shape = None if dense is None else dense.shape
        ctx.dense_dtype = None if dense is None else dense.dtype
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, g):
        (idx,) = ctx.saved_tensors
        gd = None
        if ctx.dense_shape is not None and ctx.needs_input_grad[2]:
            H, n, _ = ctx.dense_shape
            flat = idx[1].long() * n * n + idx[2].long() * n + idx[3].long()
            gd = torch.zeros(H * n * n, dtype=torch.float32, device=g.device).index_add_(0, flat, g.float())
            gd = gd.view(H, n, n).to(ctx.dense_dtype)
        return g, None, gd, None


def sp_add_rpb(sparse: SparseTensor, dense: torch.Tensor) -> SparseTensor:
    """swin3d_base.py:557-566: values + dense[head, pos_i, pos_j], dense [H, n, n]."""
    return SparseTensor(sparse.indices, _add_bias_mask.apply(sparse.values, sparse.indices.contiguous(), dense, None),
                        sparse.shape)


def sp_add_mask(sparse: SparseTensor, dense: torch.Tensor) -> SparseTensor:
    """swin3d_base.py:569-581: -100 where the two positions lie in different mask regions."""
    return SparseTensor(sparse.indices,
                        _add_bias_mask.apply(sparse.values, sparse.indices.contiguous(), None, dense.contiguous()),
                        sparse.shape)
