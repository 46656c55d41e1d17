"""Fused W-MSA / SW-MSA: the drop-in for upstream's ``WindowAttentionSparse``
(sparse_swin/swin3d_base.py:589-677)."""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn as nn

from . import _lib
from ._lib import check, dtype_code, lib, ptr, stream_ptr
from .window import WindowPlan, bucket_windows


def window_attention_fused_backward(qkv: torch.Tensor, grad_out: torch.Tensor, plan: WindowPlan, table: torch.Tensor,
                                    scale: float, use_mask: bool = False):
    """Gradients of `window_attention_fused` with respect to qkv and the bias table, given the
    gradient of its output (probabilities are recomputed, nothing of the forward is kept).
    Returns (dqkv [N,3,H,hd] in qkv's dtype, dtable fp32 in the table's shape)."""
    if not (qkv.is_cuda and qkv.is_contiguous() and qkv.dim() == 4 and qkv.shape[1] == 3):
        raise _lib.SswError("qkv must be a contiguous CUDA tensor [N, 3, heads, head_dim]")
    N, _, H, hd = qkv.shape
    if N != plan.layout.n_vox:
        raise _lib.SswError(f"plan was built for {plan.layout.n_vox} voxels, qkv has {N}")
    grad_out = grad_out.to(qkv.dtype).contiguous()
    if grad_out.shape != (N, H * hd):
        raise _lib.SswError("grad_out must be [N, heads*head_dim]")
    tab = table.detach()
    if tab.dtype != torch.float32 or not tab.is_contiguous():
        tab = tab.float().contiguous()
    dqkv = torch.empty_like(qkv)
    dtable = torch.zeros_like(tab)
    ws = torch.empty(max(int(lib.ssw_attn_fused_bwd_workspace_floats(N, H)), 4), dtype=torch.float32, device=qkv.device)
    rwc = (_lib.i32 * 3)(*plan.rpb_window)
    check(lib.ssw_attn_fused_bwd(ptr(qkv), ptr(grad_out), dtype_code(qkv.dtype), H, hd, plan.layout, ptr(plan.plan),
                                 ptr(tab), rwc, float(scale), int(bool(use_mask)), ptr(dqkv), ptr(dtable), ptr(ws),
                                 stream_ptr(qkv.device)), "ssw_attn_fused_bwd")
    return dqkv, dtable


class FusedWindowAttention(torch.autograd.Function):
    """window_attention_fused with autograd: forward keeps qkv and the table, backward recomputes.

    The backward walks the same plan again.  A plan that lives in a caller-owned ``plan_buffer``
    must therefore stay untouched until the backward has run: rebuilding another plan into that
    buffer in between makes the backward follow a plan for other inputs (the kernels hold every
    entry to its bounds and flag SSW_DEV_BAD_PLAN, but the gradients are then meaningless)."""

    @staticmethod
    def forward(ctx, qkv, table, plan, scale, use_mask):
        ctx.plan, ctx.scale, ctx.use_mask = plan, float(scale), bool(use_mask)
        ctx.save_for_backward(qkv, table)
        return window_attention_fused(qkv, plan, table, scale, use_mask=use_mask)

    @staticmethod
    def backward(ctx, grad_out):
        qkv, table = ctx.saved_tensors
        dqkv, dtable = window_attention_fused_backward(qkv, grad_out, ctx.plan, table, ctx.scale, ctx.use_mask)
        return dqkv, dtable.to(table.dtype), None, None, None


def default_tile_rows(num_heads: int, head_dim: int, dtype: torch.dtype, rpb_window: Sequence[int] = (7, 7, 7)) -> int:
    """Rows per work item the fused kernel wants for this configuration (pass it to bucket_windows)."""
    rw = (_lib.i32 * 3)(*[int(x) for x in rpb_window])
    return int(lib.ssw_default_tile_rows(num_heads, head_dim, dtype_code(dtype), rw))


def window_attention_fused(qkv: torch.Tensor, plan: WindowPlan, table: torch.Tensor, scale: float,
                           use_mask: bool = False, return_attn: bool = False, out: Optional[torch.Tensor] = None,
                           peer_out_ptrs: Sequence[int] = ()):
    """Everything between the two Linear layers of WindowAttentionSparse.forward
    (swin3d_base.py:659-675) in one kernel launch.

    qkv    [N, 3, H, hd] (or [N, 3*H*hd]) fp32 / bf16 / fp16, contiguous, CUDA
    plan   from `bucket_windows` (built with tile_rows = default_tile_rows(H, hd, dtype))
    table  relative_position_bias_table [(2Wz-1)(2Wy-1)(2Wx-1), H]
    Returns out [N, H*hd] in the caller's voxel order; with return_attn=True also the post-softmax
    COO values in upstream order (window, head, pos_i, pos_j) — that variant synchronises once to
    size the buffer.

    ``peer_out_ptrs``: device addresses of the same [N, H*hd] buffer on peer GPUs (mapped into this
    process, peer access enabled; at most seven): every finished row is stored there as well as to
    ``out`` (see ``shard.PeerRows``)."""
    if not qkv.is_cuda:
        raise _lib.SswError("qkv must be a CUDA tensor (there is no CPU path)")
    if qkv.dim() != 4 or qkv.shape[1] != 3:
        raise _lib.SswError("qkv must be [N, 3, heads, head_dim]")
    if not qkv.is_contiguous():
        raise _lib.SswError("qkv must be contiguous")
    N, _, H, hd = qkv.shape
    if N != plan.layout.n_vox:
        raise _lib.SswError(f"plan was built for {plan.layout.n_vox} voxels, qkv has {N}")
    want_padded = bool(lib.ssw_default_padded(dtype_code(qkv.dtype))) and not return_attn
    if bool(plan.layout.padded) and not want_padded:
        raise _lib.SswError("this plan was built with padded=True (tensor-core work list); fp32 tensors and "
                            "return_attn=True need a plan built with padded=False")
    if use_mask and not plan.has_regions:
        raise _lib.SswError("use_mask=True but the plan carries no region ids (no shift / no mask given)")
    table = table.detach()
    if table.dtype != torch.float32 or not table.is_contiguous():
        table = table.float().contiguous()
    rw = plan.rpb_window
    if table.shape != ((2 * rw[0] - 1) * (2 * rw[1] - 1) * (2 * rw[2] - 1), H):
        raise _lib.SswError(f"bias table shape {tuple(table.shape)} does not match window {rw} and {H} heads")
    if out is None:
        out = torch.empty((N, H * hd), dtype=qkv.dtype, device=qkv.device)
    attn = None
    if return_attn:
        st = plan.stats()
        if st["error"] & _lib.DEV_COO_RANGE or st["sum_c2"] * H >= 2 ** 31:
            raise _lib.SswError("sum c^2 * heads leaves the int32 domain of the COO layout")
        attn = torch.empty(st["sum_c2"] * H, dtype=qkv.dtype, device=qkv.device)
    rwc = (_lib.i32 * 3)(*rw)
    dests = [ptr(out)] + [int(a) for a in peer_out_ptrs]
    outs = (_lib.vp * len(dests))(*dests)
    check(lib.ssw_attn_fused_multi(ptr(qkv), dtype_code(qkv.dtype), H, hd, plan.layout, ptr(plan.plan), ptr(table), rwc,
                                   float(scale), int(bool(use_mask)), outs, len(dests), ptr(attn), stream_ptr(qkv.device)),
          "ssw_attn_fused")
    return (out, attn) if return_attn else out


def plan_params(num_heads: int, head_dim: int, dtype: torch.dtype, rpb_window: Sequence[int] = (7, 7, 7)) -> dict:
    """Keyword arguments for bucket_windows that match the kernel ssw_attn_fused runs for this
    configuration: fp32 -> CUDA-core kernel, contiguous packs; bf16/fp16 -> tensor-core kernel,
    padded packs."""
    return {"tile_rows": default_tile_rows(num_heads, head_dim, dtype, rpb_window),
            "padded": bool(lib.ssw_default_padded(dtype_code(dtype))), "rpb_window": tuple(int(x) for x in rpb_window)}


class WindowAttentionSparse(nn.Module):
    """Window multi-head self-attention with relative position bias over sparse voxel windows.

    Same constructor, parameters (``qkv``, ``proj``, ``relative_position_bias_table``) and buffer
    (``relative_position_index``) as upstream (swin3d_base.py:597-652), so a state_dict moves across
    unchanged.  ``forward(x, mask)`` accepts what upstream's forward accepts: an object with
    ``features`` [N,C], ``indices`` [N,2] int32 (window, pos), ``batch_size`` (all windows, empty
    ones included), ``spatial_shape`` (n,) and ``replace_feature`` (swin3d_base.py:654-677).
    Differentiable: with autograd recording the fused forward is paired with a fused backward."""

    def __init__(self, dim: int, num_heads: int, window_size: Sequence[int], qkv_bias: bool = False,
                 attn_drop: float = 0.0, proj_drop: float = 0.0) -> None:
        super().__init__()
        if len(window_size) != 3:
            raise ValueError("window_size must have three entries")
        self.dim, self.window_size, self.num_heads = dim, tuple(window_size), num_heads
        self.strict = True  # forward() raises on device-side error bits (see forward)
        head_dim = dim // num_heads
        self.scale = head_dim ** -0.5
        ws = self.window_size
        self.relative_position_bias_table = nn.Parameter(
            torch.zeros((2 * ws[0] - 1) * (2 * ws[1] - 1) * (2 * ws[2] - 1), num_heads))
        coords = torch.stack(torch.meshgrid(*(torch.arange(w) for w in ws), indexing="ij"))
        cf = torch.flatten(coords, 1)
        rel = (cf[:, :, None] - cf[:, None, :]).permute(1, 2, 0).contiguous()
        rel[:, :, 0] += ws[0] - 1
        rel[:, :, 1] += ws[1] - 1
        rel[:, :, 2] += ws[2] - 1
        rel[:, :, 0] *= (2 * ws[1] - 1) * (2 * ws[2] - 1)
        rel[:, :, 1] *= 2 * ws[2] - 1
        self.register_buffer("relative_position_index", rel.sum(-1))
        self.qkv = nn.Linear(dim, dim * 3, bias=qkv_bias)
        self.attn_drop = nn.Dropout(attn_drop)  # constructed but never applied upstream either
        self.proj = nn.Linear(dim, dim)
        self.proj_drop = nn.Dropout(proj_drop)
        nn.init.trunc_normal_(self.relative_position_bias_table, std=0.02, a=-2.0, b=2.0)

    def tile_rows(self, dtype: torch.dtype) -> int:
        return default_tile_rows(self.num_heads, self.dim // self.num_heads, dtype, self.window_size)

    def plan(self, x, mask: Optional[torch.Tensor], dtype: torch.dtype) -> WindowPlan:
        return bucket_windows(indices=x.indices, n_windows=int(x.batch_size), n_per_window=int(x.spatial_shape[0]),
                              mask=mask, **plan_params(self.num_heads, self.dim // self.num_heads, dtype,
                                                       self.window_size))

    def forward_features(self, features: torch.Tensor, plan: WindowPlan, use_mask: bool) -> torch.Tensor:
        qkv = self.qkv(features).reshape(-1, 3, self.num_heads, self.dim // self.num_heads)
        if torch.is_grad_enabled() and (qkv.requires_grad or self.relative_position_bias_table.requires_grad):
            core = FusedWindowAttention.apply(qkv.contiguous(), self.relative_position_bias_table, plan, self.scale, use_mask)
        else:
            core = window_attention_fused(qkv, plan, self.relative_position_bias_table, self.scale, use_mask)
        return self.proj_drop(self.proj(core))

    def forward_unfused(self, x, mask):
        """Upstream's forward, operator by operator (swin3d_base.py:654-677), on the COO operator
        surface; differentiable through the same autograd Functions upstream defines."""
        from . import ops
        from .sparse_tensor import qkv_sparse_cuda, softmax_last_dim, sp_add_mask, sp_add_rpb, spspmm_block_naive

        n = x.spatial_shape[0]
        b = x.batch_size
        c = x.features.shape[-1]
        qkv = self.qkv(x.features).reshape(-1, 3, self.num_heads, c // self.num_heads)
        q, k_t, v = qkv_sparse_cuda(qkv, x.indices, b, n)
        q = q * self.scale
        attn = spspmm_block_naive(q, k_t, "q_k")
        bias = self.relative_position_bias_table[self.relative_position_index[:n, :n].reshape(-1)].reshape(n, n, -1)
        bias = bias.permute(2, 0, 1).contiguous().to(attn.values.dtype)
        attn = sp_add_rpb(attn, bias)
        if mask is not None:
            attn = sp_add_mask(attn, mask)
        attn = softmax_last_dim(attn)
        x_ = spspmm_block_naive(attn, v, "qk_v").permute((0, 2, 1, 3))
        arg_sort = ops.return_inverse(ops.flatten_indices(x.indices.T.contiguous(), [b, n]), -1)[0]
        x = x.replace_feature(x_.values.reshape(x.features.shape).index_select(0, arg_sort))
        return x.replace_feature(self.proj_drop(self.proj(x.features)))

    def forward(self, x, mask, plan: Optional[WindowPlan] = None, fused: Optional[bool] = None,
                strict: Optional[bool] = None):
        """The fused kernels by default (differentiable: the backward recomputes the probabilities);
        fused=False runs upstream's operator chain on the COO surface instead.

        strict (default: ``self.strict``, True): after the kernels are enqueued, read the plan's
        device-side error word back and raise on duplicate voxels, (window, pos) outside
        [0, batch_size) x [0, n), an inconsistent plan or a device-side time-out - where upstream
        computes garbage silently.  This is one host synchronisation per call; it is skipped while a
        CUDA graph is being captured (check `plan.raise_on_error()` after a replay instead), and
        callers that pass their own `plan` and want no synchronisation set strict=False."""
        if fused is None:
            fused = True
        if not fused:
            return self.forward_unfused(x, mask)
        if plan is None:
            with torch.no_grad():
                plan = self.plan(x, mask, x.features.dtype)
        y = x.replace_feature(self.forward_features(x.features, plan, mask is not None))
        if (self.strict if strict is None else strict) and not torch.cuda.is_current_stream_capturing():
            plan.raise_on_error()
        return y
