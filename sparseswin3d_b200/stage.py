"""One Swin stage over sparse voxels: `SwinTransformerBlock` and `BasicLayer` with upstream's
constructors, parameter names and forward semantics (sparse_swin/swin3d_base.py:680-873), built
for reuse across the blocks of a stage:

* the window plan depends on the coordinates, the window and the shift only, so a stage buckets the
  voxels ONCE per shift (two plans: W-MSA and SW-MSA) and every block of that parity reuses its plan
  (upstream pads, rolls, partitions and sorts again in every block, swin3d_base.py:741-769, and lists
  the reuse as an open item, README.md:94);
* the rows between the GEMMs are touched once: `ssw_add_layernorm` adds a branch's output to the
  running features and normalises the sum for the next branch in one pass, also across the block
  boundary (the residual add that ends block i and norm1 of block i+1).

The GEMMs themselves (qkv, proj, the two MLP Linears) are library calls (torch / cuBLAS).

`SparseVoxels` carries the four fields of an spconv SparseConvTensor that upstream's blocks read
(`features`, `indices` [N,4] int32 (b,z,y,x), `spatial_shape`, `batch_size`) and `replace_feature`.
Autograd: with gradients recording, the element-wise shell runs as torch operations (the attention
core keeps its fused forward and backward); the fused shell is the inference path."""
from __future__ import annotations

import copy
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib
from ._lib import check, dtype_code, lib, ptr, stream_ptr
from .attention import WindowAttentionSparse, plan_params
from .window import WindowPlan, bucket_windows, resolve_geometry


class SparseVoxels:
    """features [N,C], indices [N,4] int32 (batch, z, y, x), spatial_shape (D,H,W), batch_size."""

    def __init__(self, features: torch.Tensor, indices: torch.Tensor, spatial_shape: Sequence[int], batch_size: int):
        self.features = features
        self.indices = indices
        self.spatial_shape = list(spatial_shape)
        self.batch_size = int(batch_size)
        self.indice_dict = {}          # rulebooks of the sparse convolutions, by indice_key (shared by copies)

    def replace_feature(self, new_features: torch.Tensor) -> "SparseVoxels":
        out = copy.copy(self)          # a new container over the same index tensor, as spconv does
        out.features = new_features
        return out


def add_layernorm(a: torch.Tensor, b: Optional[torch.Tensor], norm: Optional[nn.LayerNorm], want_sum: bool = True,
                  sum_out: Optional[torch.Tensor] = None):
    """(a + b, LayerNorm(a + b)) in one pass over the rows; b=None: the sum is a itself (not
    written), norm=None: only the sum.  Returns (sum, normalised); entries not asked for are None."""
    if not a.is_cuda or a.dim() != 2 or not a.is_contiguous():
        raise _lib.SswError("add_layernorm wants a contiguous [N, C] CUDA tensor")
    if b is not None and (b.shape != a.shape or b.dtype != a.dtype or not b.is_contiguous()):
        raise _lib.SswError("add_layernorm: b must match a")
    n, c = a.shape
    s = None
    if b is not None and want_sum:
        s = sum_out if sum_out is not None else torch.empty_like(a)
    y = torch.empty_like(a) if norm is not None else None
    gamma = beta = None
    eps = 0.0
    if norm is not None:
        if tuple(norm.normalized_shape) != (c,) or norm.weight is None or norm.bias is None:
            raise _lib.SswError("add_layernorm wants an affine LayerNorm over the channel dimension")
        gamma, beta, eps = norm.weight.detach().float().contiguous(), norm.bias.detach().float().contiguous(), norm.eps
    check(lib.ssw_add_layernorm(ptr(a), ptr(b), ptr(gamma), ptr(beta), float(eps), dtype_code(a.dtype), n, c, ptr(s), ptr(y),
                                stream_ptr(a.device)), "ssw_add_layernorm")
    return (a if b is None else s), y


class DropPath(nn.Module):
    """Stochastic depth over the leading dimension (swin3d_base.py:1076-1106): in training each ROW
    of the [N, C] features is dropped with probability p and the rest scaled by 1/(1-p)."""

    def __init__(self, drop_prob: float = 0.0, scale_by_keep: bool = True):
        super().__init__()
        if not 0 <= drop_prob <= 1:
            raise ValueError("Drop path prob should be between 0 and 1.")
        self.drop_prob, self.scale_by_keep = drop_prob, scale_by_keep

    def forward(self, x):
        if self.drop_prob == 0.0 or not self.training:
            return x
        keep = 1.0 - self.drop_prob
        mask = x.new_empty((x.shape[0],) + (1,) * (x.dim() - 1)).bernoulli_(keep)
        if keep > 0.0 and self.scale_by_keep:
            mask.div_(keep)
        return x * mask


class MLP(nn.Module):
    """Linear - activation - Linear with upstream's parameter names (swin3d_base.py:1109-1149)."""

    def __init__(self, hidden_size: int, mlp_dim: int, dropout_rate: float = 0.0, act: str = "GELU"):
        super().__init__()
        if not 0 <= dropout_rate <= 1:
            raise ValueError("dropout_rate should be between 0 and 1.")
        if act != "GELU":
            raise ValueError("only the GELU activation of upstream's default configuration is built")
        mlp_dim = mlp_dim or hidden_size
        self.linear1 = nn.Linear(hidden_size, mlp_dim)
        self.linear2 = nn.Linear(mlp_dim, hidden_size)
        self.fn = nn.GELU()
        self.drop1 = nn.Dropout(dropout_rate)
        self.drop2 = self.drop1

    def forward(self, x):
        return self.drop2(self.linear2(self.drop1(self.fn(self.linear1(x)))))


class SwinTransformerBlock(nn.Module):
    """norm1 - window attention - residual - norm2 - MLP - residual (swin3d_base.py:680-782)."""

    def __init__(self, dim: int, num_heads: int, window_size: Sequence[int], shift_size: Sequence[int],
                 mlp_ratio: float = 4.0, qkv_bias: bool = True, drop: float = 0.0, attn_drop: float = 0.0,
                 drop_path: float = 0.0, act_layer: str = "GELU", norm_layer=nn.LayerNorm, use_checkpoint: bool = False):
        super().__init__()
        self.dim, self.num_heads = dim, num_heads
        self.window_size, self.shift_size = tuple(window_size), tuple(shift_size)
        self.mlp_ratio, self.use_checkpoint = mlp_ratio, use_checkpoint
        self.norm1 = norm_layer(dim)
        self.attn = WindowAttentionSparse(dim, window_size=self.window_size, num_heads=num_heads, qkv_bias=qkv_bias,
                                          attn_drop=attn_drop, proj_drop=drop)
        self.drop_path = DropPath(drop_path) if drop_path > 0.0 else nn.Identity()
        self.norm2 = norm_layer(dim)
        self.mlp = MLP(hidden_size=dim, mlp_dim=int(dim * mlp_ratio), act=act_layer, dropout_rate=drop)

    # ---- geometry / plan ---------------------------------------------------------------------
    def geometry(self, x):
        return resolve_geometry(int(x.batch_size), tuple(int(v) for v in x.spatial_shape), self.window_size, self.shift_size)

    def build_plan(self, x, dtype: torch.dtype, scratch=None, plan_buffer=None) -> WindowPlan:
        """Pad, cyclic shift, partition and sort (swin3d_base.py:744-761) as one bucketing call."""
        return bucket_windows(coords=x.indices, geom=self.geometry(x), scratch=scratch, plan_buffer=plan_buffer,
                              **plan_params(self.num_heads, self.dim // self.num_heads, dtype, self.window_size))

    def fusable(self, feats: torch.Tensor) -> bool:
        """The one-pass shell needs affine LayerNorms, no stochastic depth in flight and no autograd."""
        return (isinstance(self.norm1, nn.LayerNorm) and isinstance(self.norm2, nn.LayerNorm)
                and self.norm1.elementwise_affine and self.norm2.elementwise_affine
                and not (self.training and isinstance(self.drop_path, DropPath))
                and not (torch.is_grad_enabled() and (feats.requires_grad or any(p.requires_grad for p in self.parameters())))
                and feats.is_cuda and feats.is_contiguous() and (feats.shape[1] * feats.element_size()) % 16 == 0
                and feats.shape[1] * feats.element_size() <= 2048)

    # ---- the two halves, on plain feature tensors --------------------------------------------
    def attention_branch(self, normed: torch.Tensor, plan: WindowPlan, use_mask: bool) -> torch.Tensor:
        return self.attn.forward_features(normed, plan, use_mask)

    def forward(self, x, mask_matrix=None, plan: Optional[WindowPlan] = None, fuse_shell: bool = True):
        """x: voxels in scene coordinates (`SparseVoxels` or an spconv tensor).  `mask_matrix` is
        accepted for signature compatibility: region ids come from the geometry in closed form, and
        the mask applies exactly when the resolved shift is non-zero (swin3d_base.py:755-760)."""
        feats = x.features
        geom = self.geometry(x)
        if plan is None:
            with torch.no_grad():
                plan = self.build_plan(x, feats.dtype)
        use_mask = bool(geom.shifted)
        if fuse_shell and self.fusable(feats):
            _, h = add_layernorm(feats, None, self.norm1)
            a = self.attention_branch(h, plan, use_mask)
            x1, h2 = add_layernorm(feats, a, self.norm2)
            m = self.mlp(h2)
            out, _ = add_layernorm(x1, m, None, sum_out=x1)
            return x.replace_feature(out)
        a = self.attention_branch(self.norm1(feats), plan, use_mask)
        x1 = feats + self.drop_path(a)
        return x.replace_feature(x1 + self.drop_path(self.mlp(self.norm2(x1))))


class BasicLayer(nn.Module):
    """`depth` blocks alternating W-MSA and SW-MSA (shift = window // 2), then an optional
    downsampling module (swin3d_base.py:785-873).  The two window plans of the stage are built once
    per forward and shared by the blocks of each parity; `plans=` lets a caller that keeps the
    coordinates across forwards (several passes over one scene) supply them and skip bucketing."""

    def __init__(self, dim: int, depth: int, num_heads: int, window_size: Sequence[int], drop_path=0.0,
                 mlp_ratio: float = 4.0, qkv_bias: bool = False, drop: float = 0.0, attn_drop: float = 0.0,
                 norm_layer=nn.LayerNorm, downsample=None, use_checkpoint: bool = False, indice_key=None):
        super().__init__()
        self.window_size = tuple(window_size)
        self.shift_size = tuple(i // 2 for i in window_size)
        self.no_shift = tuple(0 for _ in window_size)
        self.depth, self.use_checkpoint = depth, use_checkpoint
        self.blocks = nn.ModuleList([
            SwinTransformerBlock(dim=dim, num_heads=num_heads, window_size=self.window_size,
                                 shift_size=self.no_shift if i % 2 == 0 else self.shift_size, mlp_ratio=mlp_ratio,
                                 qkv_bias=qkv_bias, drop=drop, attn_drop=attn_drop,
                                 drop_path=drop_path[i] if isinstance(drop_path, list) else drop_path,
                                 norm_layer=norm_layer, use_checkpoint=use_checkpoint) for i in range(depth)])
        self.downsample = downsample
        if callable(self.downsample):
            self.downsample = downsample(dim=dim, norm_layer=norm_layer, spatial_dims=len(self.window_size),
                                         indice_key=indice_key)
        self.strict = True
        self.reuse_plans = True   # False: every block buckets for itself, as upstream's blocks do
        self.fuse_shell = True    # False: LayerNorm and residual adds as separate torch operations
        self._aux = None

    def build_plans(self, x, dtype: torch.dtype, buffers=None):
        """The stage's two plans: [unshifted, shifted].  The shifted plan is built on a second stream
        beside the first (both read the coordinates only).  `buffers` = [(scratch, plan_buffer)] * 2
        keeps the call free of allocations (graph capture, repeated forwards)."""
        plans = [None, None]
        if self.depth == 0:
            return plans
        cur = torch.cuda.current_stream(x.indices.device)
        with torch.no_grad():
            if self.depth > 1:
                if self._aux is None or self._aux.device != x.indices.device:
                    self._aux = torch.cuda.Stream(device=x.indices.device)
                self._aux.wait_stream(cur)
                with torch.cuda.stream(self._aux):
                    sb = buffers[1] if buffers else (None, None)
                    plans[1] = self.blocks[1].build_plan(x, dtype, scratch=sb[0], plan_buffer=sb[1])
            sb = buffers[0] if buffers else (None, None)
            plans[0] = self.blocks[0].build_plan(x, dtype, scratch=sb[0], plan_buffer=sb[1])
            if self.depth > 1:
                cur.wait_stream(self._aux)
        return plans

    def forward(self, x, plans=None):
        feats = x.features
        if plans is None and not self.reuse_plans:
            plans = []
            for blk in self.blocks:
                with torch.no_grad():
                    plans.append(blk.build_plan(x, feats.dtype))
                x = blk(x, None, plan=plans[-1], fuse_shell=self.fuse_shell)
            return self._finish(x, plans)
        if plans is None:
            plans = self.build_plans(x, feats.dtype)
        fused = self.fuse_shell and len(self.blocks) > 0 and all(b.fusable(feats) for b in self.blocks)
        if fused:
            # running features `cur`, pending branch output `pend` (added by the next one-pass call)
            cur, pend = feats, None
            for i, blk in enumerate(self.blocks):
                use_mask = bool(blk.geometry(x).shifted)
                cur, h = add_layernorm(cur, pend, blk.norm1)           # ends block i-1, opens block i
                a = blk.attention_branch(h, plans[i % 2], use_mask)
                cur, h2 = add_layernorm(cur, a, blk.norm2)
                pend = blk.mlp(h2)
            cur, _ = add_layernorm(cur, pend, None)
            x = x.replace_feature(cur)
        else:
            for i, blk in enumerate(self.blocks):
                x = blk(x, None, plan=plans[i % 2], fuse_shell=self.fuse_shell)
        return self._finish(x, plans)

    def _finish(self, x, plans):
        if self.strict and not torch.cuda.is_current_stream_capturing():
            for p in plans:
                if p is not None:
                    p.raise_on_error()
        if self.downsample is not None:
            x = self.downsample(x)
        return x
