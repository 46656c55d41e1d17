"""Drive the UNMODIFIED upstream extension (oracle/_ref/custom_ops.so) through the forward of
WindowAttentionSparse, the way upstream's own Python does.

TEST / MEASUREMENT INFRASTRUCTURE ONLY: nothing in the product package imports this file.

`sparse_swin/swin3d_base.py` cannot be imported without spconv and pointcept, so the few lines of
glue it has between its native operators (swin3d_base.py:483-498, 557-581, 659-675) are restated
here with torch ops on the device; every operator call goes to upstream's own compiled code.
"""
from __future__ import annotations

import torch


def forward(ref, idx, qkv, Bw, n, scale, table, rpi, mask):
    """idx [N,2] int32 (window,pos), qkv [N,3,H,hd], table [(2W-1)^3,H], rpi [n,n], mask [nW,n] int8 or
    None; all on the device.  Returns out [N, H*hd] in the caller's voxel order."""
    H, hd = qkv.shape[2], qkv.shape[3]
    iqv, pqv, ik, pk = ref.qkv_sparse_indices(idx, Bw, n, H, hd)           # :483-498
    iq, ikk = iqv.index_select(1, pqv), ik.index_select(1, pk)
    q_v = qkv[:, 0].reshape(-1).index_select(0, pqv) * scale               # :660
    k_v = qkv[:, 1].reshape(-1).index_select(0, pk)
    v_v = qkv[:, 2].reshape(-1).index_select(0, pqv)
    qs, ks = [Bw, H, n, hd], [Bw, H, hd, n]
    a_idx, a_val, a_shape, _ = ref.matmul_cuda_naive(q_v, iq, qs, k_v, ikk, ks, "q_k")   # :661
    bias = table[rpi[:n, :n].reshape(-1)].reshape(n, n, -1).permute(2, 0, 1).contiguous()  # :662-666
    ai = a_idx.long()
    a_val = a_val + bias.view(-1).index_select(0, ai[1] * n * n + ai[2] * n + ai[3])      # :557-566
    if mask is not None:                                                                   # :569-581
        w = ai[0] % mask.shape[0]
        d = mask.view(-1).index_select(0, w * n + ai[3]) - mask.view(-1).index_select(0, w * n + ai[2])
        d = d.to(a_val.dtype)
        d.masked_fill_(d != 0, -100)
        a_val = a_val + d
    rows = ref.unique_consecutive_indices(ref.flatten_indices(a_idx[:3].contiguous(), a_shape[:-1]))  # :161-197
    sm = ref.softmax_last_dim_forward(rows, a_val.float())
    x_idx, x_val, x_shape, _ = ref.matmul_cuda_naive(sm, a_idx, a_shape, v_v, iq, qs, "qk_v")          # :672
    dims = [0, 2, 1, 3]                                                                                 # :673
    order = ref.sort_indices(ref.flatten_indices(x_idx[dims, :].contiguous(), [x_shape[d] for d in dims]))
    x_perm = x_val.index_select(0, order)
    arg_sort, _ = ref.return_inverse(ref.flatten_indices(idx.T.contiguous(), [Bw, n]), -1)             # :674-675
    return x_perm.reshape(qkv.shape[0], H * hd).index_select(0, arg_sort)
