"""Generate the golden fixtures in this directory by running the UNMODIFIED upstream extension.

Needs a CUDA device and ``oracle/_ref/custom_ops.so`` (built by ``oracle/build_ref.py`` from the
upstream sources).  For three small seeded cases it drives upstream's ten ops exactly the way
``WindowAttentionSparse.forward`` and the two autograd Functions do (sparse_swin/swin3d_base.py:
68-197, 483-498, 557-581, 654-675; that file itself cannot be imported without spconv/pointcept, so
its few lines of glue between the ops are restated here with torch ops on the GPU) and stores every
intermediate as ``<case>.npz``.

    python tests/golden/make_golden.py [outdir]      # default: this directory
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle.build_ref import load_ref  # noqa: E402
from tests.cases import digest_i64, make_case, room_crop_case  # noqa: E402

# Larger cases are stored as digests: checksums of every index array, sums of every value array and
# a fixed sample of output rows and softmax values (inputs are regenerated from their seeds).
DIGEST_CASES = {
    "room_crop_wmsa": dict(shift=(0, 0, 0)),
    "room_crop_swmsa": dict(shift=(3, 3, 3)),
}
INT_KEYS = ("idx_qv", "perm_qv", "idx_k", "perm_k", "qk_idx", "c", "softmax_rows", "pv_idx", "c_pv", "permute_order",
            "arg_sort")
VAL_KEYS = ("qk_val", "pre_softmax", "softmax", "pv_val", "out")
N_SAMPLE = 512


def digest_of(res):
    rng = np.random.default_rng(5)
    d = {}
    for k in INT_KEYS:
        d["crc_" + k] = np.array(digest_i64(res[k]), dtype=np.int64)
        d["len_" + k] = np.array(res[k].size, dtype=np.int64)
    for k in VAL_KEYS:
        v = res[k].astype(np.float64)
        d["sum_" + k] = np.array(v.sum())
        d["abs_" + k] = np.array(np.abs(v).sum())
    rows = np.sort(rng.choice(res["out"].shape[0], size=N_SAMPLE, replace=False))
    d["sample_rows"] = rows.astype(np.int64)
    d["sample_out"] = res["out"][rows]
    pos = np.sort(rng.choice(res["softmax"].size, size=8 * N_SAMPLE, replace=False))
    d["sample_pos"] = pos.astype(np.int64)
    d["sample_softmax"] = res["softmax"][pos]
    d["sample_qk_idx"] = res["qk_idx"][:, pos]
    return d


CASES = {
    "wmsa_h3_hd32": dict(n_vox=100, grid=16, heads=3, head_dim=32, shift=(0, 0, 0), seed=11),
    "swmsa_h3_hd32": dict(n_vox=100, grid=16, heads=3, head_dim=32, shift=(3, 3, 3), seed=12),
    "swmsa_h2_hd16_dense": dict(n_vox=160, grid=14, heads=2, head_dim=16, shift=(3, 3, 3), seed=13),
}


def run_case(ref, case, dev):
    H, hd, Bw, n = case["heads"], case["head_dim"], case["n_windows"], case["n"]
    idx = case["indices"].to(dev)
    qkv = case["qkv"].to(dev)
    out = {}
    # qkv_sparse_cuda (swin3d_base.py:483-498)
    iqv, pqv, ik, pk = ref.qkv_sparse_indices(idx, Bw, n, H, hd)
    iq, ikk = iqv.index_select(1, pqv), ik.index_select(1, pk)
    q_v = qkv[:, 0].reshape(-1).index_select(0, pqv) * case["scale"]  # :660
    k_v = qkv[:, 1].reshape(-1).index_select(0, pk)
    v_v = qkv[:, 2].reshape(-1).index_select(0, pqv)
    out.update(idx_qv=iqv, perm_qv=pqv, idx_k=ik, perm_k=pk)
    qs, ks = [Bw, H, n, hd], [Bw, H, hd, n]
    # q_k (:661)
    a_idx, a_val, a_shape, c1 = ref.matmul_cuda_naive(q_v, iq, qs, k_v, ikk, ks, "q_k")
    out.update(qk_idx=a_idx, qk_val=a_val, qk_shape=torch.tensor(a_shape), c=c1)
    # sp_add_rpb (:557-566, :662-666)
    bias = case["table"].to(dev)[case["rpi"].to(dev)[:n, :n].reshape(-1)].reshape(n, n, -1).permute(2, 0, 1).contiguous()
    ai = a_idx.long()
    a_val2 = a_val + bias.view(-1).index_select(0, ai[1] * n * n + ai[2] * n + ai[3])
    # sp_add_mask (:569-581)
    if case["mask"] is not None:
        m = case["mask"].to(dev)
        w = ai[0] % m.shape[0]
        d = m.view(-1).index_select(0, w * n + ai[3]) - m.view(-1).index_select(0, w * n + ai[2])
        d = d.to(a_val2.dtype)
        d.masked_fill_(d != 0, -100)
        a_val2 = a_val2 + d
    out["pre_softmax"] = a_val2
    # softmax_last_dim (:161-197)
    rows = ref.unique_consecutive_indices(ref.flatten_indices(a_idx[:3].contiguous(), a_shape[:-1]))
    sm = ref.softmax_last_dim_forward(rows, a_val2.float())
    out.update(softmax_rows=rows, softmax=sm)
    # qk_v (:672)
    x_idx, x_val, x_shape, c2 = ref.matmul_cuda_naive(sm, a_idx, a_shape, v_v, iq, qs, "qk_v")
    out.update(pv_idx=x_idx, pv_val=x_val, pv_shape=torch.tensor(x_shape), c_pv=c2)
    # permute((0,2,1,3)) (:47-59, :673)
    dims = [0, 2, 1, 3]
    t_shape = [x_shape[d] for d in dims]
    t_idx = x_idx[dims, :].contiguous()
    order = ref.sort_indices(ref.flatten_indices(t_idx, t_shape))
    out.update(permute_order=order)
    x_perm = x_val.index_select(0, order)
    # un-sort (:674-675)
    arg_sort, cnt = ref.return_inverse(ref.flatten_indices(idx.T.contiguous(), [Bw, n]), -1)
    out.update(arg_sort=arg_sort, arg_sort_count=torch.tensor(cnt))
    out["out"] = x_perm.reshape(qkv.shape[0], H * hd).index_select(0, arg_sort)
    # backward ops, driven as _spspmm_block_naive.backward / _softmax_last_dim.backward do (:106-138, :177-188)
    g = torch.Generator(device="cpu").manual_seed(99)
    g_pv = torch.randn(x_val.shape, generator=g).to(dev)
    out["g_pv"] = g_pv
    out["g_sm_from_pv"] = ref.matmul_grad_cuda_naive(g_pv, v_v, c2, hd, "rc_cr")
    sm_t = ref.qkv_transpose(sm, c2, hd, "rr")
    g_pv_t = ref.qkv_transpose(g_pv, c2, hd, "rc")
    out.update(sm_t=sm_t, g_pv_t=g_pv_t)
    out["g_v"] = ref.matmul_grad_cuda_naive(sm_t, g_pv_t, c2, hd, "rr_rc")
    out["g_pre_softmax"] = ref.softmax_last_dim_backward(rows, sm, out["g_sm_from_pv"])
    out["g_q"] = ref.matmul_grad_cuda_naive(out["g_pre_softmax"], k_v, c1, hd, "rr_rc")
    q_t = ref.qkv_transpose(q_v, c1, hd, "rc")
    g_a_t = ref.qkv_transpose(out["g_pre_softmax"], c1, hd, "rr")
    out["g_k"] = ref.matmul_grad_cuda_naive(q_t, g_a_t, c1, hd, "cr_rr")
    return {k: v.detach().cpu().numpy() for k, v in out.items()}


def main():
    outdir = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).resolve().parent
    outdir.mkdir(parents=True, exist_ok=True)
    ref = load_ref()
    if ref is None or not torch.cuda.is_available():
        raise SystemExit("needs oracle/_ref/custom_ops.so and a CUDA device")
    dev = torch.device("cuda:0")
    for name, kw in CASES.items():
        case = make_case(**kw)
        res = run_case(ref, case, dev)
        res.update(in_coords=case["coords"].numpy(), in_indices=case["indices"].numpy(), in_qkv=case["qkv"].numpy(),
                   in_table=case["table"].numpy(), in_dims=np.array(case["dims"]), in_shift=np.array(case["shift"]),
                   in_n_windows=np.array(case["n_windows"]), in_n=np.array(case["n"]),
                   in_mask=case["mask"].numpy() if case["mask"] is not None else np.zeros((0, 0), np.int8))
        np.savez_compressed(outdir / f"{name}.npz", **res)
        print(name, {k: v.shape for k, v in res.items() if k in ("qk_val", "out", "perm_qv")})
    for name, kw in DIGEST_CASES.items():
        case = room_crop_case(**kw)
        assert case["n_windows"] * case["heads"] * case["n"] * case["head_dim"] < 2 ** 31  # upstream's index domain
        res = run_case(ref, case, dev)
        d = digest_of(res)
        d.update(in_n_vox=np.array(case["coords"].shape[0]), in_shift=np.array(case["shift"]))
        np.savez_compressed(outdir / f"digest_{name}.npz", **d)
        print(name, case["coords"].shape[0], "voxels", res["qk_val"].size, "scores")


if __name__ == "__main__":
    main()
