"""Parity at the full sizes of the benchmark configurations, through size-independent properties.

The oracle cannot run 150 000 to 1 000 000 voxels in seconds, so at full size the tests check
  * the window plan bit for bit against a numpy sort of the same keys (cheap at any size),
  * the attention output on a random sample of whole windows against the oracle's dense
    per-window reference (attention is block diagonal: a window's rows depend on that window only),
  * that every row was written (no row keeps the sentinel the output buffer was filled with).
"""
import numpy as np
import pytest
import torch

from oracle import ssw_oracle as O
from tests.cases import rel_err

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
BF16_TOL = 2e-2


def _check_sampled(coords_np, dims, window, shift, heads, hd, dtype, tol, n_sample, seed):
    from sparseswin3d_b200 import attention, window as W

    dev = torch.device("cuda:0")
    coords = torch.from_numpy(coords_np)
    N = coords.shape[0]
    idx, Bw, n, ws, ss, dp = O.window_keys(coords, 1, dims, window, shift)
    mask = O.compute_mask(dp, ws, ss) if any(s > 0 for s in ss) else None
    geom = W.resolve_geometry(1, dims, window, shift)
    plan = W.bucket_windows(coords=coords.to(dev), geom=geom, **attention.plan_params(heads, hd, dtype, window))
    st = plan.stats()
    assert st["error"] == 0 and st["voxels"] == N

    # plan: sorted order, inverse permutation, window table -- bit exact against numpy
    key = idx[:, 0].numpy().astype(np.int64) * n + idx[:, 1].numpy()
    order = np.argsort(key, kind="stable")
    assert np.array_equal(plan.perm.cpu().numpy(), order)
    inv = np.empty(N, dtype=np.int64)
    inv[order] = np.arange(N)
    assert np.array_equal(plan.inv_perm.cpu().numpy(), inv)
    wins, counts = np.unique(idx[:, 0].numpy(), return_counts=True)
    assert st["windows"] == wins.size
    assert np.array_equal(plan.win_id[: wins.size].cpu().numpy(), wins)
    assert np.array_equal(plan.occupancy().cpu().numpy(), counts)
    assert st["sum_c2"] == int((counts.astype(np.int64) ** 2).sum())
    assert np.array_equal(np.sort(plan.pack_perm.cpu().numpy()), np.arange(N))

    g = torch.Generator().manual_seed(seed)
    qkv = torch.randn(N, 3, heads, hd, generator=g).to(dtype)
    table = torch.randn((2 * window[0] - 1) * (2 * window[1] - 1) * (2 * window[2] - 1), heads, generator=g) * 0.5
    out = torch.full((N, heads * hd), float("nan"), dtype=dtype, device=dev)
    attention.window_attention_fused(qkv.to(dev), plan, table.to(dev), hd ** -0.5, use_mask=mask is not None, out=out)
    assert plan.stats()["error"] == 0
    out = out.float().cpu()
    assert not torch.isnan(out).any()  # every voxel row was written

    # a sample of whole windows, weighted towards the large ones as well as the small ones
    rng = np.random.default_rng(seed)
    big = wins[np.argsort(counts)[-max(2, n_sample // 10):]]
    pick = np.unique(np.concatenate([rng.choice(wins, size=min(n_sample, wins.size), replace=False), big]))
    rows = torch.from_numpy(np.nonzero(np.isin(idx[:, 0].numpy(), pick))[0])
    ref = O.dense_window_attention(qkv[rows].float(), idx[rows], hd ** -0.5, table, O.relative_position_index(window), mask)
    assert rel_err(out[rows], ref) <= tol
    return st


@pytest.mark.parametrize("shift", [(0, 0, 0), (3, 3, 3)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, FP32_TOL), (torch.bfloat16, BF16_TOL)])
def test_room_150k(shift, dtype, tol):
    """The benchmark's own workload: 150 000-voxel room, C = 96, 3 heads x 32, window 7^3."""
    from sparseswin3d_b200 import scenes

    coords, dims = scenes.room_scene(150_000, seed=0)
    st = _check_sampled(coords, dims, (7, 7, 7), shift, 3, 32, dtype, tol, n_sample=400, seed=11)
    assert st["voxels"] == 150_000


@pytest.mark.parametrize("stage,heads,hd", [
    (0, 3, 16), (1, 6, 16), (2, 12, 16), (3, 24, 16),   # C = 48 / 96 / 192 / 384 with 3 / 6 / 12 / 24 heads
    (1, 6, 32), (2, 12, 32), (3, 24, 32),               # the same head counts at head_dim 32 (C up to 768)
])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, FP32_TOL), (torch.bfloat16, BF16_TOL)])
def test_swin_stage_sweep(stage, heads, hd, dtype, tol):
    """Swin stages of the same scene: coordinates downsampled by 2 per stage (150 k / 40 k / 10 k /
    2.5 k voxels), 3 / 6 / 12 / 24 heads, shifted and masked.  The stage table is stated both with
    C = 48 ... 384 (head_dim 16) and with head_dim 32; both readings are covered.  (Stage 0 at
    3 heads x 32 is test_room_150k.)"""
    from sparseswin3d_b200 import scenes

    coords, dims = scenes.room_scene(150_000, seed=0)
    for _ in range(stage):
        coords, dims = scenes.downsample_scene(coords, dims)
    _check_sampled(coords, dims, (7, 7, 7), (3, 3, 3), heads, hd, dtype, tol, n_sample=300, seed=20 + stage)


def test_skewed_one_million_bf16():
    """Skewed-occupancy stress scene at full size: about 10^6 voxels, window 9^3, half of the
    windows completely full (729 voxels), C = 192, 6 heads x 32, bf16."""
    from sparseswin3d_b200 import scenes

    coords, dims = scenes.skewed_scene(grid=126, window=9, p_dense=0.5, seed=0)
    st = _check_sampled(coords, dims, (9, 9, 9), (0, 0, 0), 6, 32, torch.bfloat16, BF16_TOL, n_sample=60, seed=31)
    assert st["c_max"] == 729 and st["voxels"] > 900_000


def test_single_forward_20k_uniform_fp32():
    """The CPU-runnable configuration as stated: 20 000 unique voxels uniform in a 128^3 grid
    (seed 0), fp32 features ~N(0,1), C = 96, 3 heads x 32, window 7^3, no shift, Xavier-uniform qkv
    weights (seed 1).  This size lies inside upstream's int32 index domain, so the oracle runs
    upstream's whole operator chain; compared are the per-voxel output of the module and the COO
    softmax values."""
    from sparseswin3d_b200 import attention, window

    dev = torch.device("cuda:0")
    C, H, hd, W, grid, N = 96, 3, 32, (7, 7, 7), 128, 20_000
    rng = np.random.default_rng(0)
    flat = rng.choice(grid ** 3, size=N, replace=False)
    z, y, x = np.unravel_index(flat, (grid, grid, grid))
    coords = torch.from_numpy(np.stack([np.zeros_like(z), z, y, x], 1).astype(np.int32))
    g = torch.Generator().manual_seed(0)
    feats = torch.randn(N, C, generator=g)
    torch.manual_seed(1)
    m = attention.WindowAttentionSparse(C, H, W, qkv_bias=True)
    torch.nn.init.xavier_uniform_(m.qkv.weight)
    torch.nn.init.xavier_uniform_(m.proj.weight)
    torch.nn.init.normal_(m.relative_position_bias_table, std=0.02)
    idx, Bw, n, ws, ss, dp = O.window_keys(coords, 1, (grid,) * 3, W, (0, 0, 0))
    assert Bw * H * n * hd < 2 ** 31
    with torch.no_grad():
        ref_out, ref_core, ref_attn = O.window_attention_forward(
            feats, idx, Bw, n, H, m.qkv.weight, m.qkv.bias, m.proj.weight, m.proj.bias,
            m.relative_position_bias_table, O.relative_position_index(W), None)
        m = m.to(dev)
        geom = window.resolve_geometry(1, (grid,) * 3, W, (0, 0, 0))
        plan = window.bucket_windows(coords=coords.to(dev), geom=geom, **attention.plan_params(H, hd, torch.float32, W))
        qkv = m.qkv(feats.to(dev)).reshape(N, 3, H, hd)
        core, attn = attention.window_attention_fused(qkv, plan, m.relative_position_bias_table, m.scale,
                                                      use_mask=False, return_attn=True)
        out = m.proj(core)
    assert plan.stats()["error"] == 0
    # the Linear layers run in cuBLAS on the device and in the CPU BLAS for the oracle: their own
    # rounding differences (1e-6) pass through the attention
    assert rel_err(core.cpu(), ref_core) <= 2e-5
    assert rel_err(out.cpu(), ref_out) <= 2e-5
    assert attn.numel() == ref_attn.values.numel()
    assert rel_err(attn.cpu(), ref_attn.values) <= 2e-5


DIGESTS = sorted((__import__("pathlib").Path(__file__).parent / "golden").glob("digest_*.npz"))


@pytest.mark.parametrize("path", DIGESTS, ids=[p.stem for p in DIGESTS])
def test_room_crop_against_upstream_digest(path):
    """The CUDA path against the unmodified upstream extension on the x,y<200 corner of the benchmark
    room (35 935 voxels, 1.2 M scores), through the stored digest: the operator chain's index arrays
    by checksum (bit exact), its value arrays by their sums, the fused kernel's output and COO
    softmax values on the sampled rows / positions."""
    from sparseswin3d_b200 import attention, ops, window
    from tests.cases import digest_i64, room_crop_case

    dev = torch.device("cuda:0")
    d = dict(np.load(path))
    case = room_crop_case(shift=tuple(d["in_shift"].tolist()))
    idx, qkv = case["indices"].to(dev), case["qkv"].to(dev)
    Bw, n, H, hd = case["n_windows"], case["n"], case["heads"], case["head_dim"]

    def same(a, key):
        assert a.dtype == torch.int32 and a.numel() == int(d["len_" + key]), key
        assert digest_i64(a.cpu().numpy()) == int(d["crc_" + key]), key

    def sums(x, key):
        x = x.double()
        assert abs(float(x.abs().sum()) - float(d["abs_" + key])) <= 1e-5 * float(d["abs_" + key]), key
        assert abs(float(x.sum()) - float(d["sum_" + key])) <= 1e-5 * float(d["abs_" + key]), key

    # operator chain
    iqv, pqv, ik, pk = ops.qkv_sparse_indices(idx, Bw, n, H, hd)
    for a, k in ((iqv, "idx_qv"), (pqv, "perm_qv"), (ik, "idx_k"), (pk, "perm_k")):
        same(a, k)
    iq, ikk = iqv.index_select(1, pqv), ik.index_select(1, pk)
    q_v = qkv[:, 0].reshape(-1).index_select(0, pqv) * case["scale"]
    k_v = qkv[:, 1].reshape(-1).index_select(0, pk)
    v_v = qkv[:, 2].reshape(-1).index_select(0, pqv)
    a_idx, a_val, a_shape, c = ops.matmul_cuda_naive(q_v, iq, [Bw, H, n, hd], k_v, ikk, [Bw, H, hd, n], "q_k")
    same(a_idx, "qk_idx"), same(c, "c"), sums(a_val, "qk_val")
    arg_sort, _ = ops.return_inverse(ops.flatten_indices(idx.T.contiguous(), [Bw, n]), -1)
    same(arg_sort, "arg_sort")

    # fused kernel
    geom = window.resolve_geometry(1, case["dims"], case["window"], case["shift"])
    plan = window.bucket_windows(coords=case["coords"].to(dev), geom=geom, **attention.plan_params(H, hd, torch.float32))
    out, attn = attention.window_attention_fused(qkv, plan, case["table"].to(dev), case["scale"],
                                                 use_mask=case["mask"] is not None, return_attn=True)
    assert plan.stats()["error"] == 0
    assert torch.equal(plan.inv_perm, arg_sort)
    sums(out, "out"), sums(attn, "softmax")
    rows = torch.from_numpy(d["sample_rows"]).to(dev)
    assert rel_err(out[rows].cpu(), torch.from_numpy(d["sample_out"])) <= FP32_TOL
    pos = torch.from_numpy(d["sample_pos"]).to(dev)
    assert torch.equal(a_idx[:, pos].cpu(), torch.from_numpy(d["sample_qk_idx"]))
    assert rel_err(attn[pos].cpu(), torch.from_numpy(d["sample_softmax"])) <= FP32_TOL
