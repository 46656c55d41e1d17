#!/usr/bin/env python
"""Throughput of the sparse window-attention hot path on B200: voxels/s through W-MSA + SW-MSA.

One *step* = one W-MSA pass (no shift) followed by one SW-MSA pass (shift 3, with the shift mask)
over one synthetic room scene of 150 000 voxels (C = 96, 3 heads x 32, window 7^3): for each pass,
window bucketing from the raw voxel coordinates and the fused attention kernel.  Every voxel is
counted once per pass, so one step moves 2 * N voxels.  With --gpus N every rank works on its own
scene (seed = rank): weak scaling, no collective on the data path.

    python bench.py                       # 1 GPU, defaults
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8
    python bench.py --impl reference      # the CPU restatement of upstream, timed on the host cores

Prints one JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "voxels/sec through W-MSA+SW-MSA"
UNIT = "voxels/s"
N_VOX = 150_000
HEADS, HEAD_DIM, WINDOW, SHIFT = 3, 32, (7, 7, 7), (3, 3, 3)
C = HEADS * HEAD_DIM
# kernels of this library per pass: k_count, k_reduce, k_compact, k_order, k_scatter, then k_attn_fused
# (fp32) or k_attn_mma followed by k_attn_dense (bf16; the latter finds no window beyond a pack on the
# room and returns at once)
KERNELS_PER_PASS = {"f32": 6, "bf16": 7}
DOMINANT_KERNEL = {"f32": "k_attn_fused", "bf16": "k_attn_mma"}
# DRAM bytes one launch of the dominant kernel moves on this workload (dram__bytes_read.sum +
# dram__bytes_write.sum of the ncu captures summarised under profiles/).  Part of the output is still
# in L2 when the kernel ends, which is why the figure is below the algorithmic bytes.
NCU_TRAFFIC_BYTES = {"f32": 208_976_640, "bf16": 96_720_896}


def algorithmic_bytes_per_voxel(elt: int) -> int:
    """q, k, v rows in, out row out, int32 (window, pos) and one int32 permutation entry."""
    return 4 * C * elt + 12


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self, first: int = 0, last=None):
        """Samples [first, last): the ones delivered while the timed region ran."""
        rows = self.rows[first:last]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                for n, v in zip(names, r[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}  # region shorter than the period
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def room_variant(variant: int):
    """The benchmark room (seed 0) under the `variant`-th symmetry of its 400 x 400 floor plan (flips of
    the two long axes and their transposition: 8 scenes with different coordinates, the same voxel
    count and, within 0.4 %, the same window occupancies - sum c^2 1.767-1.773 M unshifted,
    1.681-1.698 M shifted - where rooms drawn from different seeds differ by up to 13 %).  Weak scaling
    wants the work per GPU fixed; rank r takes variant r % 8."""
    import numpy as np

    from sparseswin3d_b200 import scenes

    coords, dims = scenes.room_scene(N_VOX, seed=0)
    k = variant % 8
    a, b = coords[:, 1].copy(), coords[:, 2].copy()
    assert dims[0] == dims[1]
    if k & 4:
        a, b = b, a
    if k & 1:
        a = dims[0] - 1 - a
    if k & 2:
        b = dims[1] - 1 - b
    out = coords.copy()
    out[:, 1], out[:, 2] = a, b
    return np.ascontiguousarray(out), dims


def make_inputs(seed: int, dtype: torch.dtype, device, n_sets: int):
    coords, dims = room_variant(seed)
    g = torch.Generator().manual_seed(1000 + seed)
    qkv_host = [torch.randn(N_VOX, 3, HEADS, HEAD_DIM, generator=g).to(dtype).pin_memory() for _ in range(n_sets)]
    coords_host = torch.from_numpy(coords).pin_memory()
    table = (torch.randn((2 * WINDOW[0] - 1) ** 3, HEADS, generator=g) * 0.02).to(device)
    return coords_host, dims, qkv_host, table


class RoomSteps:
    """The step of the benchmark for one scene and one dtype on one GPU: buffers, the two plans'
    scratch, and one captured CUDA graph per rotating buffer set."""

    N_SETS = 4  # qkv/out sets; the two passes of a step use different sets, consecutive steps too

    def __init__(self, seed: int, dtype: torch.dtype, dev, host_qkv: bool = False):
        from sparseswin3d_b200 import _lib, attention, window

        self.dev, self.dtype = dev, dtype
        self.elt = torch.empty(0, dtype=dtype).element_size()
        self.coords_h, dims, self.qkv_h, self.table = make_inputs(seed, dtype, dev, self.N_SETS if host_qkv else 1)
        self.coords = self.coords_h.to(dev)
        if host_qkv:
            self.qkv = [q.to(dev) for q in self.qkv_h]
        else:  # device-side inputs are enough for the device-timed legs
            g = torch.Generator(device=dev).manual_seed(2000 + seed)
            self.qkv = [torch.randn(N_VOX, 3, HEADS, HEAD_DIM, device=dev, generator=g).to(dtype) for _ in range(self.N_SETS)]
        self.outs = [torch.empty(N_VOX, C, dtype=dtype, device=dev) for _ in range(self.N_SETS)]
        self.geoms = [window.resolve_geometry(1, dims, WINDOW, (0, 0, 0)), window.resolve_geometry(1, dims, WINDOW, SHIFT)]
        self.pp = attention.plan_params(HEADS, HEAD_DIM, dtype, WINDOW)
        L = _lib.PlanLayout()
        _lib.check(_lib.lib.ssw_plan_layout_init(L, N_VOX, self.geoms[0].n_windows, self.geoms[0].n_per_window,
                                                 self.pp["tile_rows"], int(self.pp["padded"])), "layout")
        self.layout = L
        # one scratch and one plan buffer per pass: the two plans of a step are built side by side
        self.scratch = [torch.empty(L.scratch_ints, dtype=torch.int32, device=dev) for _ in self.geoms]
        self.plan_buf = [torch.empty(L.plan_ints, dtype=torch.int32, device=dev) for _ in self.geoms]
        self.aux = torch.cuda.Stream(device=dev)
        self.scale = HEAD_DIM ** -0.5
        self.graphs = None
        self.last_plans = None

    def build_plan(self, i, coords=None, scratch=None, plan_buffer=None):
        from sparseswin3d_b200 import window

        return window.bucket_windows(coords=self.coords if coords is None else coords, geom=self.geoms[i],
                                     scratch=self.scratch[i] if scratch is None else scratch,
                                     plan_buffer=self.plan_buf[i] if plan_buffer is None else plan_buffer, **self.pp)

    def step(self, s):
        """W-MSA then SW-MSA.  Both plans depend on the coordinates only: the SW-MSA plan is built on
        a second stream while the first builds the W-MSA plan and runs W-MSA attention; SW-MSA
        attention waits for it.  (Fork and join are stream waits, so the same code captures into one
        graph.)  The two passes read and write different buffer sets."""
        from sparseswin3d_b200 import attention

        a, b = (2 * s) % self.N_SETS, (2 * s + 1) % self.N_SETS
        cur = torch.cuda.current_stream(self.dev)
        self.aux.wait_stream(cur)
        with torch.cuda.stream(self.aux):
            plan1 = self.build_plan(1)
        plan0 = self.build_plan(0)
        attention.window_attention_fused(self.qkv[a], plan0, self.table, self.scale, use_mask=False, out=self.outs[a])
        cur.wait_stream(self.aux)
        attention.window_attention_fused(self.qkv[b], plan1, self.table, self.scale, use_mask=True, out=self.outs[b])
        self.last_plans = (plan0, plan1)

    def capture(self):
        """The host side is Python: one step is about 14 launches, and enqueueing them from the
        interpreter is slower than the GPU runs them.  The product path for repeated steps is
        therefore one CUDA graph per step (captured once per buffer set, replayed)."""
        self.graphs = capture_graphs(self.step, self.N_SETS // 2, self.dev)

    def run(self, k):
        for i in range(k):
            self.graphs[i % len(self.graphs)].replay()

    def check(self):
        for plan in self.last_plans:
            err = plan.stats()["error"]
            if err:
                raise SystemExit(f"device error bits {err}")


def capture_graphs(fn, n, dev):
    side = torch.cuda.Stream(device=dev)
    graphs = []
    with torch.cuda.stream(side):
        for s in range(n):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                fn(s)
            graphs.append(g)
    torch.cuda.synchronize()
    return graphs


def timed_blocks(run, k, barrier, n_blocks):
    """Times `n_blocks` blocks of EXACTLY k steps, each bracketed by barrier + synchronize on both
    sides and timed with CUDA events on the launching stream.  Returns the block times in ms."""
    times = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(n_blocks):
        barrier()
        e0.record()
        run(k)
        e1.record()
        barrier()
        times.append(e0.elapsed_time(e1))
    return times


def time_graph(fn, reps, dev):
    g = capture_graphs(fn, 1, dev)[0]
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(7):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) / reps)
    return statistics.median(times)


def kernel_roofline(rs: RoomSteps, dtype_name: str):
    """The dominant kernel alone: a replayed graph of 12 back-to-back attention calls over rotating
    buffer sets and both plans; and the bucketing call alone the same way."""
    from sparseswin3d_b200 import attention, window

    plans = [window.bucket_windows(coords=rs.coords, geom=g, **rs.pp) for g in rs.geoms]
    torch.cuda.synchronize()
    reps = 12

    def attn_only(_):
        for i in range(reps):
            s = i % rs.N_SETS
            attention.window_attention_fused(rs.qkv[s], plans[i % 2], rs.table, rs.scale, use_mask=bool(i % 2), out=rs.outs[s])

    def bucket_only(_):
        for i in range(reps):
            window.bucket_windows(coords=rs.coords, geom=rs.geoms[i % 2], scratch=rs.scratch[0], plan_buffer=rs.plan_buf[0], **rs.pp)

    k_ms = time_graph(attn_only, reps, rs.dev)
    b_ms = time_graph(bucket_only, reps, rs.dev)
    peak, peak_src = measured_peak_gbs()
    alg_bytes = algorithmic_bytes_per_voxel(rs.elt) * N_VOX
    achieved = alg_bytes / (k_ms * 1e-3) / 1e9
    st = plans[0].stats()
    return {"bound": "hbm", "kernel": DOMINANT_KERNEL[dtype_name], "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "peak_source": peak_src, "frac_of_nominal_8000": achieved / 8000.0,
            "traffic": NCU_TRAFFIC_BYTES[dtype_name],
            "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of the ncu capture summarised under profiles/ "
                              "(not re-measured in this run)",
            "algorithmic_bytes": alg_bytes, "kernel_ms": k_ms, "bucketing_ms": b_ms,
            "timing": "CUDA events around a replayed CUDA graph of 12 back-to-back attention calls, median of 7"}, st


def crop_vs_upstream(dev):
    """The same-size anchor against upstream's own kernels: W-MSA + SW-MSA on the x,y < 200 corner of
    the scene (the largest piece inside upstream's int32 index domain), fp32: this library's step
    (bucketing from raw coordinates + fused attention) as a replayed graph, and its unfused operator
    chain (the compatibility path, enqueued from Python) - upstream's time for the same sample comes
    from the baseline leg."""
    from sparseswin3d_b200 import attention, window
    from sparseswin3d_b200.attention import WindowAttentionSparse

    c, dims, qkv, table = _cpu_sample()
    n = c.shape[0]
    coords, qkv_d, table_d = c.to(dev), qkv.to(dev), table.to(dev)
    geoms = [window.resolve_geometry(1, dims, WINDOW, (0, 0, 0)), window.resolve_geometry(1, dims, WINDOW, SHIFT)]
    pp = attention.plan_params(HEADS, HEAD_DIM, torch.float32, WINDOW)
    out = torch.empty(n, C, device=dev)
    plans = [window.bucket_windows(coords=coords, geom=g, **pp) for g in geoms]
    scr = torch.empty(max(p.layout.scratch_ints for p in plans), dtype=torch.int32, device=dev)
    buf = torch.empty(max(p.layout.plan_ints for p in plans), dtype=torch.int32, device=dev)

    def step(_):
        for g in geoms:
            plan = window.bucket_windows(coords=coords, geom=g, scratch=scr, plan_buffer=buf, **pp)
            attention.window_attention_fused(qkv_d, plan, table_d, HEAD_DIM ** -0.5, use_mask=bool(g.shifted), out=out)

    for _ in range(3):
        step(0)
    torch.cuda.synchronize()
    fused_ms = time_graph(step, 1, dev)
    # unfused chain through the module's operator path (upstream's forward on this library's ops)
    m = WindowAttentionSparse(C, HEADS, WINDOW).to(dev)  # for its relative_position_index and bias table
    passes = []
    for g in geoms:
        idx, region, _ = window.window_keys(coords, g, with_region=True)
        mask = None
        if g.shifted:  # compute_mask's table [nW, n] rebuilt from the per-voxel region ids
            mask = torch.zeros(g.n_windows, g.n_per_window, dtype=torch.int8, device=dev)
            mask[idx[:, 0].long(), idx[:, 1].long()] = region
        passes.append((idx, g.n_windows, g.n_per_window, mask))

    class _Chain(torch.nn.Module):
        def forward(self, idx, bw, npw, mask):
            from sparseswin3d_b200 import ops
            from sparseswin3d_b200.sparse_tensor import qkv_sparse_cuda, softmax_last_dim, sp_add_mask, sp_add_rpb, \
                spspmm_block_naive

            q, k_t, v = qkv_sparse_cuda(qkv_d, idx, bw, npw)
            attn = spspmm_block_naive(q * (HEAD_DIM ** -0.5), k_t, "q_k")
            bias = m.relative_position_bias_table[m.relative_position_index[:npw, :npw].reshape(-1)].reshape(npw, npw, -1)
            attn = sp_add_rpb(attn, bias.permute(2, 0, 1).contiguous())
            if mask is not None:
                attn = sp_add_mask(attn, mask)
            x_ = spspmm_block_naive(softmax_last_dim(attn), v, "qk_v").permute((0, 2, 1, 3))
            arg_sort = ops.return_inverse(ops.flatten_indices(idx.T.contiguous(), [bw, npw]), -1)[0]
            return x_.values.reshape(n, C).index_select(0, arg_sort)

    chain = _Chain()
    with torch.no_grad():
        for _ in range(2):
            for ps in passes:
                chain(*ps)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        reps = 5
        for _ in range(reps):
            for ps in passes:
                chain(*ps)
        torch.cuda.synchronize()
        chain_ms = (time.perf_counter() - t0) / reps * 1e3
    return {"voxels": n, "fused_step_ms": fused_ms, "fused_voxels_per_s": 2.0 * n / (fused_ms * 1e-3),
            "unfused_ops_chain_step_ms": chain_ms, "unfused_ops_chain_voxels_per_s": 2.0 * n / (chain_ms * 1e-3),
            "sample": "W-MSA + SW-MSA on the x,y<200 corner of the scene, fp32; fused = replayed CUDA graph of bucketing + "
                      "fused attention; unfused = this library's ten-operator surface driven from Python (wall clock)"}


def run_ours(args):
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # One clock sampler per job (rank 0's GPU), started now: nvidia-smi needs a moment to deliver its
    # first line.  Only samples that fall inside the timed region are reported.
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.__enter__()
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def all_ranks(x):
        """[world] list of a per-rank float."""
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        if world == 1:
            return [float(x)]
        out = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(out, t)
        return [float(o.item()) for o in out]

    def max_over_ranks(xs):
        t = torch.tensor(xs, dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    warm = max(args.warmup, 3)

    def measure(dtype_name, seed, primary):
        dtype = {"f32": torch.float32, "bf16": torch.bfloat16}[dtype_name]
        rs = RoomSteps(seed, dtype, dev, host_qkv=primary)
        for i in range(warm):  # eager warm-up (also builds every lazily initialised CUDA object before capture)
            rs.step(i)
        barrier()
        rs.check()
        rs.capture()
        rs.run(warm)
        barrier()
        # At least 10 blocks, and for the headline as many more as keep the GPU under this load for
        # 0.6 s, so that the clock sampler (0.1 s period) sees the region; the count is agreed between
        # the ranks (every block holds two barriers).
        calib = max(max_over_ranks([statistics.median(timed_blocks(rs.run, args.steps, barrier, 3))])[0], 1e-3)
        n_blocks = max(10, min(400, int(600.0 / calib) + 1)) if primary else 5
        if args.blocks > 0:
            n_blocks = args.blocks
        n0 = len(sampler.rows) if (sampler and primary) else 0
        blocks = timed_blocks(rs.run, args.steps, barrier, n_blocks)
        n1 = len(sampler.rows) if (sampler and primary) else 0
        rs.check()
        return rs, blocks, (n0, n1)

    # ---- timed region: blocks of K steps, device-timed, max over ranks per block ---------------
    rs, blocks, (n0, n1) = measure(args.dtype, rank, True)
    clk_summary = sampler.summary(n0, n1) if sampler else None
    if sampler:
        sampler.__exit__(None, None, None)
    n_blocks = len(blocks)
    job_blocks = max_over_ranks(blocks)                      # per block: the slowest rank
    ms = statistics.median(job_blocks)
    value = 2.0 * N_VOX * world * args.steps / (ms * 1e-3)
    per_rank_ms = all_ranks(statistics.median(blocks) / args.steps)

    roof, st = kernel_roofline(rs, args.dtype)
    elt = rs.elt

    # ---- end to end: host buffers in, host result out, through the public Python API ---------
    # Every step copies its coordinates and qkv from pinned host memory, runs both passes and copies
    # both results back to pinned host memory.  Two steps are in flight on two streams (each with its
    # own device buffers, scratch and captured graph), so the upload of one step overlaps the
    # download of the step before it: the link is full duplex and the copies are what bounds a step.
    from sparseswin3d_b200 import attention, window

    n_fly = 2
    e2e_streams = [torch.cuda.Stream(device=dev) for _ in range(n_fly)]
    out_h = [torch.empty(2, N_VOX, C, dtype=rs.dtype).pin_memory() for _ in range(n_fly)]
    c_d = [torch.empty_like(rs.coords) for _ in range(n_fly)]
    q_d = [torch.empty_like(rs.qkv[0]) for _ in range(n_fly)]
    o_d = [torch.empty(N_VOX, C, dtype=rs.dtype, device=dev) for _ in range(n_fly)]
    scr = [torch.empty(rs.layout.scratch_ints, dtype=torch.int32, device=dev) for _ in range(n_fly)]
    pbuf = [torch.empty(rs.layout.plan_ints, dtype=torch.int32, device=dev) for _ in range(n_fly)]

    def e2e_step(k):
        c_d[k].copy_(rs.coords_h, non_blocking=True)
        q_d[k].copy_(rs.qkv_h[k], non_blocking=True)
        for i, g in enumerate(rs.geoms):
            plan = rs.build_plan(i, coords=c_d[k], scratch=scr[k], plan_buffer=pbuf[k])
            o = attention.window_attention_fused(q_d[k], plan, rs.table, rs.scale, use_mask=bool(g.shifted), out=o_d[k])
            out_h[k][i].copy_(o, non_blocking=True)

    e2e_graphs = []
    for k in range(n_fly):
        with torch.cuda.stream(e2e_streams[k]):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=e2e_streams[k]):
                e2e_step(k)
            e2e_graphs.append(g)
    torch.cuda.synchronize()

    def e2e_run(n):
        for i in range(n):
            with torch.cuda.stream(e2e_streams[i % n_fly]):
                e2e_graphs[i % n_fly].replay()

    e2e_run(4)
    barrier()
    k_e2e = max(4, min(args.steps, 20))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_times = []
    for _ in range(5):
        barrier()
        e0.record(e2e_streams[0])
        e2e_run(k_e2e)
        for st_ in e2e_streams[1:]:
            e2e_streams[0].wait_stream(st_)
        e1.record(e2e_streams[0])
        barrier()
        e2e_times.append(e0.elapsed_time(e1))
    e2e_ms = statistics.median(max_over_ranks(e2e_times))
    e2e_value = 2.0 * N_VOX * world * k_e2e / (e2e_ms * 1e-3)
    h2d = rs.coords_h.numel() * 4 + rs.qkv_h[0].numel() * elt
    d2h = 2 * N_VOX * C * elt

    res = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": args.dtype, "data": "synthetic",
        "config": {"workload": "configs[1]: W-MSA + SW-MSA(shift 3, masked) on one synthetic 8x8x3 m room at 2 cm, "
                               f"{N_VOX} voxels per GPU, C=96, 3 heads x 32, window 7^3, bucketing + fused attention core "
                               "(qkv resident in HBM)",
                   "voxels_per_step_per_gpu": 2 * N_VOX, "windows": st["windows"], "sum_c2": st["sum_c2"],
                   "c_max": st["c_max"], "tile_rows": rs.pp["tile_rows"],
                   "l2": f"{rs.N_SETS} rotating qkv/out sets ({rs.N_SETS * roof['algorithmic_bytes'] / 1e6:.0f} MB) > 126 MB L2; "
                         "the two passes of a step and consecutive steps use different sets",
                   "parallelism": f"scene per GPU x{world}: rank r runs the seed-0 room under the r-th symmetry of its floor plan "
                                  "(distinct coordinates, equal work); control_same_scene: every rank on variant 0",
                   "launch": "one CUDA graph replay per step; the SW-MSA plan is built on a second stream beside the W-MSA pass"},
        "timing": {"blocks": n_blocks, "steps_per_block": args.steps, "block_ms_min": min(job_blocks),
                   "block_ms_median": ms, "block_ms_max": max(job_blocks),
                   "rule": "every block is exactly `steps` graph replays between barrier + synchronize, CUDA events on the "
                           "launching stream, max over ranks per block; value uses the median block"},
        "per_rank_ms_per_step": per_rank_ms,
        "clocks": clk_summary,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": k_e2e, "in_flight": n_fly},
        "gpu_launches": KERNELS_PER_PASS[args.dtype] * 2 * args.steps,
        "roofline": roof,
    }
    del e2e_graphs, out_h, c_d, q_d, o_d

    # ---- secondary lines (not the headline): the other dtype on the same step ------------------
    secondary = []
    if not args.no_secondary:
        other = "bf16" if args.dtype == "f32" else "f32"
        rs2, blocks2, _ = measure(other, rank, False)
        nb2 = len(blocks2)
        ms2 = statistics.median(max_over_ranks(blocks2))
        roof2, _ = kernel_roofline(rs2, other)
        secondary.append({"dtype": other, "value": 2.0 * N_VOX * world * args.steps / (ms2 * 1e-3), "unit": UNIT,
                          "ms_per_step": ms2 / args.steps, "blocks": nb2, "roofline": roof2})
        del rs2
        if world > 1:
            # control for the scaling loss: every rank runs the SAME scene (seed 0); what is left of the
            # spread between ranks is then not scene heterogeneity
            rs3, blocks3, _ = measure(args.dtype, 0, False)
            res["control_same_scene"] = {"per_rank_ms_per_step": all_ranks(statistics.median(blocks3) / args.steps),
                                         "job_ms_per_step": statistics.median(max_over_ranks(blocks3)) / args.steps}
            del rs3
    res["secondary"] = secondary
    if not args.no_secondary:
        res["shard"] = shard_lines(dev, rank, world)
        if rank == 0:
            try:
                res["stage"] = stage_line(dev, args.dtype, depth=6, reps=3)
            except Exception as e:
                res["stage"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    if world > 1:
        dist.barrier()
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            res["vs_upstream_gpu"] = crop_vs_upstream(dev)
            res["cpu_baseline"] = cpu_baseline(seconds=args.cpu_seconds)
            up = res["cpu_baseline"].get("upstream_gpu")
            if up and up.get("ms_per_step"):
                res["vs_upstream_gpu"]["upstream_step_ms"] = up["ms_per_step"]
                res["vs_upstream_gpu"]["ratio_fused"] = up["ms_per_step"] / res["vs_upstream_gpu"]["fused_step_ms"]
                res["vs_upstream_gpu"]["ratio_unfused_ops_chain"] = \
                    up["ms_per_step"] / res["vs_upstream_gpu"]["unfused_ops_chain_step_ms"]
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _gather_floats(x, dev, world):
    t = torch.tensor([float(x)], dtype=torch.float64, device=dev)
    if world == 1:
        return [float(x)]
    import torch.distributed as dist

    out = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return [float(o.item()) for o in out]


def skewed_shard(dev, rank, world, steps=10, warm=3, grid=126, dtype=torch.bfloat16):
    """One skewed-occupancy scene (window 9^3, half of the windows completely full, C = 192, 6 heads
    x 32) cut into contiguous window ranges over the ranks.  The cuts are computed once (outside
    the timed region: they depend on the coordinates only).  A timed pass is, on every rank:
    bucketing restricted to its range, the fused kernels on its windows storing every finished row
    into the output buffer of every rank, and a one-word all-reduce that closes the pass.  Strong
    scaling: the scene is fixed, so a single-GPU run of the same function is the base."""
    from sparseswin3d_b200 import attention, scenes, shard, window

    if world > 1:
        import torch.distributed as dist
    H, hd, W = 6, 32, (9, 9, 9)
    coords_np, dims = scenes.skewed_scene(grid=grid, window=9, p_dense=0.5, seed=0)
    n = coords_np.shape[0]
    coords = torch.from_numpy(coords_np).to(dev)
    g = torch.Generator(device=dev).manual_seed(1)
    qkv = torch.randn(n, 3, H, hd, device=dev, generator=g).to(dtype)
    table = torch.randn(17 ** 3, H, device=dev, generator=g) * 0.02
    geom = window.resolve_geometry(1, dims, W, (0, 0, 0))
    pp = attention.plan_params(H, hd, dtype, W)
    full = window.bucket_windows(coords=coords, geom=geom, **pp)
    st = full.stats()
    bounds = shard.plan_window_ranges(coords, geom, world, **pp)
    rows = shard.PeerRows(n, H * hd, dtype, dev)
    scratch = torch.empty(full.layout.scratch_ints, dtype=torch.int32, device=dev)
    pbuf = torch.empty(full.layout.plan_ints, dtype=torch.int32, device=dev)

    def step():
        return shard.sharded_window_attention(coords, qkv, geom, table, hd ** -0.5, W, rank, world, bounds, rows=rows,
                                              scratch=scratch, plan_buffer=pbuf)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(warm, 3)):
        res = step()
    barrier()
    err = int(res.error.item())
    own = res.plan.stats()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(5):
        barrier()
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        barrier()
        times.append(e0.elapsed_time(e1) / steps)
    mine = statistics.median(times)
    per_rank = _gather_floats(mine, dev, world)
    t = torch.tensor(times, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = statistics.median(t.tolist())
    # the sharded output against a single-GPU pass over the whole scene, computed here on this rank
    ref = attention.window_attention_fused(qkv, full, table, hd ** -0.5, use_mask=False)
    same = bool(torch.equal(ref, rows.local))
    same_all = min(_gather_floats(1.0 if same else 0.0, dev, world)) == 1.0
    flops = 4.0 * H * hd * st["sum_c2"]
    out = {"workload": f"one skewed-occupancy scene of {n} voxels, window 9^3, half of the windows full (729 voxels), C=192, "
                       "6 heads x 32, one W-MSA pass: bucketing of this rank's window range + fused attention with the "
                       "rows stored on every rank (peer stores over NVLink) + a one-word all-reduce",
           "scaling": "strong", "dtype": {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32"}[dtype],
           "voxels": n, "windows": st["windows"], "sum_c2": st["sum_c2"], "n_gpus": world,
           "ms_per_pass": ms, "per_rank_ms_per_pass": per_rank, "voxels_per_s": n / (ms * 1e-3),
           "tflops": flops / (ms * 1e-3) / 1e12, "window_id_bounds": list(bounds),
           "voxels_per_rank": [int(v) for v in _gather_floats(own["voxels"], dev, world)],
           "sum_c2_per_rank": [int(v) for v in _gather_floats(own["sum_c2"], dev, world)],
           "bitwise_equal_to_single_gpu_pass_on_every_rank": same_all, "error_word": err,
           "host_synchronisations_per_pass": 0, "collectives_per_pass": "one 4-byte all-reduce (max of the error words)"}
    barrier()
    rows.close()
    return out


def shard_lines(dev, rank, world):
    """Evidence for the window-range split of one scene: the strong-scaling time of the skewed
    10^6-voxel scene over the ranks of this run, with the output checked bit for bit against a
    single-GPU pass over the whole scene on every rank.  At one GPU it gives the base time."""
    try:
        return skewed_shard(dev, rank, world)
    except Exception as e:  # the headline must not be lost to its side line
        return {"unavailable": f"{type(e).__name__}: {e}"[:300]}


def run_skewed(args):
    """Secondary workload (not the default line): `skewed_shard` as the whole job."""
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    steps = max(1, min(args.steps, 20))
    with ClockSampler(local) as clk:
        sh = skewed_shard(dev, rank, world, steps=steps, warm=args.warmup, grid=args.skew_grid,
                          dtype={"bf16": torch.bfloat16, "f32": torch.float32}[args.dtype])
    peak = 1394.5
    try:
        peak = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops_sustained"])
    except Exception:
        pass
    res = {"metric": METRIC, "value": sh["voxels_per_s"], "unit": UNIT, "n_gpus": world, "steps": steps,
           "warmup": max(args.warmup, 3), "ms_per_step": sh["ms_per_pass"], "higher_is_better": True, "scaling": "strong",
           "vs_baseline": None, "dtype": sh["dtype"], "data": "synthetic",
           "config": {"workload": "configs[4]: " + sh["workload"], "parallelism": f"contiguous window ranges x{world}"},
           "clocks": clk.summary(), "shard": sh,
           "roofline": {"bound": "tensor", "achieved": sh["tflops"], "peak": peak * world, "unit": "TFLOP/s",
                        "frac": sh["tflops"] / (peak * world), "traffic": None,
                        "note": "flops = 4*C*sum c^2 (QK^T and P.V); the whole pass is timed, bucketing and the closing "
                                "all-reduce included; peak = measured sustained cuBLAS bf16 x GPUs"}}
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def stage_line(dev, dtype_name="f32", depth=6, reps=5):
    """A whole Swin stage on the benchmark room (150 000 voxels, C=96, 3 heads x 32, window 7^3):
    `depth` blocks alternating W-MSA and SW-MSA, each norm1 - qkv - attention core - proj - residual -
    norm2 - MLP - residual (the four Linears are library GEMMs).  Three forms of the same forward,
    each captured into a CUDA graph and replayed: the stage as built here (two plans per stage,
    one-pass add + LayerNorm), plans still shared but the shell as separate torch operations, and
    upstream's structure (every block buckets for itself, separate shell)."""
    from sparseswin3d_b200 import scenes, stage

    dtype = {"f32": torch.float32, "bf16": torch.bfloat16}[dtype_name]
    coords_np, dims = scenes.room_scene(N_VOX, seed=0)
    coords = torch.from_numpy(coords_np).to(dev)
    torch.manual_seed(0)
    layer = stage.BasicLayer(dim=C, depth=depth, num_heads=HEADS, window_size=WINDOW, qkv_bias=True).to(dev).to(dtype).eval()
    layer.strict = False
    g = torch.Generator(device=dev).manual_seed(3)
    feats = torch.randn(N_VOX, C, device=dev, generator=g).to(dtype)
    x = stage.SparseVoxels(feats, coords, dims, 1)
    out = {}
    ref = None
    for name, reuse, fuse in (("stage", True, True), ("shared_plans_torch_shell", True, False),
                              ("per_block_bucketing_torch_shell", False, False)):
        layer.reuse_plans, layer.fuse_shell = reuse, fuse
        with torch.no_grad():
            for _ in range(3):
                y = layer(x).features
            torch.cuda.synchronize()
            side = torch.cuda.Stream(device=dev)
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(gr, stream=side):
                    y = layer(x).features
        for _ in range(3):
            gr.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(4):
                gr.replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) / 4)
        ms = statistics.median(ts)
        if ref is None:
            ref = y.float().clone()
        dev_rel = float(((y.float() - ref).abs().max() / ref.abs().max()).item())
        out[name] = {"ms_per_forward": ms, "voxel_blocks_per_s": N_VOX * depth / (ms * 1e-3), "max_rel_dev_from_stage": dev_rel}
        del gr
    # the element-wise shell kernel alone: sum = a + b and norm = LayerNorm(sum) over rotating buffers
    # (4 sets > L2), algorithmic bytes 4 * C * elt per row (two rows in, two rows out)
    n_sets = 6 if dtype == torch.float32 else 10
    bufs = [(torch.randn(N_VOX, C, device=dev).to(dtype), torch.randn(N_VOX, C, device=dev).to(dtype),
             torch.empty(N_VOX, C, device=dev, dtype=dtype)) for _ in range(n_sets)]
    norm = layer.blocks[0].norm2

    def shell(_):
        for a_, b_, s_ in bufs:
            stage.add_layernorm(a_, b_, norm, sum_out=s_)

    sh_ms = time_graph(shell, n_sets, dev)
    sh_bytes = 4 * C * feats.element_size() * N_VOX
    peak, peak_src = measured_peak_gbs()
    out["add_layernorm_kernel"] = {"us": sh_ms * 1e3, "algorithmic_bytes": sh_bytes, "achieved_gbs": sh_bytes / (sh_ms * 1e-3) / 1e9,
                                   "frac": sh_bytes / (sh_ms * 1e-3) / 1e9 / peak, "peak": peak, "peak_source": peak_src,
                                   "l2": f"{n_sets} rotating sets of {sh_bytes / 1e6:.0f} MB"}
    return {"workload": f"one Swin stage, depth {depth}, on the {N_VOX}-voxel room, C={C}, {HEADS} heads x {HEAD_DIM}, window 7^3, "
                        f"{dtype_name}; bucketing from raw coordinates inside every forward",
            "unit": "voxel-blocks/s", **out}


def conv_lines(dev, dtype_name="f32", cin=48):
    """The sparse convolutions around the stages on the benchmark room: a 3^3 submanifold convolution
    (cin -> cin), the 2^3 stride-2 patch merging (cin -> 2 cin) and its inverse.  Each is a rulebook
    (built once per coordinate set), a gather kernel of this library and a library GEMM; the gather
    is timed alone over rotating outputs and held against the HBM copy bandwidth (its algorithmic
    bytes: the gathered operand written once + the source rows read once)."""
    from sparseswin3d_b200 import scenes, sparse_conv, stage

    dtype = {"f32": torch.float32, "bf16": torch.bfloat16}[dtype_name]
    elt = torch.empty(0, dtype=dtype).element_size()
    coords_np, dims = scenes.room_scene(N_VOX, seed=0)
    coords = torch.from_numpy(coords_np).to(dev)
    g = torch.Generator(device=dev).manual_seed(5)
    x = stage.SparseVoxels(torch.randn(N_VOX, cin, device=dev, generator=g).to(dtype), coords, dims, 1)
    peak, peak_src = measured_peak_gbs()

    def timed(fn, reps=5):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts)

    out = {"workload": f"sparse convolutions on the {N_VOX}-voxel room ({dims[0]}x{dims[1]}x{dims[2]} cells), {dtype_name}, Cin={cin}"}
    with torch.no_grad():
        subm = sparse_conv.SubMConv3d(cin, cin, 3, bias=False, indice_key="s").to(dev).to(dtype)
        down = sparse_conv.SparseConv3d(cin, 2 * cin, 2, 2, bias=False, indice_key="d").to(dev).to(dtype)
        up = sparse_conv.SparseInverseConv3d(2 * cin, cin, 2, indice_key="d", bias=False).to(dev).to(dtype)
        rb_ms = timed(lambda: sparse_conv.subm_rulebook(x, 3), 3)
        rbd_ms = timed(lambda: sparse_conv.strided_rulebook(x, 2), 3)
        y = subm(x)
        yd = down(x)
        rb, rbd = x.indice_dict["s"], x.indice_dict["d"]
        # the kernels of the submanifold convolution alone, over rotating outputs larger than L2
        n_sets = 3
        k3 = 27
        sub = {"rulebook_ms": rb_ms, "forward_ms": timed(lambda: subm(x)), "active_neighbours_mean": float((rb.nbr >= 0).sum().item()) / N_VOX,
               "form": "pairs grouped by tap" if rb.seg else "dense gathered operand"}
        if rb.seg:
            slots = (k3 - 1) * rb.seg
            xp_sets = [torch.empty(slots, cin, dtype=dtype, device=dev) for _ in range(n_sets * 4)]
            gp_ms = timed(lambda: [_lib_check_gather(x.features, rb.pair_in, c_) for c_ in xp_sets]) / len(xp_sets)
            yp = torch.randn(slots, cin, device=dev).to(dtype)
            base = torch.randn(N_VOX, cin, device=dev).to(dtype)
            outs_ = [torch.empty(N_VOX, cin, dtype=dtype, device=dev) for _ in range(n_sets * 4)]
            n_pairs = int(rb.row_slots.shape[0])
            gp_bytes = (slots + n_pairs) * cin * elt + slots * 4    # every slot written, every pair's row read, the slot table

            def reduce_all():
                from sparseswin3d_b200._lib import check, dtype_code, lib, ptr, stream_ptr
                for o_ in outs_:
                    check(lib.ssw_gather_reduce(ptr(base), ptr(yp), dtype_code(dtype), slots, ptr(rb.row_start), ptr(rb.row_slots),
                                                n_pairs, N_VOX, cin, ptr(o_), stream_ptr(dev)), "ssw_gather_reduce")

            gr_ms = timed(reduce_all) / len(outs_)
            gr_bytes = (2 * N_VOX + n_pairs) * cin * elt + (N_VOX + n_pairs) * 4   # base in, out, the pairs' rows, the row lists
            sub.update({"pair_slots": slots, "pairs": n_pairs, "dense_operand_rows": k3 * N_VOX,
                        "gather_pairs_kernel": {"ms": gp_ms, "algorithmic_bytes": gp_bytes, "gbs": gp_bytes / (gp_ms * 1e-3) / 1e9,
                                                "frac_of_hbm": gp_bytes / (gp_ms * 1e-3) / 1e9 / peak},
                        "gather_reduce_kernel": {"ms": gr_ms, "algorithmic_bytes": gr_bytes, "gbs": gr_bytes / (gr_ms * 1e-3) / 1e9,
                                                 "frac_of_hbm": gr_bytes / (gr_ms * 1e-3) / 1e9 / peak}})
            del xp_sets, outs_
        cols_sets = [torch.empty(N_VOX, k3 * cin, dtype=dtype, device=dev) for _ in range(n_sets)]
        g_ms = timed(lambda: [_lib_check_gather(x.features, rb.nbr, c_) for c_ in cols_sets]) / n_sets
        g_bytes = (k3 * cin + cin) * elt * N_VOX
        sub["dense_operand_gather_kernel"] = {"ms": g_ms, "algorithmic_bytes": g_bytes, "gbs": g_bytes / (g_ms * 1e-3) / 1e9,
                                              "frac_of_hbm": g_bytes / (g_ms * 1e-3) / 1e9 / peak}
        del cols_sets
        out["subm_3x3x3"] = sub
        out["strided_2x2x2"] = {"rulebook_ms": rbd_ms, "forward_ms": timed(lambda: down(x)), "output_voxels": int(yd.features.shape[0])}
        out["inverse_2x2x2"] = {"forward_ms": timed(lambda: up(yd))}
    out["peak"] = peak
    out["peak_source"] = peak_src
    return out


def _lib_check_gather(x, nbr, cols):
    from sparseswin3d_b200._lib import check, dtype_code, lib, ptr, stream_ptr

    check(lib.ssw_gather_cols(ptr(x), dtype_code(x.dtype), x.shape[0], nbr.shape[0], nbr.shape[1], x.shape[1], ptr(nbr), ptr(cols),
                              stream_ptr(x.device)), "ssw_gather_cols")


def run_conv(args):
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    res = {"metric": "sparse convolutions around the stages", "n_gpus": 1, "data": "synthetic",
           "lines": [conv_lines(dev, dt, cin) for dt in ("f32", "bf16") for cin in (48, 96)]}
    print(json.dumps(res), flush=True)


def run_stage(args):
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    res = {"metric": "voxel-blocks/sec through one Swin stage", "n_gpus": 1, "data": "synthetic",
           "lines": [stage_line(dev, dt, depth) for dt in ("f32", "bf16") for depth in (2, 6)]}
    print(json.dumps(res), flush=True)


# ------------------------------------------------------------------------------------------------
# CPU legs: the oracle (a PyTorch CPU restatement of upstream; upstream itself has no CPU path)
# ------------------------------------------------------------------------------------------------
def _cpu_sample(seed: int = 0, crop: int = 200):
    """A bounded sample of the workload: the x,y < `crop` corner of the room (about a quarter of the
    voxels), small enough for upstream's int32 index hash (B_w*H*n*hd < 2^31) to be valid."""
    from sparseswin3d_b200 import scenes

    coords, dims = scenes.room_scene(N_VOX, seed=seed)
    keep = (coords[:, 1] < crop) & (coords[:, 2] < crop)
    c = torch.from_numpy(coords[keep].copy())
    g = torch.Generator().manual_seed(1000 + seed)
    qkv = torch.randn(c.shape[0], 3, HEADS, HEAD_DIM, generator=g)
    table = torch.randn((2 * WINDOW[0] - 1) ** 3, HEADS, generator=g) * 0.02
    return c, (crop, crop, dims[2]), qkv, table


def _cpu_step(O, c, dims, qkv, table, rpi):
    for shift in ((0, 0, 0), SHIFT):
        idx, Bw, n, ws, ss, dp = O.window_keys(c, 1, dims, WINDOW, shift)
        mask = O.compute_mask(dp, ws, ss) if any(ss) else None
        O.window_attention_core(qkv, idx, Bw, n, HEAD_DIM ** -0.5, table, rpi, mask)


def cpu_baseline(seconds: float = 15.0):
    from oracle import ssw_oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    c, dims, qkv, table = _cpu_sample()
    rpi = O.relative_position_index(WINDOW)
    t0 = time.perf_counter()
    n = 0
    while True:
        _cpu_step(O, c, dims, qkv, table, rpi)
        n += 1
        if time.perf_counter() - t0 > seconds or n >= 5:
            break
    dt = time.perf_counter() - t0
    res = {"value": 2.0 * c.shape[0] * n / dt, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
           "sample": f"{n} step(s) of W-MSA+SW-MSA on the x,y<200 corner of the scene ({c.shape[0]} voxels, fp32), "
                     "oracle/ssw_oracle.py on torch CPU"}
    # beside the CPU number: upstream's own CUDA extension on the same sample, where it was built
    up = _upstream_on_gpu(O, c, dims, qkv, table, rpi)
    if up is not None:
        res["upstream_gpu"] = up
    return res


def _upstream_on_gpu(O, c, dims, qkv, table, rpi, reps: int = 5):
    """Extra information beside the CPU number: upstream's own CUDA extension (built unmodified into
    oracle/_ref/ where the upstream sources were available), driven through the same two passes on
    the same sample, on cuda:0.  None when there is no GPU or no such build."""
    try:
        if not torch.cuda.is_available():
            return None
        from oracle import upstream_chain
        from oracle.build_ref import load_ref

        ref = load_ref()
        if ref is None:
            return None
        dev = torch.device("cuda:0")
        passes = []
        for shift in ((0, 0, 0), SHIFT):
            idx, Bw, n, ws, ss, dp = O.window_keys(c, 1, dims, WINDOW, shift)
            mask = O.compute_mask(dp, ws, ss).to(dev) if any(ss) else None
            passes.append((idx.to(dev), Bw, n, mask))
        qkv_d, table_d, rpi_d = qkv.to(dev), table.to(dev), rpi.to(dev)

        def step():
            for idx, Bw, n, mask in passes:
                upstream_chain.forward(ref, idx, qkv_d, Bw, n, HEAD_DIM ** -0.5, table_d, rpi_d, mask)

        for _ in range(2):
            step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            step()
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / reps
        return {"value": 2.0 * c.shape[0] / dt, "unit": UNIT, "ms_per_step": dt * 1e3,
                "sample": f"upstream ops.cu, unmodified, on cuda:0: W-MSA+SW-MSA attention core (qkv given, window "
                          f"indices and mask given) on the same {c.shape[0]}-voxel sample, wall clock over {reps} steps"}
    except Exception as e:  # informational only
        return {"unavailable": f"{type(e).__name__}: {e}"[:200]}


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    from oracle import ssw_oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    c, dims, qkv, table = _cpu_sample()
    rpi = O.relative_position_index(WINDOW)
    steps = max(1, min(args.steps, 5))
    warm = 1
    for _ in range(warm):
        _cpu_step(O, c, dims, qkv, table, rpi)
    t0 = time.perf_counter()
    for _ in range(steps):
        _cpu_step(O, c, dims, qkv, table, rpi)
    dt = time.perf_counter() - t0
    v = 2.0 * c.shape[0] * steps / dt
    sample = (f"each step = W-MSA+SW-MSA on the x,y<200 corner of the scene ({c.shape[0]} voxels, fp32); upstream has no "
              "CPU path and its CUDA extension needs a GPU, so this is oracle/ssw_oracle.py (a PyTorch CPU restatement)")
    upstream_gpu = _upstream_on_gpu(O, c, dims, qkv, table, rpi)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "configs[1] (bounded sample): W-MSA + SW-MSA on a synthetic room, C=96, 3 heads x 32, "
                               "window 7^3", "voxels_per_step": 2 * c.shape[0]},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "upstream_gpu": upstream_gpu,
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="f32", choices=["f32", "bf16"])
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary measurements (other dtype, "
                                                               "same-scene control, window-range shard lines)")
    ap.add_argument("--skew-grid", type=int, default=126,
                    help="edge of the skewed scene's grid in voxels (126 = the 10^6-voxel scene; smaller for profiler captures)")
    ap.add_argument("--workload", default="room", choices=["room", "skewed", "stage", "conv"],
                    help="room: the default line (W-MSA + SW-MSA on a 150k-voxel room); skewed: one 10^6-voxel "
                         "skewed-occupancy scene sharded by window ranges (secondary)")
    ap.add_argument("--blocks", type=int, default=0,
                    help="timed blocks of `steps` steps (0: at least 10 and enough for 0.6 s under load)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "skewed":
        run_skewed(args)
    elif args.workload == "stage":
        run_stage(args)
    elif args.workload == "conv":
        run_conv(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
