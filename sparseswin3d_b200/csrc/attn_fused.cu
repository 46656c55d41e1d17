// Fused window attention for sparse voxel windows: QK^T, relative-position bias, shift mask,
// row softmax (upstream semantics: max starts at 0, denominator + 1e-8) and P.V in one kernel.
//
// CUDA-core path, one persistent CTA per SM, software-pipelined.  The plan's work items are
// either *packs* of windows that all hold exactly c voxels (c <= tile) or query tiles of a window
// with c > tile.
//
// Phase A (packs).  CTA b owns every grid-th item of the pack list, walked from its heavy end;
// item i uses pipeline stage i % S and is computed by consumer group i % G.  The producer warps run
// ahead: they read the item descriptor and the voxel ids of the item's rows (requested a few items
// ahead with small asynchronous copies into shared-memory rings) and gather the whole q|k|v rows
// (3*C contiguous elements each) into the stage with one 1-D bulk (TMA) copy per voxel, completing
// on the stage's `full` mbarrier; the rows of an item are dealt round-robin to the producer warps,
// because a warp submits its copies one lane after the other.  The bias table lives in shared
// memory, staged by the consumers
// while the producers already gather.  In a consumer group, thread (hg, r) owns query row r for
// heads hg, hg+HG, ...: q comes from the staged row, the thread walks the keys of its own window
// with a chunked online softmax in the log2 domain (dot products and the P.V update are packed
// fp32 FMAs, fma.rn.f32x2) and writes its output slice straight to global memory; the group's
// warps hand the stage back through `empty`.  16-bit inputs are copied into the upper half of
// each fp32 row and widened in place once per item.
//
// Phase B (windows with c > tile): the same arithmetic, one query tile per item, key tiles
// streamed through stage 0 without overlap; q and the output go straight through global memory.
//
// Every wait is a bounded poll of an mbarrier; on expiry the kernel sets SSW_DEV_TIMEOUT in the
// plan header and every thread leaves through the same exit, where the threads that issued bulk
// copies first wait (again bounded) for the copies still in flight towards this CTA's shared memory.
#include <math.h>

#include <type_traits>

#include "attn_common.cuh"

namespace ssw {

// Shared memory: [barriers 256 B][plan-prefetch rings of the producer warps][bias table][stage 0][stage 1]...
// Stage: [desc int4][item number int, 12 B unused][vox int[kMaxTile]][rows tile*row_stride]
// Row:   [q | k | v as 3*C floats][meta int2 {byte offset of the key's bias-table row,
//         region | (query-side relative-position code << 8)}][8 B unused]
// The 16 bytes after the data skew consecutive rows across the shared-memory banks and carry the
// per-row metadata, so one base pointer reaches both a key's channels and its metadata.
constexpr int kBarBytes = 256;
constexpr int kStageSeqOff = 16;
constexpr int kStageVoxOff = 32;
constexpr int kStageRowsOff = kStageVoxOff + kMaxTile * 4;

// Online-softmax state of one (query row, head).
template <int HD>
struct RowState {
  float2 q[HD / 2];
  float2 acc[HD / 2];
  float m, l;
  __device__ __forceinline__ void reset() {
#pragma unroll
    for (int e = 0; e < HD / 2; ++e) acc[e] = make_float2(0.f, 0.f);
    m = 0.f;  // upstream's row maximum starts from 0 (ops.cu:137)
    l = 0.f;
  }
};

// q row of one head from global memory -> fp32 pairs scaled by `scale`.
template <typename T, int HD>
__device__ __forceinline__ void load_q_global(const T* src, float scale, float2 (&q)[HD / 2]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int e = 0; e < HD / 4; ++e) {
      float4 v = __ldg(reinterpret_cast<const float4*>(src) + e);
      q[2 * e] = make_float2(v.x * scale, v.y * scale);
      q[2 * e + 1] = make_float2(v.z * scale, v.w * scale);
    }
  } else {
#pragma unroll
    for (int e = 0; e < HD / 8; ++e) {
      uint4 u = __ldg(reinterpret_cast<const uint4*>(src) + e);
      float4 a, b;
      widen8<T>(u, a, b);
      q[4 * e] = make_float2(a.x * scale, a.y * scale);
      q[4 * e + 1] = make_float2(a.z * scale, a.w * scale);
      q[4 * e + 2] = make_float2(b.x * scale, b.y * scale);
      q[4 * e + 3] = make_float2(b.z * scale, b.w * scale);
    }
  }
}
template <int HD>
__device__ __forceinline__ void load_q_smem(const float4* src, float scale, float2 (&q)[HD / 2]) {
#pragma unroll
  for (int e = 0; e < HD / 4; ++e) {
    const float4 v = src[e];
    q[2 * e] = make_float2(v.x * scale, v.y * scale);
    q[2 * e + 1] = make_float2(v.z * scale, v.w * scale);
  }
}

// In-place widening of `n_rows` staged 16-bit rows (each copied to byte offset row_elems*2 of its
// fp32 row) by `n_thr` cooperating threads.  Chunks are handled in ascending order, eight per
// thread per round, reads before writes: a float write only ever lands on sources of the same or
// an earlier chunk.  `sync` separates the reads from the writes; returns false if it timed out.
template <typename T, typename Sync>
__device__ __forceinline__ bool widen_rows(unsigned char* rows, int row_stride, int row_elems, int n_rows, int tid,
                                           int n_thr, Sync sync) {
  bool ok = true;
  if constexpr (sizeof(T) == 2) {
    const int cpr = row_elems / 8;  // 16-byte chunks per row
    const int total = n_rows * cpr;
    for (int base = 0; base < total; base += n_thr * 8) {
      uint4 u[8];
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        const int ci = base + x * n_thr + tid;
        if (ci < total) {
          const int rr = ci / cpr, cc = ci - rr * cpr;
          u[x] = *reinterpret_cast<const uint4*>(rows + (size_t)rr * row_stride + row_elems * 2 + cc * 16);
        }
      }
      ok = sync() && ok;
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        const int ci = base + x * n_thr + tid;
        if (ci < total) {
          const int rr = ci / cpr, cc = ci - rr * cpr;
          float4 a, b;
          widen8<T>(u[x], a, b);
          float4* dst = reinterpret_cast<float4*>(rows + (size_t)rr * row_stride + cc * 32);
          dst[0] = a;
          dst[1] = b;
        }
      }
      ok = sync() && ok;
    }
  }
  return ok;
}

// N keys starting at `kp` (= first key's row + byte offset of this head's k slice).  Scores are in
// the log2 domain: q carries scale*log2(e), the shared-memory bias table is pre-multiplied.
template <typename T, int HD, int N, bool kEmit, bool kTableSmem, bool kMask>
__device__ __forceinline__ void attend_chunk(RowState<HD>& st, const unsigned char* kp, int row_stride, int meta_off,
                                             int v_off, const unsigned char* table_h, int my_region, float inv_l,
                                             T* emit_dst) {
  const float mask_add = -100.0f * kLog2e;
  float s[N];
#pragma unroll
  for (int u = 0; u < N; ++u) {
    const unsigned char* rp = kp + u * row_stride;
    const float4* kr = reinterpret_cast<const float4*>(rp);
    // two independent partial sums per key keep the FMA dependency chains short
    float2 sa = make_float2(0.f, 0.f), sb = make_float2(0.f, 0.f);
#pragma unroll
    for (int e = 0; e < HD / 4; ++e) {
      const float4 kv = kr[e];
      sa = __ffma2_rn(st.q[2 * e], make_float2(kv.x, kv.y), sa);
      sb = __ffma2_rn(st.q[2 * e + 1], make_float2(kv.z, kv.w), sb);
    }
    const int2 km = *reinterpret_cast<const int2*>(rp + meta_off);
    const float bias = kTableSmem ? *reinterpret_cast<const float*>(table_h - km.x)
                                  : __ldg(reinterpret_cast<const float*>(table_h - km.x)) * kLog2e;
    float sc = ((sa.x + sb.x) + (sa.y + sb.y)) + bias;
    if (kMask && my_region != (km.y & 31)) sc += mask_add;
    s[u] = sc;
  }
  if constexpr (!kEmit) {
    float mc = s[0];
#pragma unroll
    for (int u = 1; u < N; ++u) mc = fmaxf(mc, s[u]);
    if (mc > st.m) {
      const float corr = fast_exp2(st.m - mc);
      st.l *= corr;
      const float2 c2 = make_float2(corr, corr);
#pragma unroll
      for (int e = 0; e < HD / 2; ++e) st.acc[e] = __fmul2_rn(st.acc[e], c2);
      st.m = mc;
    }
#pragma unroll
    for (int u = 0; u < N; ++u) {
      const float pu = fast_exp2(s[u] - st.m);
      st.l += pu;
      const float2 p2 = make_float2(pu, pu);
      const float4* vr = reinterpret_cast<const float4*>(kp + u * row_stride + v_off);
#pragma unroll
      for (int e = 0; e < HD / 4; ++e) {
        const float4 vv = vr[e];
        st.acc[2 * e] = __ffma2_rn(p2, make_float2(vv.x, vv.y), st.acc[2 * e]);
        st.acc[2 * e + 1] = __ffma2_rn(p2, make_float2(vv.z, vv.w), st.acc[2 * e + 1]);
      }
    }
  } else {
#pragma unroll
    for (int u = 0; u < N; ++u) emit_dst[u] = from_float<T>(fast_exp2(s[u] - st.m) * inv_l);
  }
}

// `n_keys` consecutive staged rows starting at row `first_row` of `rows`: full chunks of four keys,
// then one chunk of the remaining 1-3 (every thread of an item has the same key count, so the
// tail costs no divergence).  `k_off`: byte offset of this head's k slice inside a row; v sits C
// floats further; the row's metadata sits at byte `data_bytes`.  kEmit: second pass that writes
// the normalised probabilities instead of accumulating.
template <typename T, int HD, bool kEmit, bool kTableSmem, bool kMask>
__device__ __forceinline__ void attend_keys(RowState<HD>& st, const unsigned char* rows, int row_stride,
                                            int data_bytes, int first_row, int n_keys, int k_off, int C,
                                            const float* table_h, int my_region, float inv_l, T* emit_dst) {
  const unsigned char* kp = rows + (size_t)first_row * row_stride + k_off;
  const int meta_off = data_bytes - k_off;
  const int v_off = C * 4;
  const unsigned char* tab = reinterpret_cast<const unsigned char*>(table_h);
  int j = 0;
  for (; j + 4 <= n_keys; j += 4, kp += 4 * row_stride)
    attend_chunk<T, HD, 4, kEmit, kTableSmem, kMask>(st, kp, row_stride, meta_off, v_off, tab, my_region, inv_l,
                                                     emit_dst + j);
  switch (n_keys - j) {
    case 1:
      attend_chunk<T, HD, 1, kEmit, kTableSmem, kMask>(st, kp, row_stride, meta_off, v_off, tab, my_region, inv_l,
                                                       emit_dst + j);
      break;
    case 2:
      attend_chunk<T, HD, 2, kEmit, kTableSmem, kMask>(st, kp, row_stride, meta_off, v_off, tab, my_region, inv_l,
                                                       emit_dst + j);
      break;
    case 3:
      attend_chunk<T, HD, 3, kEmit, kTableSmem, kMask>(st, kp, row_stride, meta_off, v_off, tab, my_region, inv_l,
                                                       emit_dst + j);
      break;
    default: break;
  }
}
template <typename T, int HD, bool kEmit, bool kTableSmem>
__device__ __forceinline__ void attend_keys_m(bool use_mask, RowState<HD>& st, const unsigned char* rows,
                                              int row_stride, int data_bytes, int first_row, int n_keys, int k_off,
                                              int C, const float* table_h, int my_region, float inv_l, T* emit_dst) {
  if (use_mask)
    attend_keys<T, HD, kEmit, kTableSmem, true>(st, rows, row_stride, data_bytes, first_row, n_keys, k_off, C,
                                                table_h, my_region, inv_l, emit_dst);
  else
    attend_keys<T, HD, kEmit, kTableSmem, false>(st, rows, row_stride, data_bytes, first_row, n_keys, k_off, C,
                                                 table_h, my_region, inv_l, emit_dst);
}

// Channel-split form: two adjacent lanes share one (query row, head), each holding half of the
// head's channels (q, K/V slices, accumulators).  The partial dot products are combined with one
// shuffle per key.  Same shared-memory traffic as the one-thread form, twice the warps to hide the
// dependent max / exp / accumulate chain behind.
template <int HH, int N, bool kTableSmem, bool kMask>
__device__ __forceinline__ void attend_chunk_split(RowState<HH>& st, const unsigned char* kp, int row_stride, int meta_off,
                                                   int v_off, const unsigned char* table_h, int my_region,
                                                   unsigned lanes) {
  const float mask_add = -100.0f * kLog2e;
  float s[N];
#pragma unroll
  for (int u = 0; u < N; ++u) {
    const float4* kr = reinterpret_cast<const float4*>(kp + u * row_stride);
    float2 sa = make_float2(0.f, 0.f), sb = make_float2(0.f, 0.f);
#pragma unroll
    for (int e = 0; e < HH / 4; ++e) {
      const float4 kv = kr[e];
      sa = __ffma2_rn(st.q[2 * e], make_float2(kv.x, kv.y), sa);
      sb = __ffma2_rn(st.q[2 * e + 1], make_float2(kv.z, kv.w), sb);
    }
    s[u] = (sa.x + sb.x) + (sa.y + sb.y);
  }
#pragma unroll
  for (int u = 0; u < N; ++u) s[u] += __shfl_xor_sync(lanes, s[u], 1);
#pragma unroll
  for (int u = 0; u < N; ++u) {
    const int2 km = *reinterpret_cast<const int2*>(kp + u * row_stride + meta_off);
    const float bias = kTableSmem ? *reinterpret_cast<const float*>(table_h - km.x)
                                  : __ldg(reinterpret_cast<const float*>(table_h - km.x)) * kLog2e;
    s[u] += bias;
    if (kMask && my_region != (km.y & 31)) s[u] += mask_add;
  }
  float mc = s[0];
#pragma unroll
  for (int u = 1; u < N; ++u) mc = fmaxf(mc, s[u]);
  if (mc > st.m) {
    const float corr = fast_exp2(st.m - mc);
    st.l *= corr;
    const float2 c2 = make_float2(corr, corr);
#pragma unroll
    for (int e = 0; e < HH / 2; ++e) st.acc[e] = __fmul2_rn(st.acc[e], c2);
    st.m = mc;
  }
#pragma unroll
  for (int u = 0; u < N; ++u) {
    const float pu = fast_exp2(s[u] - st.m);
    st.l += pu;
    const float2 p2 = make_float2(pu, pu);
    const float4* vr = reinterpret_cast<const float4*>(kp + u * row_stride + v_off);
#pragma unroll
    for (int e = 0; e < HH / 4; ++e) {
      const float4 vv = vr[e];
      st.acc[2 * e] = __ffma2_rn(p2, make_float2(vv.x, vv.y), st.acc[2 * e]);
      st.acc[2 * e + 1] = __ffma2_rn(p2, make_float2(vv.z, vv.w), st.acc[2 * e + 1]);
    }
  }
}

// k_off: byte offset of this lane's half of the head's k slice; meta_off is taken from there
template <int HH, bool kTableSmem, bool kMask>
__device__ __forceinline__ void attend_keys_split(RowState<HH>& st, const unsigned char* rows, int row_stride,
                                                  int data_bytes, int first_row, int n_keys, int k_off, int C,
                                                  const float* table_h, int my_region, unsigned lanes) {
  const unsigned char* kp = rows + (size_t)first_row * row_stride + k_off;
  const int meta_off = data_bytes - k_off;
  const int v_off = C * 4;
  const unsigned char* tab = reinterpret_cast<const unsigned char*>(table_h);
  int j = 0;
  for (; j + 4 <= n_keys; j += 4, kp += 4 * row_stride)
    attend_chunk_split<HH, 4, kTableSmem, kMask>(st, kp, row_stride, meta_off, v_off, tab, my_region, lanes);
  switch (n_keys - j) {
    case 1: attend_chunk_split<HH, 1, kTableSmem, kMask>(st, kp, row_stride, meta_off, v_off, tab, my_region, lanes); break;
    case 2: attend_chunk_split<HH, 2, kTableSmem, kMask>(st, kp, row_stride, meta_off, v_off, tab, my_region, lanes); break;
    case 3: attend_chunk_split<HH, 3, kTableSmem, kMask>(st, kp, row_stride, meta_off, v_off, tab, my_region, lanes); break;
    default: break;
  }
}

// acc * inv_l as T, 16-byte vector stores (global or shared destination)
template <typename T, int HD>
__device__ __forceinline__ void store_out(T* dst, const RowState<HD>& st, float inv_l) {
  const float2 i2 = make_float2(inv_l, inv_l);
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int e = 0; e < HD / 4; ++e) {
      const float2 a = __fmul2_rn(st.acc[2 * e], i2), b = __fmul2_rn(st.acc[2 * e + 1], i2);
      reinterpret_cast<float4*>(dst)[e] = make_float4(a.x, a.y, b.x, b.y);
    }
  } else {
#pragma unroll
    for (int e = 0; e < HD / 8; ++e) {
      uint32_t w[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const float2 a = __fmul2_rn(st.acc[4 * e + x], i2);
        w[x] = pack2<T>(a.x, a.y);
      }
      reinterpret_cast<uint4*>(dst)[e] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// MAXT: the most threads a launch of this variant uses.  One CTA per SM; its warps are spread over
// the SM's four sub-partitions, each with 16384 registers, allocated 8 per thread at a time.
constexpr int regs_for_threads(int max_threads) {
  const int warps_per_part = ((max_threads + 31) / 32 + 3) / 4;
  const int r = (16384 / (warps_per_part * 32)) / 8 * 8;
  return r > 255 ? 255 : r;
}
template <typename T, int HD, bool kTableSmem, int MAXT, bool kSplit>
__global__ void __maxnreg__(regs_for_threads(MAXT)) k_attn_fused(AttnParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  constexpr bool kHalf = sizeof(T) == 2;
  const int tile = p.tile, C = p.C, H = p.H;
  const int S = p.stages, G = p.groups;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);   // [kMaxStages] data landed
  uint64_t* empty = full + kMaxStages;                   // [kMaxStages] stage may be refilled
  uint64_t* gbar = empty + kMaxStages;                   // [kMaxGroups] group-internal barrier
  uint64_t* bbar = gbar + kMaxGroups;                    // phase B copies
  uint64_t* tbar = reinterpret_cast<uint64_t*>(smem) + 30;  // bias table landed
  unsigned char* prod_scratch = smem + kBarBytes;
  float* table_s = reinterpret_cast<float*>(prod_scratch + p.prod_warps * producer_scratch_bytes(p.tile));
  bool table_ok = true;
  unsigned char* stage0 = reinterpret_cast<unsigned char*>(table_s) + (kTableSmem ? ((p.table_floats * 4 + 15) & ~15) : 0);
  const float* table_base = kTableSmem ? table_s : p.table;
  const int gsize = p.group_threads;
  const int gwarps = gsize >> 5;
  const int n_cons = gsize * G;
  const bool is_producer = (int)threadIdx.x >= n_cons;
  const int lane = threadIdx.x & 31;
  const int row_elems = 3 * C;  // q|k|v elements staged per voxel
  const uint32_t copy_bytes = row_elems * sizeof(T);
  const int copy_off = kHalf ? row_elems * 2 : 0;  // 16-bit rows land in the upper half of the fp32 row
  const int n_hiter = H / p.HG;
  const int data_bytes = row_elems * 4;      // fp32 payload of a staged row; its metadata follows
  const float qscale = p.scale * kLog2e;     // scores are kept in the log2 domain

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full + s, p.prod_warps);  // one arrive (with its byte count) per producer warp
      mbar_init(empty + s, gwarps);  // every warp of the consuming group hands the stage back
    }
    for (int g = 0; g < G; ++g) mbar_init(gbar + g, gwarps);
    mbar_init(bbar, 1);
    mbar_init(bbar + 1, 1);
    mbar_init(tbar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  // Only the barrier set-up may run ahead of the kernel this launch is chained behind: the plan,
  // qkv and the bias table may all have been written by it.
  grid_dependency_wait();
  const int n_items = checked_count(p.header[SSW_H_PACKS], p);
  const int n_small = min(checked_count(p.header[SSW_H_PACKS_SMALL], p), n_items);
  if constexpr (kTableSmem) {
    if (!is_producer) {  // the producers are already gathering the first items
      table_ok = stage_table(table_s, p.table, p.table_floats, threadIdx.x, n_cons, tbar);
      consumer_sync(n_cons);
    }
  }

  // ------------------------------------------------------------------------------------------
  // Phase A: packs, producer / consumer pipeline
  // ------------------------------------------------------------------------------------------
  const int my_items =
      n_small > (int)blockIdx.x ? (n_small - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  bool timed_out = !table_ok;
  int issued = 0;  // producer warps: items this warp has submitted its share of row copies for
  if (is_producer) {
    // The rows of an item are dealt round-robin to the producer warps (a warp submits its bulk
    // copies one lane after the other, so two warps submit two rows at a time): this warp's j-th
    // row of an item is row j * PW + pw, lane l looks after j = l and l + 32.  Every producer warp
    // visits every item, so each of them sees every phase of every `empty` barrier (a parity wait
    // tells two consecutive phases apart and no more).  Descriptors, voxel ids and metadata come
    // through the warp's plan-prefetch rings.
    const int PW = p.prod_warps, pw = ((int)threadIdx.x - n_cons) >> 5;
    const int spw = (tile + PW - 1) / PW;  // rows of an item this warp looks after, at most
    unsigned char* pscr = prod_scratch + (size_t)pw * producer_scratch_bytes(tile);
    int4* dring = reinterpret_cast<int4*>(pscr);
    int2* vring = reinterpret_cast<int2*>(pscr + kDescRing * 16);  // [kVoxRing][spw] {voxel id, metadata}
    // The plan lists packs by ascending occupancy; walking the list backwards puts the long items
    // first and leaves the short ones for the tail of the kernel.
    auto item_index = [&](int k) { return n_small - 1 - ((int)blockIdx.x + k * (int)gridDim.x); };
    for (int t = -kDescAhead; t < my_items; ++t) {
      const int td = t + kDescAhead;
      if (lane == 0 && td < my_items) cp_async16(dring + (td & (kDescRing - 1)), p.pack_desc + item_index(td));
      // every iteration commits one group; what was requested kVoxAhead iterations ago has landed
      // once at most kVoxAhead - 1 groups are pending: the descriptor of item t + kVoxAhead (asked for
      // kDescAhead - kVoxAhead iterations before that) and the ids / metadata of item t
      cp_async_wait<kVoxAhead - 1>();
      __syncwarp();
      const int tv = t + kVoxAhead;
      if (tv >= 0 && tv < my_items) {
        const int4 d = checked_desc(dring[tv & (kDescRing - 1)], p, true);
        const int nr = d.z * d.y;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int j = lane + 32 * k, rr = j * PW + pw;
          if (j < spw && rr < nr) {
            int2* dst = vring + (tv & (kVoxRing - 1)) * spw + j;
            cp_async4(&dst->x, p.pack_perm + d.x + rr);
            cp_async4(&dst->y, p.pack_meta + d.x + rr);
          }
        }
      }
      cp_async_commit();
      if (t < 0) continue;
      const int s = t % S, use = t / S;
      const int4 d_cur = checked_desc(dring[t & (kDescRing - 1)], p, true);
      const int nr = d_cur.z * d_cur.y;
      int vox[2], km[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int j = lane + 32 * k, rr = j * PW + pw;
        vox[k] = 0;
        km[k] = 0;
        if (j < spw && rr < nr) {
          const int2 e = vring[(t & (kVoxRing - 1)) * spw + j];
          vox[k] = checked_voxel(e.x, p);
          km[k] = checked_meta(e.y, p);
        }
      }
      if (use > 0 && !mbar_wait_bounded(empty + s, (use - 1) & 1)) {
        timed_out = true;
        break;
      }
      unsigned char* st = stage0 + (size_t)s * p.stage_bytes;
      if (lane == 0 && pw == 0) {
        *reinterpret_cast<int4*>(st) = d_cur;
        *reinterpret_cast<int*>(st + kStageSeqOff) = t;
      }
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int j = lane + 32 * k, rr = j * PW + pw;
        if (j < spw && rr < nr) {
          reinterpret_cast<int*>(st + kStageVoxOff)[rr] = vox[k];
          *reinterpret_cast<int2*>(st + kStageRowsOff + (size_t)rr * p.row_stride + data_bytes) = make_int2(
              meta_rel(km[k]) * H * 4, meta_region(km[k]) | ((meta_rel(km[k]) + p.rel_off) << 8));
        }
      }
      // rows pw, pw + PW, ... below nr are this warp's
      const int my_rows = nr > pw ? (nr - pw + PW - 1) / PW : 0;
      // The arrive releases the stage to the consumers: every lane's metadata stores must come
      // before it, and the warp's copies after the byte count they complete against is announced.
      __syncwarp();
      if (lane == 0) mbar_expect_tx(full + s, (uint32_t)my_rows * copy_bytes);
      __syncwarp();
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int j = lane + 32 * k, rr = j * PW + pw;
        if (j < spw && rr < nr)
          bulk_g2s(st + kStageRowsOff + (size_t)rr * p.row_stride + copy_off,
                   reinterpret_cast<const T*>(p.qkv) + (int64_t)vox[k] * 3 * C, copy_bytes, full + s);
      }
      issued = t + 1;
    }
    cp_async_wait<0>();  // nothing of the plan prefetch may still be under way towards this CTA's shared memory
  } else {
    const int g = threadIdx.x / gsize;
    const int ltid = threadIdx.x - g * gsize;
    const int hg = ltid / tile;
    const int r = ltid - hg * tile;
    const bool thread_used = hg < p.HG;
    uint32_t gphase = 0;
    RowState<HD> st;
    for (int i = g; i < my_items && !timed_out; i += G) {
      const int s = i % S;
      const int use = i / S;
      unsigned char* sp = stage0 + (size_t)s * p.stage_bytes;
      unsigned char* rows = sp + kStageRowsOff;
      // A group skips the uses of a stage that belong to the other groups, and a parity wait tells
      // two consecutive phases apart, no more: should the stage still be in the phase before the one
      // awaited, the wait answers at once.  The item number in the stage header (written before the
      // producer's arrive) settles it: it can only read i once this use's phase has begun.
      bool landed = mbar_wait_bounded(full + s, use & 1);
      for (int again = 0; landed && *reinterpret_cast<volatile const int*>(sp + kStageSeqOff) != i; ++again)
        landed = again < (1 << 16) && mbar_wait_bounded(full + s, use & 1);
      if (!landed) {
        timed_out = true;
        break;
      }
      const int4 d = *reinterpret_cast<const int4*>(sp);
      const int c = d.y;
      const int q_rows = d.z * c;
      if constexpr (kHalf) {
        if (!widen_rows<T>(rows, p.row_stride, row_elems, q_rows, ltid, gsize,
                           [&]() { return group_barrier(gbar + g, gphase, lane); })) {
          timed_out = true;
          break;
        }
      }
      if constexpr (kSplit) {
        // lanes 2t, 2t+1 share (row, head): lane parity picks the half of the head's channels
        constexpr int HH = HD / 2;
        const int x = ltid & 1, rh = ltid >> 1;
        const int hgs = rh / tile, rs = rh - hgs * tile;
        if (hgs < p.HG && rs < q_rows) {
          const unsigned lanes = __activemask();  // both lanes of a pair are here or neither is
          const int kbeg = (rs / c) * c;
          const unsigned char* myrow = rows + (size_t)rs * p.row_stride;
          const int my_vox = reinterpret_cast<const int*>(sp + kStageVoxOff)[rs];
          const int2 me = *reinterpret_cast<const int2*>(myrow + data_bytes);
          for (int hi = 0; hi < n_hiter; ++hi) {
            const int h = hi * p.HG + hgs;
            RowState<HH> hs;
            load_q_smem<HH>(reinterpret_cast<const float4*>(myrow) + (h * HD + x * HH) / 4, qscale, hs.q);
            hs.reset();
            const float* table_h = table_base + (me.y >> 8) * H + h;
            if (p.use_mask)
              attend_keys_split<HH, kTableSmem, true>(hs, rows, p.row_stride, data_bytes, kbeg, c,
                                                      (C + h * HD + x * HH) * 4, C, table_h, me.y & 31, lanes);
            else
              attend_keys_split<HH, kTableSmem, false>(hs, rows, p.row_stride, data_bytes, kbeg, c,
                                                       (C + h * HD + x * HH) * 4, C, table_h, 0, lanes);
            const float inv_l = 1.0f / (hs.l + 1e-8f);  // ops.cu:164
            store_out<T, HH>(reinterpret_cast<T*>(p.out) + (int64_t)my_vox * C + h * HD + x * HH, hs, inv_l);
            for (int d = 1; d < p.outs.n; ++d)  // the same row on peer GPUs
              store_out<T, HH>(reinterpret_cast<T*>(p.outs.base[d]) + (int64_t)my_vox * C + h * HD + x * HH, hs, inv_l);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
        continue;
      }
      const bool row_active = thread_used && r < q_rows;
      const int wl = r / c;
      const int kbeg = wl * c;
      if (row_active) {
        unsigned char* myrow = rows + (size_t)r * p.row_stride;
        const int my_vox = reinterpret_cast<const int*>(sp + kStageVoxOff)[r];
        const int2 me = *reinterpret_cast<const int2*>(myrow + data_bytes);
        const int my_rel = (me.y >> 8) * H;
        const int my_region = me.y & 31;
        for (int hi = 0; hi < n_hiter; ++hi) {
          const int h = hi * p.HG + hg;
          load_q_smem<HD>(reinterpret_cast<const float4*>(myrow) + (h * HD) / 4, qscale, st.q);
          st.reset();
          const float* table_h = table_base + my_rel + h;
          attend_keys_m<T, HD, false, kTableSmem>(p.use_mask != 0, st, rows, p.row_stride, data_bytes, kbeg, c,
                                                  (C + h * HD) * 4, C, table_h, my_region, 0.f, (T*)nullptr);
          const float inv_l = 1.0f / (st.l + 1e-8f);  // ops.cu:164
          if (p.attn_vals) {
            const int64_t blk = checked_coo_block(d.w + wl, c, p);
            T* dst = reinterpret_cast<T*>(p.attn_vals) + (blk * H + (int64_t)h * c * c) + (int64_t)(r - kbeg) * c;
            if (blk >= 0)
              attend_keys_m<T, HD, true, kTableSmem>(p.use_mask != 0, st, rows, p.row_stride, data_bytes, kbeg, c,
                                                     (C + h * HD) * 4, C, table_h, my_region, inv_l, dst);
          }
          // Straight to global memory: each thread owns a 16-byte-aligned run of HD outputs of one
          // row (bulk stores of whole rows were tried; one bulk operation per row is what bounds them).
          store_out<T, HD>(reinterpret_cast<T*>(p.out) + (int64_t)my_vox * C + h * HD, st, inv_l);
          for (int d = 1; d < p.outs.n; ++d)  // the same row on peer GPUs
            store_out<T, HD>(reinterpret_cast<T*>(p.outs.base[d]) + (int64_t)my_vox * C + h * HD, st, inv_l);
        }
      }
      // widen_rows wrote the stage through the generic proxy; the next bulk copy into it goes
      // through the async proxy
      if constexpr (kHalf) fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(empty + s);
    }
  }
  if (timed_out) atomicOr(reinterpret_cast<unsigned*>(p.header + SSW_H_ERROR), SSW_DEV_TIMEOUT);
  // A timed-out role leaves; the other roles then time out on their own bounded waits.
  if (__syncthreads_or(timed_out)) {
    // Nobody consumes what is still in flight, but the CTA must not retire under copies that
    // target its shared memory: each producer warp waits, bounded, for the last use of every stage
    // it submitted copies to (whether the phase completes or not, the wait outlasts any copy).
    if (is_producer && lane == 0)
      for (int j = max(0, issued - S); j < issued; ++j) mbar_wait_bounded(full + j % S, (j / S) & 1);
    if (kTableSmem && threadIdx.x == 0 && !table_ok) mbar_wait_bounded(tbar, 0);
    return;
  }

  // ------------------------------------------------------------------------------------------
  // Phase B: windows with c > tile; one query tile per item, key tiles through stage 0
  // ------------------------------------------------------------------------------------------
  // Key tiles alternate between stages 0 and 1: the copy of the next tile is in flight while the
  // current one is used.  In the lane-pair form two adjacent threads share a (row, head).
  constexpr int HB = kSplit ? HD / 2 : HD;  // channels per thread
  const int xh = kSplit ? (int)(threadIdx.x & 1) : 0;
  const int rh = kSplit ? (int)(threadIdx.x >> 1) : (int)threadIdx.x;
  const int hg = rh / tile;
  const int r = rh - hg * tile;
  const bool thread_used = hg < p.HG;
  uint64_t* tbars[2] = {bbar, bbar + 1};
  uint32_t tphase[2] = {0, 0};
  for (int item = n_small + blockIdx.x; item < n_items; item += gridDim.x) {
    const int4 d = checked_desc(__ldg(p.pack_desc + item), p, false);
    const int c = d.y;
    const int q_first = (-d.z - 1) * tile;
    const int q_rows = min(tile, c - q_first);
    const bool row_active = thread_used && r < q_rows;
    int my_vox = 0, my_rel = 0, my_region = 0;
    if (row_active) {
      const int row = d.x + q_first + r;
      my_vox = checked_voxel(__ldg(p.pack_perm + row), p);
      const int m = checked_meta(__ldg(p.pack_meta + row), p);
      my_rel = (meta_rel(m) + p.rel_off) * H;
      my_region = meta_region(m);
    }
    const int n_tiles = (c + tile - 1) / tile;
    const int n_pass = p.attn_vals ? 2 : 1;
    const int n_seq = n_pass * n_tiles;
    auto issue_tile = [&](int q) {  // key tile q % n_tiles into buffer q & 1
      const int k0 = (q % n_tiles) * tile;
      const int rows_t = min(tile, c - k0);
      unsigned char* rb = stage0 + (size_t)(q & 1) * p.stage_bytes + kStageRowsOff;
      if (threadIdx.x == 0) mbar_expect_tx(tbars[q & 1], rows_t * copy_bytes);
      if ((int)threadIdx.x < rows_t) {
        const int row = d.x + k0 + threadIdx.x;
        const int vj = checked_voxel(__ldg(p.pack_perm + row), p);
        const int km = checked_meta(__ldg(p.pack_meta + row), p);
        *reinterpret_cast<int2*>(rb + (size_t)threadIdx.x * p.row_stride + data_bytes) =
            make_int2(meta_rel(km) * H * 4, meta_region(km));
        bulk_g2s(rb + (size_t)threadIdx.x * p.row_stride + copy_off,
                 reinterpret_cast<const T*>(p.qkv) + (int64_t)vj * 3 * C, copy_bytes, tbars[q & 1]);
      }
    };
    for (int hi = 0; hi < n_hiter; ++hi) {
      const int h = hi * p.HG + hg;
      RowState<HB> st;
      st.reset();
      float inv_l = 0.f;
      if (row_active)
        load_q_global<T, HB>(reinterpret_cast<const T*>(p.qkv) + (int64_t)my_vox * 3 * C + h * HD + xh * HB, qscale, st.q);
      const float* table_h = table_base + my_rel + h;
      T* emit = nullptr;
      if (n_pass == 2 && row_active) {
        const int64_t blk = checked_coo_block(d.w, c, p);
        if (blk >= 0)
          emit = reinterpret_cast<T*>(p.attn_vals) + (blk * H + (int64_t)h * c * c) + (int64_t)(q_first + r) * c;
      }
      issue_tile(0);
      for (int q = 0; q < n_seq; ++q) {
        const int b = q & 1;
        const int k0 = (q % n_tiles) * tile;
        const int rows_t = min(tile, c - k0);
        unsigned char* rows = stage0 + (size_t)b * p.stage_bytes + kStageRowsOff;
        if (q + 1 < n_seq) issue_tile(q + 1);  // its buffer was released by the barrier that ended tile q-1
        __syncthreads();                        // row metadata of tile q visible
        const bool ok = mbar_wait_bounded(tbars[b], tphase[b]);
        if (__syncthreads_or(!ok)) {
          if (threadIdx.x == 0) {
            atomicOr(reinterpret_cast<unsigned*>(p.header + SSW_H_ERROR), SSW_DEV_TIMEOUT);
            // drain: this tile's copies and, if issued, the next tile's, before the CTA retires
            mbar_wait_bounded(tbars[b], tphase[b]);
            if (q + 1 < n_seq) mbar_wait_bounded(tbars[b ^ 1], tphase[b ^ 1]);
          }
          return;
        }
        tphase[b] ^= 1;
        if constexpr (kHalf)
          widen_rows<T>(rows, p.row_stride, row_elems, rows_t, threadIdx.x, blockDim.x, []() {
            __syncthreads();
            return true;
          });
        if (row_active) {
          if constexpr (kSplit) {
            const unsigned lanes = __activemask();  // both lanes of a pair are here or neither is
            if (p.use_mask)
              attend_keys_split<HB, kTableSmem, true>(st, rows, p.row_stride, data_bytes, 0, rows_t,
                                                      (C + h * HD + xh * HB) * 4, C, table_h, my_region, lanes);
            else
              attend_keys_split<HB, kTableSmem, false>(st, rows, p.row_stride, data_bytes, 0, rows_t,
                                                       (C + h * HD + xh * HB) * 4, C, table_h, my_region, lanes);
          } else {
            if (q < n_tiles)
              attend_keys_m<T, HD, false, kTableSmem>(p.use_mask != 0, st, rows, p.row_stride, data_bytes, 0, rows_t,
                                                      (C + h * HD) * 4, C, table_h, my_region, 0.f, (T*)nullptr);
            else if (emit)
              attend_keys_m<T, HD, true, kTableSmem>(p.use_mask != 0, st, rows, p.row_stride, data_bytes, 0, rows_t,
                                                     (C + h * HD) * 4, C, table_h, my_region, inv_l, emit + k0);
          }
        }
        if (q == n_tiles - 1) inv_l = 1.0f / (st.l + 1e-8f);
        if constexpr (kHalf) fence_async_smem();  // the widened rows were written through the generic proxy
        __syncthreads();  // everyone done with this tile before it is overwritten
      }
      if (row_active) {
        store_out<T, HB>(reinterpret_cast<T*>(p.out) + (int64_t)my_vox * C + h * HD + xh * HB, st, inv_l);
        for (int d = 1; d < p.outs.n; ++d)  // the same row on peer GPUs
          store_out<T, HB>(reinterpret_cast<T*>(p.outs.base[d]) + (int64_t)my_vox * C + h * HD + xh * HB, st, inv_l);
      }
    }
  }
}

// Shape of the kernel for (tile, heads, head_dim, dtype, window): heads processed in parallel (a
// divisor of `heads`, at most 256 threads per group), pipeline stages and consumer groups that
// fit the SM's shared memory next to the bias table (kept in shared memory when it is small: the
// L1 that remains beside ~200 KB of stages is too small to hold it).
constexpr int kTableSmemMax = 40 * 1024;
constexpr size_t kSmemBudget = 226 * 1024;
struct KernelShape {
  int hg, group_threads, groups, stages, prod_warps, row_stride, stage_bytes, out_off, table_floats;
  size_t smem;
};
static int table_entries(const int32_t w[3], int heads) {
  return (2 * w[0] - 1) * (2 * w[1] - 1) * (2 * w[2] - 1) * heads;
}
static KernelShape kernel_shape(int tile, int heads, int head_dim, int elt, const int32_t rpb_window[3], bool split = false) {
  KernelShape s;
  int cap = 256 / tile;
  if (cap < 1) cap = 1;
  s.hg = 1;
  for (int g = 1; g <= heads && g <= cap; ++g)
    if (heads % g == 0) s.hg = g;
  s.group_threads = ((split ? 2 * tile : tile) * s.hg + 31) & ~31;
  const int C = heads * head_dim;
  s.row_stride = 3 * C * 4 + 16;  // +16 B skews rows across shared-memory banks
  const int rows_bytes = kStageRowsOff + tile * s.row_stride;
  s.out_off = 0;
  s.stage_bytes = rows_bytes;
  (void)elt;
  const int tf = table_entries(rpb_window, heads);
  s.table_floats = tf * 4 <= kTableSmemMax ? tf : 0;
  // per stage: the stage itself and the plan-prefetch rings of its producer warp
  const size_t fixed = kBarBytes + ((s.table_floats * 4 + 15) & ~15);
  // (the plan-prefetch rings of the two producer warps are counted once per stage: room to spare)
  const size_t per_stage = (size_t)s.stage_bytes + producer_scratch_bytes(tile);
  int stages = (int)((kSmemBudget - fixed) / per_stage);
  if (stages > kMaxStages) stages = kMaxStages;
  s.stages = stages;
  // One stage is always in flight.  The lane-pair form wants 96 registers per thread, which 20
  // warps at most can have (five per sub-partition); the other forms run with up to 1024 threads.
  s.prod_warps = 2;
  int groups = stages - 1;
  if (groups > kMaxGroups) groups = kMaxGroups;
  while (groups > 1 && groups * s.group_threads + 32 * s.prod_warps > (split ? 640 : 1024)) --groups;
  if (groups < 1) groups = 1;
  s.groups = groups;
  s.smem = fixed + (size_t)(stages > 0 ? stages : 1) * per_stage;
  return s;
}

template <typename T, int HD, bool kTableSmem>
static int launch_attn(const AttnParams& p, int threads, size_t smem, cudaStream_t stream) {
  int dev = 0, sms = 0;
  SSW_CUDA_TRY(cudaGetDevice(&dev));
  SSW_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if constexpr (sizeof(T) == 4) {
    if (p.split) {
      if (threads > 640) return SSW_E_UNSUPPORTED;
      void (*kern)(AttnParams) = k_attn_fused<T, HD, kTableSmem, 640, true>;
      SSW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      SSW_CUDA_TRY(launch_chained(kern, dim3(sms), dim3(threads), smem, stream, p));
      SSW_LAUNCH_CHECK("k_attn_fused");
      return SSW_OK;
    }
  }
  if (threads <= 384) {
    auto kern = k_attn_fused<T, HD, kTableSmem, 384, false>;
    SSW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    SSW_CUDA_TRY(launch_chained(kern, dim3(sms), dim3(threads), smem, stream, p));
  } else if (threads <= 512) {
    auto kern = k_attn_fused<T, HD, kTableSmem, 512, false>;
    SSW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    SSW_CUDA_TRY(launch_chained(kern, dim3(sms), dim3(threads), smem, stream, p));
  } else {
    auto kern = k_attn_fused<T, HD, kTableSmem, 1024, false>;
    SSW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    SSW_CUDA_TRY(launch_chained(kern, dim3(sms), dim3(threads), smem, stream, p));
  }
  SSW_LAUNCH_CHECK("k_attn_fused");
  return SSW_OK;
}

template <typename T>
static int dispatch(const AttnParams& p, int hd, int threads, size_t smem, cudaStream_t stream) {
  const bool ts = p.table_floats > 0;
  if (hd == 16)
    return ts ? launch_attn<T, 16, true>(p, threads, smem, stream) : launch_attn<T, 16, false>(p, threads, smem, stream);
  if (hd == 32)
    return ts ? launch_attn<T, 32, true>(p, threads, smem, stream) : launch_attn<T, 32, false>(p, threads, smem, stream);
  return SSW_E_UNSUPPORTED;
}

int mma_default_tile(int heads, int head_dim, const int32_t rpb_window[3]);
int run_attn_mma(AttnParams p, int dtype, int head_dim, const int32_t rpb_window[3], const int32_t* bins,
                 const int32_t* win_start, const int32_t* win_pstart, int n_per_window, cudaStream_t stream);

}  // namespace ssw

using namespace ssw;

extern "C" int32_t ssw_default_padded(int dtype) { return dtype == SSW_BF16 || dtype == SSW_F16; }

extern "C" int32_t ssw_default_tile_rows(int32_t heads, int32_t head_dim, int dtype, const int32_t rpb_window[3]) {
  if (heads <= 0 || head_dim <= 0 || !rpb_window) return 0;
  if (ssw_default_padded(dtype)) return mma_default_tile(heads, head_dim, rpb_window);
  const int elt = dtype == SSW_F32 ? 4 : 2;
  // the largest tile that still leaves three pipeline stages
  static const int kTiles[] = {64, 48, 32, 24, 16};
  for (int tile : kTiles)
    if (kernel_shape(tile, heads, head_dim, elt, rpb_window).stages >= 3) return tile;
  return 8;
}

extern "C" int ssw_attn_fused(const void* qkv, int dtype, int32_t heads, int32_t head_dim, const ssw_plan_layout* L,
                              const int32_t* plan, const float* table, const int32_t rpb_window[3], float scale,
                              int use_mask, void* out, void* attn_vals, void* stream_) {
  void* outs[1] = {out};
  return ssw_attn_fused_multi(qkv, dtype, heads, head_dim, L, plan, table, rpb_window, scale, use_mask, outs, 1, attn_vals,
                              stream_);
}

extern "C" int ssw_attn_fused_multi(const void* qkv, int dtype, int32_t heads, int32_t head_dim, const ssw_plan_layout* L,
                                    const int32_t* plan, const float* table, const int32_t rpb_window[3], float scale,
                                    int use_mask, void* const* outs, int32_t n_outs, void* attn_vals, void* stream_) {
  if (!L || !plan || !table || !rpb_window || heads <= 0 || head_dim <= 0) return SSW_E_INVALID;
  if (!outs || n_outs < 1 || n_outs > kMaxOuts) return SSW_E_INVALID;
  if (L->n_vox == 0) return SSW_OK;
  void* out = outs[0];
  if (!qkv || !out) return SSW_E_INVALID;
  for (int d = 0; d < n_outs; ++d)
    if (!outs[d] || (reinterpret_cast<uintptr_t>(outs[d]) & 15)) return SSW_E_INVALID;
  const int elt = dtype == SSW_F32 ? 4 : (dtype == SSW_BF16 || dtype == SSW_F16) ? 2 : 0;
  if (!elt) return SSW_E_INVALID;
  const int C = heads * head_dim;
  if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return SSW_E_INVALID;
  if ((head_dim * elt) % 16) return SSW_E_UNSUPPORTED;
  const int tile = L->tile_rows;
  if (tile > kMaxTile) return SSW_E_UNSUPPORTED;
  cudaStream_t stream = (cudaStream_t)stream_;
  AttnParams p = {};
  p.qkv = qkv;
  p.out = out;
  p.outs.n = n_outs;
  for (int d = 0; d < n_outs; ++d) p.outs.base[d] = outs[d];
  p.attn_vals = attn_vals;
  p.header = const_cast<int32_t*>(plan + L->off_header);
  p.pack_desc = reinterpret_cast<const int4*>(plan + L->off_pack_desc);
  p.pack_perm = plan + L->off_pack_perm;
  p.pack_meta = plan + L->off_pack_meta;
  p.pack_win = plan + L->off_pack_win;
  p.coo_start = plan + L->off_coo_start;
  p.table = table;
  p.rel_off = ((rpb_window[0] - 1) * (2 * rpb_window[1] - 1) + (rpb_window[1] - 1)) * (2 * rpb_window[2] - 1) +
              (rpb_window[2] - 1);
  p.H = heads;
  p.C = C;
  p.tile = tile;
  p.scale = scale;
  p.use_mask = use_mask;
  p.n_vox = (int)L->n_vox;
  p.pack_cap = (int)L->pack_cap;
  p.w_cap = (int)L->w_cap;
  if (L->padded) {
    // padded plan: the tensor-core kernel takes both the packs and the windows beyond a pack
    if (elt != 2 || attn_vals) return SSW_E_INVALID;
    return run_attn_mma(p, dtype, head_dim, rpb_window, plan + L->off_bins, plan + L->off_win_start,
                        plan + L->off_win_pstart, (int)L->n_per_window, stream);
  }
  // fp32 without the COO output: the channels of a (row, head) are split over a lane pair
  bool split = dtype == SSW_F32 && !attn_vals && head_dim % 8 == 0;
  KernelShape s = kernel_shape(tile, heads, head_dim, elt, rpb_window, split);
  if (split && s.groups * s.group_threads + 32 * s.prod_warps > 640) {
    split = false;
    s = kernel_shape(tile, heads, head_dim, elt, rpb_window, false);
  }
  if (s.stages < 2 || s.smem > 227 * 1024) return SSW_E_UNSUPPORTED;
  p.split = split ? 1 : 0;
  const int threads = s.groups * s.group_threads + 32 * s.prod_warps;
  p.HG = s.hg;
  p.group_threads = s.group_threads;
  p.groups = s.groups;
  p.stages = s.stages;
  p.prod_warps = s.prod_warps;
  p.row_stride = s.row_stride;
  p.stage_bytes = s.stage_bytes;
  p.out_off = s.out_off;
  p.table_floats = s.table_floats;
  switch (dtype) {
    case SSW_F32: return dispatch<float>(p, head_dim, threads, s.smem, stream);
    case SSW_BF16: return dispatch<__nv_bfloat16>(p, head_dim, threads, s.smem, stream);
    case SSW_F16: return dispatch<__half>(p, head_dim, threads, s.smem, stream);
  }
  return SSW_E_INVALID;
}
