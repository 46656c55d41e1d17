// Device helpers shared by the fused attention kernels: fast exp2, mbarrier arrive, bulk (TMA)
// stores, proxy fence, mbarrier-based group barrier, 16-bit widening and packing.
#pragma once

#include <type_traits>

#include "ssw_common.cuh"

namespace ssw {

constexpr float kLog2e = 1.4426950408889634f;

constexpr int kMaxStages = 6;
constexpr int kMaxGroups = 4;
constexpr int kMaxTile = 64, kMaxProducerWarps = kMaxStages;

// Destinations of the output rows: the caller's buffer and, when one scene is split over several
// GPUs, the same [N, C] buffer on every peer (mapped into this process): a finished row is stored
// to all of them with ordinary stores, so no gather step follows the kernel.
constexpr int kMaxOuts = 8;
struct OutSet {
  void* base[kMaxOuts];
  int n;
};

struct AttnParams {
  const void* qkv;
  void* out;          // = outs.base[0]
  OutSet outs;
  void* attn_vals;
  int32_t* header;
  const int4* pack_desc;
  const int32_t* pack_perm;
  const int32_t* pack_meta;
  const int32_t* pack_win;
  const int32_t* coo_start;
  const float* table;
  int rel_off;
  int H, C, tile, HG;
  int group_threads;  // threads of one consumer group (multiple of 32) = ceil32(tile * HG)
  int groups, stages;
  int prod_warps;     // warps that issue the row copies of an item
  int n_vox, pack_cap, w_cap;  // bounds the kernels hold the plan's voxel ids, item and window counts to
  int split;          // CUDA-core kernel: a (row, head) is shared by two lanes, half the channels each
  float scale;
  int use_mask;
  int row_stride;     // bytes between fp32 rows in a stage
  int stage_bytes;    // bytes of one pipeline stage
  int out_off;        // byte offset of the 16-bit output staging area inside a stage (0 for fp32)
  int table_floats;   // > 0: the bias table is staged in shared memory (that many floats)
  int skip_big;       // tensor-core kernel: windows beyond a pack are left to the tcgen05 kernel
};



// The attention kernels turn plan entries into addresses.  A plan that is stale or was overwritten
// must not become a wild access: entries are held to their bounds, violations set SSW_DEV_BAD_PLAN
// and are replaced by harmless values (the output is then meaningless, and flagged).  `P` is any
// parameter block with header, n_vox, pack_cap, tile and rel_off members.
template <typename P>
__device__ __forceinline__ void flag_bad_plan(const P& p) {
  atomicOr(reinterpret_cast<unsigned*>(p.header + SSW_H_ERROR), SSW_DEV_BAD_PLAN);
}
template <typename P>
__device__ __forceinline__ int checked_voxel(int v, const P& p) {
  if ((unsigned)v < (unsigned)p.n_vox) return v;
  flag_bad_plan(p);
  return 0;
}
// pack descriptor {first row, c, windows (or -(tile index)-1), window slot}.  `want_pack`: the
// position in the work list says which of the two forms the entry must have.
template <typename P>
__device__ __forceinline__ int4 checked_desc(int4 d, const P& p, bool want_pack) {
  const bool pack = d.z >= 0;
  // 32-bit arithmetic is safe here: every product is formed only after its factors are known small
  bool ok = pack == want_pack && (unsigned)d.x < (unsigned)p.n_vox && (unsigned)(d.y - 1) < 1023u && d.w >= 0;
  if (pack) ok = ok && d.z <= p.tile && d.z * d.y <= p.tile && d.z * d.y <= p.n_vox - d.x;
  else ok = ok && d.y > p.tile && d.y <= p.n_vox - d.x && -d.z - 1 <= (d.y - 1) / p.tile;
  if (ok) return d;
  flag_bad_plan(p);
  return want_pack ? make_int4(0, 1, 0, 0) : make_int4(0, 1, -1, 0);  // an empty pack / a one-row window
}
template <typename P>
__device__ __forceinline__ int checked_count(int n, const P& p) {
  if ((unsigned)n <= (unsigned)p.pack_cap) return n;
  flag_bad_plan(p);
  return 0;
}
// The relative-position code of a row metadata word selects a row of the bias table: codes of real
// positions lie in [0, rel_off].
template <typename P>
__device__ __forceinline__ int checked_meta(int m, const P& p) {
  if (meta_rel(m) <= p.rel_off) return m;
  flag_bad_plan(p);
  return m & 0xffff;
}

// First element (per head) of the COO block of the window in pack-order slot `slot` (occupancy c),
// as an offset into the attn_vals output; the block must lie inside the sum c^2 elements the
// caller sized that output from.  A violation is flagged and answered with -1: nothing is written.
__device__ __forceinline__ int64_t checked_coo_block(int slot, int c, const AttnParams& p) {
  if ((unsigned)slot < (unsigned)p.w_cap) {
    const int kwin = __ldg(p.pack_win + slot);
    if ((unsigned)kwin < (unsigned)p.w_cap) {
      const unsigned start = (unsigned)__ldg(p.coo_start + kwin);
      const unsigned total = (unsigned)p.header[SSW_H_SUMC2_LO];
      if (p.header[SSW_H_SUMC2_HI] == 0 && start <= total && (unsigned)(c * c) <= total - start) return start;
    }
  }
  flag_bad_plan(p);
  return -1;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// shared -> global bulk (TMA) store of `bytes` (multiple of 16, both addresses 16-byte aligned)
__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// make generic-proxy writes to shared memory visible to the async proxy (bulk stores)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Stage the relative-position bias table in shared memory, pre-multiplied by log2(e).  Loads are
// issued eight at a time so that the loop is bound by bandwidth, not by one L2 round trip per value.
// Stage the bias table in shared memory, pre-multiplied by log2 e.  Called by the first `step`
// threads of the CTA (tid = 0..step-1).  When the table starts on a 16-byte boundary its bulk
// comes in with one bulk (TMA) copy completing on `bar` (initialised with count 1) and is scaled
// in place; otherwise, and for the last few entries, plain loads.  False if the copy's wait ran out.
__device__ __forceinline__ bool stage_table(float* dst, const float* __restrict__ src, int n, int tid, int step,
                                            uint64_t* bar) {
  const int nb = (reinterpret_cast<uintptr_t>(src) & 15) == 0 ? (n & ~3) : 0;  // entries the bulk copy brings
  if (nb > 0 && tid == 0) {
    mbar_expect_tx(bar, (uint32_t)nb * 4u);
    bulk_g2s(dst, src, (uint32_t)nb * 4u, bar);
  }
  for (int i0 = nb + tid; i0 < n; i0 += step * 8) {
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = (i0 + k * step < n) ? __ldg(src + i0 + k * step) : 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (i0 + k * step < n) dst[i0 + k * step] = v[k] * kLog2e;
  }
  if (nb > 0) {
    if (!mbar_wait_bounded(bar, 0)) return false;
    for (int i = tid * 4; i < nb; i += step * 4) {
      float4 v = *reinterpret_cast<float4*>(dst + i);
      v.x *= kLog2e; v.y *= kLog2e; v.z *= kLog2e; v.w *= kLog2e;
      *reinterpret_cast<float4*>(dst + i) = v;
    }
  }
  return true;
}

// ---- producer-side plan prefetch ------------------------------------------------------------
// Work items are dealt to the producer warps whole, and every pipeline stage has exactly one
// producer warp: warp w owns the stages w, w + PW, ... and gathers the items that fall into them.  (What an item costs its producer is mostly
// fixed - a few hundred dependent instructions of one warp, about a microsecond - so the warps must
// not all pay it for every item.  And a stage must have a single producer: a parity wait on the
// stage's `empty` barrier tells two consecutive phases apart and no more, so the waiter has to see
// every phase, which a warp that skipped uses of the stage would not.)  Per item a warp needs the
// item's descriptor and then, at addresses the descriptor gives, the voxel id and metadata word of
// each row slot.  Both come from the plan in global memory and are requested a few of the warp's own
// items ahead with asynchronous 4/16-byte copies into small shared-memory rings;
// cp.async.wait_group keeps exactly the wanted number of requests in flight.
constexpr int kDescRing = 8, kDescAhead = 4;  // descriptor of the warp's item t + 4 is requested while item t is issued
constexpr int kVoxRing = 4, kVoxAhead = 2;    // voxel ids / metadata of its item t + 2
// bytes of plan-prefetch rings one producer warp owns: descriptors, then (voxel id, metadata) pairs
__host__ __device__ inline int producer_scratch_bytes(int tile) { return kDescRing * 16 + kVoxRing * tile * 8; }
// Before a timed-out CTA retires: wait (bounded) for the row copies this producer warp submitted
// and nobody will consume.  The warp owns stages pw, pw + PW, ... (K = S / PW of them) and has
// submitted `issued` items, the t-th into stage pw + (t % K) * PW as that stage's use t / K; only
// the latest use of each stage can still be in flight.
__device__ __forceinline__ void drain_producer(uint64_t* full, int pw, int PW, int S, int issued) {
  const int K = S / PW;
  for (int t = issued - 1; t >= 0 && t >= issued - K; --t) mbar_wait_bounded(full + pw + (t % K) * PW, (t / K) & 1);
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Hardware barrier 1 over the first `n` threads of the CTA (the consumers): the producers do not
// take part, so they can start gathering rows while the consumers stage the bias table.
__device__ __forceinline__ void consumer_sync(int n) { asm volatile("bar.sync 1, %0;" ::"r"(n) : "memory"); }

// Barrier among the warps of one consumer group, built on an mbarrier so that the wait is bounded.
__device__ __forceinline__ bool group_barrier(uint64_t* bar, uint32_t& phase, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
  const bool ok = mbar_wait_bounded(bar, phase);
  phase ^= 1;
  return ok;
}

template <typename T>
__device__ __forceinline__ void widen8(const uint4& u, float4& a, float4& b);
template <>
__device__ __forceinline__ void widen8<__nv_bfloat16>(const uint4& u, float4& a, float4& b) {
  a = make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                  __uint_as_float(u.y & 0xffff0000u));
  b = make_float4(__uint_as_float(u.z << 16), __uint_as_float(u.z & 0xffff0000u), __uint_as_float(u.w << 16),
                  __uint_as_float(u.w & 0xffff0000u));
}
template <>
__device__ __forceinline__ void widen8<__half>(const uint4& u, float4& a, float4& b) {
  float2 p0 = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
  float2 p1 = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
  float2 p2 = __half22float2(*reinterpret_cast<const __half2*>(&u.z));
  float2 p3 = __half22float2(*reinterpret_cast<const __half2*>(&u.w));
  a = make_float4(p0.x, p0.y, p1.x, p1.y);
  b = make_float4(p2.x, p2.y, p3.x, p3.y);
}
template <>
__device__ __forceinline__ void widen8<float>(const uint4&, float4&, float4&) {}

template <typename T>
__device__ __forceinline__ T from_float(float f);
template <>
__device__ __forceinline__ float from_float<float>(float f) { return f; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float f) { return __float2bfloat16_rn(f); }
template <>
__device__ __forceinline__ __half from_float<__half>(float f) { return __float2half_rn(f); }

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}


}  // namespace ssw
