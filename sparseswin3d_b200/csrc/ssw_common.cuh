// Shared device/host helpers of the sm_100a sparse window-attention library.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/ssw_b200.h"

namespace ssw {

// ---- host-side error plumbing ---------------------------------------------------------
void set_cuda_error(cudaError_t e, const char* where);
void set_error_text(const char* text);  // shown by ssw_last_cuda_error() next to a non-CUDA status

#define SSW_CUDA_TRY(expr)                                   \
  do {                                                       \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) {                                 \
      ::ssw::set_cuda_error(_e, #expr);                      \
      return SSW_E_CUDA;                                     \
    }                                                        \
  } while (0)

#define SSW_LAUNCH_CHECK(name)                               \
  do {                                                       \
    cudaError_t _e = cudaGetLastError();                     \
    if (_e != cudaSuccess) {                                 \
      ::ssw::set_cuda_error(_e, name);                       \
      return SSW_E_CUDA;                                     \
    }                                                        \
  } while (0)

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- bit layout of one pack_meta entry --------------------------------------------------
// bits 0..9  : in-window position (pos < 1024)
// bits 10..14: shift-mask region id (0..26)
// bits 16..30: relative-position code L = pz*(2Wy-1)(2Wx-1) + py*(2Wx-1) + px, so that the
//              bias-table row of a (query i, key j) pair is L_i - L_j + L(Wz-1,Wy-1,Wx-1).
constexpr int kMetaRegionShift = 10;
constexpr int kMetaRelShift = 16;
constexpr int kMaxPerWindow = 1023;

__host__ __device__ inline int meta_pos(int m) { return m & 1023; }
__host__ __device__ inline int meta_region(int m) { return (m >> kMetaRegionShift) & 31; }
__host__ __device__ inline int meta_rel(int m) { return (m >> kMetaRelShift) & 0x7fff; }

// ---- per-occupancy ("bin") tables: 5 arrays of (n_per_window + 2) ints ---------------------
struct BinTables {
  int32_t* cnt;        // windows with occupancy c
  int32_t* wstart;     // first window slot (pack order) of bin c
  int32_t* rowstart;   // first row (pack order) of bin c
  int32_t* packstart;  // first work item of bin c
  int32_t* fill;       // running slot counter
  __host__ __device__ BinTables(int32_t* base, int n_per_window) {
    int s = n_per_window + 2;
    cnt = base;
    wstart = base + s;
    rowstart = base + 2 * s;
    packstart = base + 3 * s;
    fill = base + 4 * s;
  }
};

// Row slots a window of occupancy c takes inside a pack.  Contiguous plans (CUDA-core kernel) use
// exactly c.  Padded plans (tensor-core kernel) round c up to a power of two below 16 and to a
// multiple of 16 above, so that 16-row MMA tiles never straddle windows of different position.
__host__ __device__ inline int slots_of_window(int c, int padded) {
  if (!padded) return c;
  if (c > 16) return (c + 15) & ~15;
  int s = 1;
  while (s < c) s <<= 1;
  return s;
}
__host__ __device__ inline int windows_per_pack(int c, int tile, int padded) {
  const int w = tile / slots_of_window(c, padded);
  return w > 0 ? w : 1;
}
// Work items a bin of `cnt` windows with occupancy c needs when one item holds `tile` rows.
__host__ __device__ inline int packs_of_bin(int c, int cnt, int tile, int padded) {
  if (cnt == 0 || c == 0) return 0;
  if (c <= tile) {
    int wpp = windows_per_pack(c, tile, padded);
    return (cnt + wpp - 1) / wpp;
  }
  return cnt * ((c + tile - 1) / tile);
}

#ifdef __CUDACC__
// ---- programmatic dependent launch ------------------------------------------------------------
// Kernels of one call are chained with programmatic stream serialization: a kernel may be
// scheduled while its predecessor drains, runs whatever does not depend on the predecessor, and
// calls grid_dependency_wait() before it touches anything the predecessor wrote.  Every kernel
// calls it, so completion is transitive along the chain.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                         Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ---- warp / block primitives ------------------------------------------------------------
__device__ __forceinline__ int warp_incl_scan(int v) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) >= o) v += t;
  }
  return v;
}

// ---- mbarrier + 1-D bulk (TMA) copy wrappers ----------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` polls and reports false (the caller sets an error
// bit and leaves); a healthy copy completes within a few polls.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22)) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}
// global -> shared bulk copy; addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
#endif  // __CUDACC__

}  // namespace ssw
