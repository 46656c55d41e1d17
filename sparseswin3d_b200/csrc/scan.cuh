// Device-wide exclusive prefix sum of int32 values, two launches, no spinning: every block
// reduces its chunk and takes a ticket; the block that draws the last ticket scans the block
// totals; the second launch rescans each chunk on top of its block offset.
#pragma once

#include "ssw_common.cuh"

namespace ssw {

constexpr int kScanT = 256;       // threads per block
constexpr int kScanI = 8;         // items per thread
constexpr int kScanChunk = kScanT * kScanI;

// Workspace (int64 units): [0] ticket, [1] grand total, [2 .. 2+blocks) block offsets.
inline int64_t scan_workspace_i64(int64_t n) { return 2 + ceil_div64(n > 0 ? n : 1, kScanChunk); }

#ifdef __CUDACC__
__device__ __forceinline__ long long block_excl_scan_i64(long long v, long long& total) {
  __shared__ long long warp_tot[kScanT / 32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  long long inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    long long t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) warp_tot[wid] = inc;
  __syncthreads();
  long long base = 0, tot = 0;
#pragma unroll
  for (int i = 0; i < kScanT / 32; ++i) {
    if (i < wid) base += warp_tot[i];
    tot += warp_tot[i];
  }
  total = tot;
  __syncthreads();
  return base + inc - v;
}

// F: int64 index -> int value to be summed (evaluated twice per element).
template <typename F>
__global__ void __launch_bounds__(kScanT) k_scan_reduce(F f, int64_t n, long long* ws, int n_blocks) {
  const int64_t base = (int64_t)blockIdx.x * kScanChunk + (int64_t)threadIdx.x * kScanI;
  long long t = 0;
#pragma unroll
  for (int i = 0; i < kScanI; ++i)
    if (base + i < n) t += f(base + i);
  long long tot;
  block_excl_scan_i64(t, tot);
  __shared__ bool last;
  if (threadIdx.x == 0) {
    ws[2 + blockIdx.x] = tot;
    __threadfence();
    last = atomicAdd(reinterpret_cast<unsigned long long*>(ws), 1ull) == (unsigned long long)(n_blocks - 1);
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  long long carry = 0;
  for (int b0 = 0; b0 < n_blocks; b0 += kScanT) {
    const int b = b0 + threadIdx.x;
    long long v = b < n_blocks ? __ldcg(ws + 2 + b) : 0;
    long long tot2;
    long long ex = block_excl_scan_i64(v, tot2) + carry;
    if (b < n_blocks) ws[2 + b] = ex;
    carry += tot2;
  }
  if (threadIdx.x == 0) {
    ws[1] = carry;
    ws[0] = 0;  // ticket ready for the next use of this workspace
  }
}

// G: (int64 index, int value, long long exclusive prefix) -> void, called for every element.
template <typename F, typename G>
__global__ void __launch_bounds__(kScanT) k_scan_apply(F f, G g, int64_t n, const long long* ws) {
  const int64_t base = (int64_t)blockIdx.x * kScanChunk + (int64_t)threadIdx.x * kScanI;
  int v[kScanI];
  long long t = 0;
#pragma unroll
  for (int i = 0; i < kScanI; ++i) {
    v[i] = base + i < n ? f(base + i) : 0;
    t += v[i];
  }
  long long tot;
  long long ex = block_excl_scan_i64(t, tot) + __ldcg(ws + 2 + blockIdx.x);
#pragma unroll
  for (int i = 0; i < kScanI; ++i) {
    if (base + i < n) g(base + i, v[i], ex);
    ex += v[i];
  }
}

// Runs both launches.  `ws` must hold scan_workspace_i64(n) int64 and ws[0] must be 0 on entry
// (it is reset on exit); the grand total is left in ws[1].
template <typename F, typename G>
static inline int device_scan(F f, G g, int64_t n, long long* ws, cudaStream_t stream) {
  if (n <= 0) return SSW_OK;
  const int blocks = (int)ceil_div64(n, kScanChunk);
  k_scan_reduce<<<blocks, kScanT, 0, stream>>>(f, n, ws, blocks);
  SSW_LAUNCH_CHECK("k_scan_reduce");
  k_scan_apply<<<blocks, kScanT, 0, stream>>>(f, g, n, ws);
  SSW_LAUNCH_CHECK("k_scan_apply");
  return SSW_OK;
}
#endif

}  // namespace ssw
