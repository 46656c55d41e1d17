// Stable argsort of int32 keys (upstream's sort_indices, ops.cu:276-289, a thrust sort_by_key
// over a 0..n-1 sequence): least-significant-digit radix sort, 8 bits per pass, signed order.
//
// Per pass: k_radix_hist counts the digit of every key per 2048-key tile into a digit-major
// table, a device-wide exclusive scan turns the table into global offsets, and k_radix_scatter
// re-reads the tile 256 keys at a time, ranks equal digits in key order (warp match + per-warp
// counters, so the pass is stable) and scatters (key, index) pairs.
#include "scan.cuh"
#include "ssw_common.cuh"

namespace ssw {

constexpr int kRadixBits = 8;
constexpr int kRadix = 1 << kRadixBits;
constexpr int kSortThreads = 256;
constexpr int kSortRounds = 8;
constexpr int kSortTile = kSortThreads * kSortRounds;

__device__ __forceinline__ uint32_t digit_of(int32_t key, int shift) {
  return (((uint32_t)key ^ 0x80000000u) >> shift) & (kRadix - 1);
}

__global__ void __launch_bounds__(kSortThreads) k_radix_hist(const int32_t* __restrict__ keys, int64_t n, int shift,
                                                             int32_t* __restrict__ hist, int n_tiles) {
  __shared__ int cnt[kRadix];
  cnt[threadIdx.x] = 0;
  __syncthreads();
  const int64_t base = (int64_t)blockIdx.x * kSortTile;
#pragma unroll
  for (int r = 0; r < kSortRounds; ++r) {
    const int64_t e = base + r * kSortThreads + threadIdx.x;
    if (e < n) atomicAdd(&cnt[digit_of(keys[e], shift)], 1);
  }
  __syncthreads();
  hist[(int64_t)threadIdx.x * n_tiles + blockIdx.x] = cnt[threadIdx.x];
}

__global__ void __launch_bounds__(kSortThreads) k_radix_scatter(const int32_t* __restrict__ keys_in,
                                                                const int32_t* __restrict__ vals_in, int64_t n,
                                                                int shift, const int32_t* __restrict__ offsets,
                                                                int n_tiles, int32_t* __restrict__ keys_out,
                                                                int32_t* __restrict__ vals_out, int first_pass) {
  __shared__ int base[kRadix];                      // next global slot of each digit for this tile
  __shared__ int wcnt[kSortThreads / 32][kRadix];   // per-warp digit counts of the current round
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  base[threadIdx.x] = offsets[(int64_t)threadIdx.x * n_tiles + blockIdx.x];
  const int64_t tile0 = (int64_t)blockIdx.x * kSortTile;
  for (int r = 0; r < kSortRounds; ++r) {
    for (int i = threadIdx.x; i < (kSortThreads / 32) * kRadix; i += kSortThreads) (&wcnt[0][0])[i] = 0;
    __syncthreads();
    const int64_t e = tile0 + r * kSortThreads + threadIdx.x;
    const bool live = e < n;
    int32_t key = 0, val = 0;
    uint32_t d = 0;
    if (live) {
      key = keys_in[e];
      val = first_pass ? (int32_t)e : vals_in[e];
      d = digit_of(key, shift);
    }
    // lanes with the same digit, in lane (= key) order
    const unsigned peers = __match_any_sync(0xffffffffu, live ? d : 0xffffffffu);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (live && rank_in_warp == 0) wcnt[wid][d] = __popc(peers);
    __syncthreads();
    // exclusive prefix over warps for my digit
    int before = 0;
    if (live)
      for (int w = 0; w < wid; ++w) before += wcnt[w][d];
    if (live) {
      const int dst = base[d] + before + rank_in_warp;
      keys_out[dst] = key;
      vals_out[dst] = val;
    }
    __syncthreads();
    int tot = 0;
#pragma unroll
    for (int w = 0; w < kSortThreads / 32; ++w) tot += wcnt[w][threadIdx.x];
    base[threadIdx.x] += tot;
    __syncthreads();
  }
}

}  // namespace ssw

using namespace ssw;

extern "C" int64_t ssw_argsort_workspace_bytes(int64_t n) {
  if (n <= 0) return 64;
  const int64_t tiles = ceil_div64(n, kSortTile);
  const int64_t table = (int64_t)kRadix * tiles;
  // two key buffers, one value buffer, digit table, scan workspace
  return 4 * (3 * n + table) + 8 * scan_workspace_i64(table) + 64;
}

extern "C" int ssw_argsort_i32(const int32_t* keys, int64_t n, int32_t* perm_out, void* workspace,
                               int64_t workspace_bytes, void* stream) {
  if (n < 0) return SSW_E_INVALID;
  if (n == 0) return SSW_OK;
  if (n >= (int64_t(1) << 31)) return SSW_E_RANGE;
  if (!keys || !perm_out || !workspace) return SSW_E_INVALID;
  if (workspace_bytes < ssw_argsort_workspace_bytes(n)) return SSW_E_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  const int tiles = (int)ceil_div64(n, kSortTile);
  const int64_t table = (int64_t)kRadix * tiles;
  long long* ws = (long long*)workspace;
  const int64_t ws_i64 = scan_workspace_i64(table);
  int32_t* kbuf0 = reinterpret_cast<int32_t*>(ws + ws_i64);
  int32_t* kbuf1 = kbuf0 + n;
  int32_t* vbuf = kbuf1 + n;
  int32_t* hist = vbuf + n;
  SSW_CUDA_TRY(cudaMemsetAsync(ws, 0, 16, st));
  const int32_t* kin = keys;
  const int32_t* vin = nullptr;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = pass * kRadixBits;
    // values ping-pong between vbuf and perm_out so that the last pass lands in perm_out
    int32_t* kout = (pass & 1) ? kbuf1 : kbuf0;
    int32_t* vout = (pass & 1) ? perm_out : vbuf;
    k_radix_hist<<<tiles, kSortThreads, 0, st>>>(kin, n, shift, hist, tiles);
    SSW_LAUNCH_CHECK("k_radix_hist");
    auto f = [hist] __device__(int64_t i) -> int { return hist[i]; };
    auto g = [hist] __device__(int64_t i, int, long long ex) { hist[i] = (int32_t)ex; };
    int rc = device_scan(f, g, table, ws, st);
    if (rc) return rc;
    k_radix_scatter<<<tiles, kSortThreads, 0, st>>>(kin, vin, n, shift, hist, tiles, kout, vout, pass == 0);
    SSW_LAUNCH_CHECK("k_radix_scatter");
    kin = kout;
    vin = vout;
  }
  return SSW_OK;
}
