// COO-emitting operators: the unfused operator surface upstream exports from sparse_swin/ops.cpp,
// rebuilt on the window bucketing instead of radix sorts over N*C keys, cuSPARSE transposes and
// ATen unique/bincount chains.  Layouts and index conventions are upstream's, bit for bit:
// int32 indices everywhere, q/v values ordered (window, head, pos, ch), k ordered
// (window, head, ch, pos), attention values ordered (window, head, pos_i, pos_j).
#include <math.h>

#include "scan.cuh"
#include "ssw_common.cuh"

namespace ssw {

// ---------------------------------------------------------------------------------------------
// flatten_indices (ops.cu:232-273): row-major hash accumulated in int32 (wraps like upstream)
// ---------------------------------------------------------------------------------------------
struct Strides {
  uint32_t s[8];
};
__global__ void k_flatten(const int32_t* __restrict__ idx, int D, int64_t nnz, Strides st, int32_t* __restrict__ out) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= nnz) return;
  uint32_t h = 0;
  for (int d = 0; d < D; ++d) h += (uint32_t)__ldg(idx + (int64_t)d * nnz + e) * st.s[d];
  out[e] = (int32_t)h;
}

// ---------------------------------------------------------------------------------------------
// return_inverse (ops.cu:718-730): presence bitmap -> popcount prefix -> rank
// ---------------------------------------------------------------------------------------------
__global__ void k_mark(const int32_t* __restrict__ x, int64_t n, int64_t maxnum, uint32_t* __restrict__ bitmap,
                       int32_t* __restrict__ err) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  const int32_t v = x[e];
  if (v < 0 || v >= maxnum) {
    atomicOr(reinterpret_cast<unsigned*>(err), SSW_DEV_BAD_COORD);
    return;
  }
  atomicOr(bitmap + (v >> 5), 1u << (v & 31));
}
__global__ void k_rank(const int32_t* __restrict__ x, int64_t n, int64_t maxnum, const uint32_t* __restrict__ bitmap,
                       const int32_t* __restrict__ word_prefix, int32_t* __restrict__ out) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  const int32_t v = x[e];
  if (v < 0 || v >= maxnum) {
    out[e] = 0;
    return;
  }
  out[e] = word_prefix[v >> 5] + __popc(bitmap[v >> 5] & ((1u << (v & 31)) - 1u));
}
__global__ void k_store_total(const long long* ws, int32_t* out) { out[0] = (int32_t)ws[1]; }

// ---------------------------------------------------------------------------------------------
// qkv_sparse_indices (ops.cu:206-227, 293-335)
// ---------------------------------------------------------------------------------------------
// unsorted index blocks, element order (voxel, head, channel)
__global__ void k_expand(const int32_t* __restrict__ indices, int64_t M, int hc, int c, int32_t* __restrict__ qv,
                         int32_t* __restrict__ k) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= M) return;
  const int64_t v = e / hc;
  const int local = (int)(e - v * hc);
  const int h = local / c, ch = local - h * c;
  const int2 wp = __ldg(reinterpret_cast<const int2*>(indices) + v);
  qv[e] = wp.x;  k[e] = wp.x;
  qv[M + e] = h; k[M + e] = h;
  qv[2 * M + e] = wp.y; k[2 * M + e] = ch;
  qv[3 * M + e] = ch;   k[3 * M + e] = wp.y;
}
// argsort permutations straight from the window bucketing: the element that lands at sorted
// position (window k, head h, row i, channel ch) is voxel perm[start_k + i]'s (h, ch) element.
__global__ void k_qkv_perms(const int32_t* __restrict__ header, const int32_t* __restrict__ perm,
                            const int32_t* __restrict__ win_start, int64_t M, int H, int c,
                            int32_t* __restrict__ perm_qv, int32_t* __restrict__ perm_k) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= M) return;
  const int hc = H * c;
  const int s = (int)(e / hc);  // sorted row
  const int local = (int)(e - (int64_t)s * hc);
  const int h = local / c, ch = local - h * c;
  int lo = 0, hi = header[SSW_H_W];  // window k with win_start[k] <= s < win_start[k+1]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (win_start[mid] <= s) lo = mid; else hi = mid;
  }
  const int start = win_start[lo], cw = win_start[lo + 1] - start, i = s - start;
  const int64_t base = (int64_t)start * hc + (int64_t)h * cw * c;
  const int32_t src = perm[s] * hc + local;
  perm_qv[base + (int64_t)i * c + ch] = src;
  perm_k[base + (int64_t)ch * cw + i] = src;
}

// ---------------------------------------------------------------------------------------------
// block structure of a coalesced COO operand: rows of `row_len` elements, a block = a run of
// rows with equal (idx[0], idx[1]) = (window, head)
// ---------------------------------------------------------------------------------------------
__global__ void k_finish_blocks(const long long* ws, int32_t* blk_start, int64_t R, long long* counts) {
  const long long nb = ws[1];
  blk_start[nb] = (int32_t)R;
  counts[0] = nb;
}
__global__ void k_finish_sq(const long long* ws, int32_t* sq_start, const long long* counts_nb, long long* counts) {
  sq_start[counts_nb[0]] = (int32_t)ws[1];
  counts[1] = ws[1];
}
__global__ void k_block_counts(const int32_t* __restrict__ blk_start, const long long* __restrict__ counts,
                               int32_t* __restrict__ c_out) {
  const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b < counts[0]) c_out[b] = blk_start[b + 1] - blk_start[b];
}

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// q_k (ops.cu:344-378): per block A[c,C] . Kt[C,c] -> [c,c]; sequential FMA chain over the channel,
// the order upstream's kernel uses.  One CTA per block.
template <typename T>
__global__ void k_matmul_qk(const T* __restrict__ m1, const int32_t* __restrict__ idx1, int64_t nnz1,
                            const T* __restrict__ m2, const int32_t* __restrict__ blk_start,
                            const int32_t* __restrict__ sq_start, int C, T* __restrict__ out_v,
                            int32_t* __restrict__ out_idx, int64_t total) {
  const int b = blockIdx.x;
  const int r0 = blk_start[b], c = blk_start[b + 1] - r0;
  const int64_t mat = (int64_t)r0 * C;
  const int64_t o0 = sq_start[b];
  const int w = idx1[mat], h = idx1[nnz1 + mat];
  for (int t = threadIdx.x; t < c * c; t += blockDim.x) {
    const int i = t / c, j = t - i * c;
    float s = 0.f;
    for (int k = 0; k < C; ++k) s = fmaf(to_f(m1[mat + (int64_t)i * C + k]), to_f(m2[mat + (int64_t)k * c + j]), s);
    out_v[o0 + t] = from_f<T>(s);
    out_idx[o0 + t] = w;
    out_idx[total + o0 + t] = h;
    out_idx[2 * total + o0 + t] = idx1[2 * nnz1 + mat + (int64_t)i * C];
    out_idx[3 * total + o0 + t] = idx1[2 * nnz1 + mat + (int64_t)j * C];
  }
}
// qk_v (ops.cu:381-418): per block P[c,c] . V[c,C] -> [c,C]
template <typename T>
__global__ void k_matmul_pv(const T* __restrict__ m1, const int32_t* __restrict__ idx1, int64_t nnz1,
                            const T* __restrict__ m2, const int32_t* __restrict__ blk_start,
                            const int32_t* __restrict__ sq_start, int C, T* __restrict__ out_v,
                            int32_t* __restrict__ out_idx, int64_t total) {
  const int b = blockIdx.x;
  const int r0 = blk_start[b], c = blk_start[b + 1] - r0;
  const int64_t mat = (int64_t)r0 * C;
  const int64_t p0 = sq_start[b];
  const int w = idx1[p0], h = idx1[nnz1 + p0];
  for (int t = threadIdx.x; t < c * C; t += blockDim.x) {
    const int i = t / C, ch = t - i * C;
    float s = 0.f;
    for (int k = 0; k < c; ++k) s = fmaf(to_f(m1[p0 + (int64_t)i * c + k]), to_f(m2[mat + (int64_t)k * C + ch]), s);
    out_v[mat + t] = from_f<T>(s);
    out_idx[mat + t] = w;
    out_idx[total + mat + t] = h;
    out_idx[2 * total + mat + t] = idx1[2 * nnz1 + p0 + (int64_t)i * c];
    out_idx[3 * total + mat + t] = ch;
  }
}

// Backward matmuls (ops.cu:422-515): out[i,j] = sum_k m1[i*K+k] * m2[j*K+k] with per-block shapes
//   mode 0 "rc_cr": (I,J,K) = (c,c,C)   mode 1 "rr_rc": (c,C,c)   mode 2 "cr_rr": (C,c,c)
template <typename T>
__global__ void k_matmul_grad(const T* __restrict__ m1, const T* __restrict__ m2, const int32_t* __restrict__ cstart,
                              const int32_t* __restrict__ sqstart, int C, int mode, T* __restrict__ out) {
  const int b = blockIdx.x;
  const int c = cstart[b + 1] - cstart[b];
  const int64_t lin = (int64_t)cstart[b] * C, sq = sqstart[b];
  int I, J, K;
  int64_t o0, a0, b0;
  if (mode == 0) { I = c; J = c; K = C; o0 = sq; a0 = lin; b0 = lin; }
  else if (mode == 1) { I = c; J = C; K = c; o0 = lin; a0 = sq; b0 = lin; }
  else { I = C; J = c; K = c; o0 = lin; a0 = lin; b0 = sq; }
  for (int t = threadIdx.x; t < I * J; t += blockDim.x) {
    const int i = t / J, j = t - i * J;
    float s = 0.f;
    for (int k = 0; k < K; ++k) s = fmaf(to_f(m1[a0 + (int64_t)i * K + k]), to_f(m2[b0 + (int64_t)j * K + k]), s);
    out[o0 + t] = from_f<T>(s);
  }
}
// Blocked transposes (ops.cu:518-557): "rc": [c,C] -> [C,c]; "rr": [c,c] -> transposed
template <typename T>
__global__ void k_block_transpose(const T* __restrict__ m1, const int32_t* __restrict__ cstart,
                                  const int32_t* __restrict__ sqstart, int C, int rr, T* __restrict__ out) {
  const int b = blockIdx.x;
  const int c = cstart[b + 1] - cstart[b];
  const int64_t o0 = rr ? (int64_t)sqstart[b] : (int64_t)cstart[b] * C;
  const int I = rr ? c : C;  // rows of the output block
  for (int t = threadIdx.x; t < I * c; t += blockDim.x) {
    const int i = t / c, j = t - i * c;
    out[o0 + t] = m1[o0 + i + (int64_t)j * I];
  }
}

// ---------------------------------------------------------------------------------------------
// row-wise sparse softmax (ops.cu:128-194); one warp per row
// ---------------------------------------------------------------------------------------------
__global__ void k_row_starts(const int32_t* __restrict__ ids, int64_t nnz, int32_t* __restrict__ row_start) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= nnz) return;
  const int id = ids[e];
  if (e == 0 || ids[e - 1] != id) row_start[id] = (int32_t)e;
  if (e == nnz - 1) row_start[id + 1] = (int32_t)nnz;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__global__ void k_softmax_fwd(const int32_t* __restrict__ row_start, int n_rows, const float* __restrict__ v,
                              float* __restrict__ out) {
  const int row = (int)(((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const int a = row_start[row], b = row_start[row + 1];
  float m = 0.f;  // upstream's scatter-max starts from zeros (ops.cu:137)
  for (int e = a + lane; e < b; e += 32) m = fmaxf(m, v[e]);
  m = warp_max(m);
  float s = 0.f;
  for (int e = a + lane; e < b; e += 32) s += expf(v[e] - m);
  s = warp_sum(s) + 1e-8f;  // ops.cu:164
  for (int e = a + lane; e < b; e += 32) out[e] = expf(v[e] - m) / s;
}
__global__ void k_softmax_bwd(const int32_t* __restrict__ row_start, int n_rows, const float* __restrict__ y,
                              const float* __restrict__ g, float* __restrict__ out) {
  const int row = (int)(((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const int a = row_start[row], b = row_start[row + 1];
  float s = 0.f;
  for (int e = a + lane; e < b; e += 32) s += g[e] * y[e];
  s = warp_sum(s);
  for (int e = a + lane; e < b; e += 32) out[e] = g[e] * y[e] - y[e] * s;
}

// ---------------------------------------------------------------------------------------------
// sp_add_rpb / sp_add_mask (swin3d_base.py:557-581) as one pass over the COO values
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void k_add_bias_mask(const T* __restrict__ v, const int32_t* __restrict__ idx, int64_t nnz,
                                const T* __restrict__ dense, int n, const int8_t* __restrict__ mask, int mask_windows,
                                int mask_n, T* __restrict__ out) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= nnz) return;
  const int w = idx[e], h = idx[nnz + e], pi = idx[2 * nnz + e], pj = idx[3 * nnz + e];
  float x = to_f(v[e]);
  if (dense) x = to_f(from_f<T>(x + to_f(dense[((int64_t)h * n + pi) * n + pj])));
  if (mask) {
    const int64_t base = (int64_t)(w % mask_windows) * mask_n;
    if (mask[base + pi] != mask[base + pj]) x += -100.0f;
  }
  out[e] = from_f<T>(x);
}

template <typename T>
static int run_matmul(int is_pv, const void* m1, const int32_t* idx1, int64_t nnz1, const void* m2,
                      const int32_t* blk_start, const int32_t* sq_start, int64_t nb, int C, void* out_v,
                      int32_t* out_idx, int64_t total, cudaStream_t st) {
  if (nb == 0) return SSW_OK;
  if (is_pv)
    k_matmul_pv<T><<<(unsigned)nb, 128, 0, st>>>((const T*)m1, idx1, nnz1, (const T*)m2, blk_start, sq_start, C,
                                                 (T*)out_v, out_idx, total);
  else
    k_matmul_qk<T><<<(unsigned)nb, 128, 0, st>>>((const T*)m1, idx1, nnz1, (const T*)m2, blk_start, sq_start, C,
                                                 (T*)out_v, out_idx, total);
  SSW_LAUNCH_CHECK("k_matmul");
  return SSW_OK;
}

}  // namespace ssw

using namespace ssw;

#define BLOCKS(n) ((unsigned)ceil_div64((n), 256))

extern "C" int ssw_flatten_indices(const int32_t* indices, int32_t D, int64_t nnz, const int32_t* sizes, int32_t* out,
                                   void* stream) {
  if (D < 1 || D > 8 || nnz < 0 || !sizes) return SSW_E_INVALID;
  if (nnz == 0) return SSW_OK;
  if (!indices || !out) return SSW_E_INVALID;
  Strides st;
  uint32_t s = 1;
  for (int d = D - 1; d >= 0; --d) {  // strides are int32 products of the trailing sizes (ops.cu:237-245)
    st.s[d] = s;
    s *= (uint32_t)sizes[d];
  }
  k_flatten<<<BLOCKS(nnz), 256, 0, (cudaStream_t)stream>>>(indices, D, nnz, st, out);
  SSW_LAUNCH_CHECK("k_flatten");
  return SSW_OK;
}

extern "C" int64_t ssw_scan_workspace_bytes(int64_t n) { return 8 * scan_workspace_i64(n); }

extern "C" int ssw_unique_consecutive_inverse(const int32_t* x, int64_t n, int32_t* out, void* workspace,
                                              int64_t workspace_bytes, void* stream) {
  if (n < 0) return SSW_E_INVALID;
  if (n == 0) return SSW_OK;
  if (!x || !out || !workspace) return SSW_E_INVALID;
  if (workspace_bytes < ssw_scan_workspace_bytes(n)) return SSW_E_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  long long* ws = (long long*)workspace;
  SSW_CUDA_TRY(cudaMemsetAsync(ws, 0, 16, st));
  auto f = [x] __device__(int64_t e) -> int { return e > 0 && x[e] != x[e - 1]; };
  auto g = [out] __device__(int64_t e, int v, long long ex) { out[e] = (int32_t)(ex + v); };
  return device_scan(f, g, n, ws, st);
}

extern "C" int64_t ssw_return_inverse_workspace_bytes(int64_t maxnum) {
  const int64_t words = ceil_div64(maxnum > 0 ? maxnum : 1, 32);
  return 8 * scan_workspace_i64(words) + 8 * words + 16;
}
// rank_out[i] = number of distinct values < x[i] present in x; count_out[0] (device) = number of
// distinct values; err (device int32, may be NULL... must be non-NULL) flags values outside [0, maxnum).
extern "C" int ssw_return_inverse(const int32_t* x, int64_t n, int64_t maxnum, int32_t* rank_out, int32_t* count_out,
                                  int32_t* err, void* workspace, int64_t workspace_bytes, void* stream) {
  if (n < 0 || maxnum <= 0 || !count_out || !err || !workspace) return SSW_E_INVALID;
  if (maxnum >= (int64_t(1) << 31)) return SSW_E_RANGE;
  if (workspace_bytes < ssw_return_inverse_workspace_bytes(maxnum)) return SSW_E_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t words = ceil_div64(maxnum, 32);
  long long* ws = (long long*)workspace;
  const int64_t ws_i64 = scan_workspace_i64(words);
  uint32_t* bitmap = reinterpret_cast<uint32_t*>(ws + ws_i64);
  int32_t* prefix = reinterpret_cast<int32_t*>(bitmap + words);
  SSW_CUDA_TRY(cudaMemsetAsync(ws, 0, 16, st));
  SSW_CUDA_TRY(cudaMemsetAsync(bitmap, 0, 4 * words, st));
  if (n > 0) {
    k_mark<<<BLOCKS(n), 256, 0, st>>>(x, n, maxnum, bitmap, err);
    SSW_LAUNCH_CHECK("k_mark");
  }
  auto f = [bitmap] __device__(int64_t w) -> int { return __popc(bitmap[w]); };
  auto g = [prefix] __device__(int64_t w, int, long long ex) { prefix[w] = (int32_t)ex; };
  int rc = device_scan(f, g, words, ws, st);
  if (rc) return rc;
  k_store_total<<<1, 1, 0, st>>>(ws, count_out);
  if (n > 0) {
    k_rank<<<BLOCKS(n), 256, 0, st>>>(x, n, maxnum, bitmap, prefix, rank_out);
    SSW_LAUNCH_CHECK("k_rank");
  }
  return SSW_OK;
}

extern "C" int ssw_qkv_sparse_indices(const int32_t* indices, int64_t n_vox, int32_t heads, int32_t c,
                                      const ssw_plan_layout* L, const int32_t* plan, int32_t* idx_qv,
                                      int32_t* perm_qv, int32_t* idx_k, int32_t* perm_k, void* stream) {
  if (n_vox < 0 || heads <= 0 || c <= 0 || !L || !plan) return SSW_E_INVALID;
  const int64_t M = n_vox * heads * c;
  if (M >= (int64_t(1) << 31)) return SSW_E_RANGE;
  if (M == 0) return SSW_OK;
  if (!indices || !idx_qv || !perm_qv || !idx_k || !perm_k || L->n_vox != n_vox) return SSW_E_INVALID;
  cudaStream_t st = (cudaStream_t)stream;
  k_expand<<<BLOCKS(M), 256, 0, st>>>(indices, M, heads * c, c, idx_qv, idx_k);
  SSW_LAUNCH_CHECK("k_expand");
  k_qkv_perms<<<BLOCKS(M), 256, 0, st>>>(plan + L->off_header, plan + L->off_perm, plan + L->off_win_start, M, heads,
                                         c, perm_qv, perm_k);
  SSW_LAUNCH_CHECK("k_qkv_perms");
  return SSW_OK;
}

extern "C" int64_t ssw_coo_plan_workspace_bytes(int64_t n_rows) { return 8 * scan_workspace_i64(n_rows + 1) + 64; }

// Block structure of a coalesced operand: idx [4, nnz], rows of `row_len` consecutive elements.
//   blk_start [n_rows + 1]: first row of every block, then n_rows
//   sq_start  [n_rows + 1]: exclusive sums of c_b^2
//   counts (device int64[2]): number of blocks, sum of c_b^2
extern "C" int ssw_coo_block_plan(const int32_t* idx, int64_t nnz, int32_t row_len, int32_t* blk_start,
                                  int32_t* sq_start, int64_t* counts, void* workspace, int64_t workspace_bytes,
                                  void* stream) {
  if (nnz < 0 || row_len <= 0 || nnz % row_len || !counts || !workspace) return SSW_E_INVALID;
  const int64_t R = nnz / row_len;
  if (workspace_bytes < ssw_coo_plan_workspace_bytes(R)) return SSW_E_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  long long* ws = (long long*)workspace;
  SSW_CUDA_TRY(cudaMemsetAsync(ws, 0, 16, st));
  SSW_CUDA_TRY(cudaMemsetAsync(counts, 0, 16, st));
  if (R == 0) return SSW_OK;
  if (!idx || !blk_start || !sq_start) return SSW_E_INVALID;
  const int32_t* i0 = idx;
  const int32_t* i1 = idx + nnz;
  const int64_t rl = row_len;
  auto f = [i0, i1, rl] __device__(int64_t r) -> int {
    if (r == 0) return 1;
    return i0[r * rl] != i0[(r - 1) * rl] || i1[r * rl] != i1[(r - 1) * rl];
  };
  auto g = [blk_start] __device__(int64_t r, int v, long long ex) {
    if (v) blk_start[ex] = (int32_t)r;
  };
  int rc = device_scan(f, g, R, ws, st);
  if (rc) return rc;
  k_finish_blocks<<<1, 1, 0, st>>>(ws, blk_start, R, (long long*)counts);
  const long long* cnt = (const long long*)counts;
  auto f2 = [blk_start, cnt] __device__(int64_t b) -> int {
    if (b >= cnt[0]) return 0;
    const int c = blk_start[b + 1] - blk_start[b];
    return c * c;
  };
  auto g2 = [sq_start, cnt] __device__(int64_t b, int, long long ex) {
    if (b < cnt[0]) sq_start[b] = (int32_t)ex;
  };
  rc = device_scan(f2, g2, R, ws, st);
  if (rc) return rc;
  k_finish_sq<<<1, 1, 0, st>>>(ws, sq_start, cnt, (long long*)counts);
  SSW_LAUNCH_CHECK("k_finish_sq");
  return SSW_OK;
}

// mul_type 0 = "q_k", 1 = "qk_v".  idx1/nnz1 belong to the LHS.  `n_blocks`, `total` (= sum c^2
// for q_k, nnz of the RHS for qk_v) are the host copies of what ssw_coo_block_plan counted.
extern "C" int ssw_coo_matmul(int mul_type, int dtype, const void* m1_v, const int32_t* m1_idx, int64_t nnz1,
                              const void* m2_v, int32_t C, const int32_t* blk_start, const int32_t* sq_start,
                              int64_t n_blocks, int64_t total, void* out_v, int32_t* out_idx, int32_t* c_out,
                              const int64_t* counts, void* stream) {
  if ((mul_type != 0 && mul_type != 1) || C <= 0 || n_blocks < 0 || total < 0) return SSW_E_INVALID;
  if (total >= (int64_t(1) << 31)) return SSW_E_RANGE;
  if (n_blocks == 0) return SSW_OK;
  if (!m1_v || !m1_idx || !m2_v || !blk_start || !sq_start || !out_v || !out_idx || !c_out || !counts)
    return SSW_E_INVALID;
  cudaStream_t st = (cudaStream_t)stream;
  k_block_counts<<<BLOCKS(n_blocks), 256, 0, st>>>(blk_start, (const long long*)counts, c_out);
  SSW_LAUNCH_CHECK("k_block_counts");
  switch (dtype) {
    case SSW_F32: return run_matmul<float>(mul_type, m1_v, m1_idx, nnz1, m2_v, blk_start, sq_start, n_blocks, C, out_v, out_idx, total, st);
    case SSW_F16: return run_matmul<__half>(mul_type, m1_v, m1_idx, nnz1, m2_v, blk_start, sq_start, n_blocks, C, out_v, out_idx, total, st);
    case SSW_BF16: return run_matmul<__nv_bfloat16>(mul_type, m1_v, m1_idx, nnz1, m2_v, blk_start, sq_start, n_blocks, C, out_v, out_idx, total, st);
  }
  return SSW_E_INVALID;
}

// Offsets from a `_c` vector: cstart[nb+1] = exclusive sums of c, sqstart[nb+1] of c^2.
extern "C" int ssw_coo_offsets_from_counts(const int32_t* c, int64_t nb, int32_t* cstart, int32_t* sqstart,
                                           void* workspace, int64_t workspace_bytes, void* stream) {
  if (nb < 0 || !workspace) return SSW_E_INVALID;
  if (workspace_bytes < ssw_coo_plan_workspace_bytes(nb)) return SSW_E_WORKSPACE;
  if (!cstart || !sqstart || (nb > 0 && !c)) return SSW_E_INVALID;
  cudaStream_t st = (cudaStream_t)stream;
  long long* ws = (long long*)workspace;
  SSW_CUDA_TRY(cudaMemsetAsync(ws, 0, 16, st));
  // one extra element so that the totals land in slot nb
  auto f = [c, nb] __device__(int64_t b) -> int { return b < nb ? c[b] : 0; };
  auto g = [cstart] __device__(int64_t b, int, long long ex) { cstart[b] = (int32_t)ex; };
  int rc = device_scan(f, g, nb + 1, ws, st);
  if (rc) return rc;
  auto f2 = [c, nb] __device__(int64_t b) -> int { return b < nb ? c[b] * c[b] : 0; };
  auto g2 = [sqstart] __device__(int64_t b, int, long long ex) { sqstart[b] = (int32_t)ex; };
  return device_scan(f2, g2, nb + 1, ws, st);
}

template <typename T>
static int grad_t(int mode, const void* m1, const void* m2, const int32_t* cs, const int32_t* ss, int64_t nb, int C,
                  void* out, cudaStream_t st) {
  k_matmul_grad<T><<<(unsigned)nb, 128, 0, st>>>((const T*)m1, (const T*)m2, cs, ss, C, mode, (T*)out);
  SSW_LAUNCH_CHECK("k_matmul_grad");
  return SSW_OK;
}
// mode 0 "rc_cr", 1 "rr_rc", 2 "cr_rr" (ops.cu:945-1031)
extern "C" int ssw_coo_matmul_grad(int mode, int dtype, const void* m1_v, const void* m2_v, const int32_t* cstart,
                                   const int32_t* sqstart, int64_t nb, int32_t C, void* out_v, void* stream) {
  if (mode < 0 || mode > 2 || C <= 0 || nb < 0) return SSW_E_INVALID;
  if (nb == 0) return SSW_OK;
  if (!m1_v || !m2_v || !cstart || !sqstart || !out_v) return SSW_E_INVALID;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case SSW_F32: return grad_t<float>(mode, m1_v, m2_v, cstart, sqstart, nb, C, out_v, st);
    case SSW_F16: return grad_t<__half>(mode, m1_v, m2_v, cstart, sqstart, nb, C, out_v, st);
    case SSW_BF16: return grad_t<__nv_bfloat16>(mode, m1_v, m2_v, cstart, sqstart, nb, C, out_v, st);
  }
  return SSW_E_INVALID;
}

template <typename T>
static int transpose_t(int rr, const void* m1, const int32_t* cs, const int32_t* ss, int64_t nb, int C, void* out,
                       cudaStream_t st) {
  k_block_transpose<T><<<(unsigned)nb, 128, 0, st>>>((const T*)m1, cs, ss, C, rr, (T*)out);
  SSW_LAUNCH_CHECK("k_block_transpose");
  return SSW_OK;
}
// rr = 0: "rc" ([c,C] -> [C,c]);  rr = 1: "rr" ([c,c] transposed)  (ops.cu:663-715)
extern "C" int ssw_coo_block_transpose(int rr, int dtype, const void* m1_v, const int32_t* cstart,
                                       const int32_t* sqstart, int64_t nb, int32_t C, void* out_v, void* stream) {
  if ((rr != 0 && rr != 1) || C <= 0 || nb < 0) return SSW_E_INVALID;
  if (nb == 0) return SSW_OK;
  if (!m1_v || !cstart || !sqstart || !out_v) return SSW_E_INVALID;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case SSW_F32: return transpose_t<float>(rr, m1_v, cstart, sqstart, nb, C, out_v, st);
    case SSW_F16: return transpose_t<__half>(rr, m1_v, cstart, sqstart, nb, C, out_v, st);
    case SSW_BF16: return transpose_t<__nv_bfloat16>(rr, m1_v, cstart, sqstart, nb, C, out_v, st);
  }
  return SSW_E_INVALID;
}

// row_ids: sorted, consecutive from 0 (the output of ssw_unique_consecutive_inverse); n_rows =
// row_ids[nnz-1] + 1; row_start: caller-provided [n_rows + 1] int32.
extern "C" int ssw_softmax_rows_fwd(const int32_t* row_ids, int64_t nnz, int32_t n_rows, const float* vals, float* out,
                                    int32_t* row_start, void* stream) {
  if (nnz < 0 || n_rows < 0) return SSW_E_INVALID;
  if (nnz == 0) return SSW_OK;
  if (!row_ids || !vals || !out || !row_start || n_rows == 0) return SSW_E_INVALID;
  cudaStream_t st = (cudaStream_t)stream;
  k_row_starts<<<BLOCKS(nnz), 256, 0, st>>>(row_ids, nnz, row_start);
  SSW_LAUNCH_CHECK("k_row_starts");
  k_softmax_fwd<<<BLOCKS((int64_t)n_rows * 32), 256, 0, st>>>(row_start, n_rows, vals, out);
  SSW_LAUNCH_CHECK("k_softmax_fwd");
  return SSW_OK;
}
extern "C" int ssw_softmax_rows_bwd(const int32_t* row_ids, int64_t nnz, int32_t n_rows, const float* y, const float* g,
                                    float* out, int32_t* row_start, void* stream) {
  if (nnz < 0 || n_rows < 0) return SSW_E_INVALID;
  if (nnz == 0) return SSW_OK;
  if (!row_ids || !y || !g || !out || !row_start || n_rows == 0) return SSW_E_INVALID;
  cudaStream_t st = (cudaStream_t)stream;
  k_row_starts<<<BLOCKS(nnz), 256, 0, st>>>(row_ids, nnz, row_start);
  SSW_LAUNCH_CHECK("k_row_starts");
  k_softmax_bwd<<<BLOCKS((int64_t)n_rows * 32), 256, 0, st>>>(row_start, n_rows, y, g, out);
  SSW_LAUNCH_CHECK("k_softmax_bwd");
  return SSW_OK;
}

// vals + dense[h, pos_i, pos_j] (dense may be NULL) and -100 where the two positions lie in
// different mask regions (mask may be NULL).  idx [4, nnz] = (window, head, pos_i, pos_j).
extern "C" int ssw_coo_add_bias_mask(int dtype, const void* vals, const int32_t* idx, int64_t nnz, const void* dense,
                                     int32_t n, const int8_t* mask, int32_t mask_windows, int32_t mask_n, void* out,
                                     void* stream) {
  if (nnz < 0) return SSW_E_INVALID;
  if (nnz == 0) return SSW_OK;
  if (!vals || !idx || !out || (mask && (mask_windows <= 0 || mask_n <= 0)) || (dense && n <= 0)) return SSW_E_INVALID;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case SSW_F32:
      k_add_bias_mask<float><<<BLOCKS(nnz), 256, 0, st>>>((const float*)vals, idx, nnz, (const float*)dense, n, mask,
                                                          mask_windows, mask_n, (float*)out);
      break;
    case SSW_F16:
      k_add_bias_mask<__half><<<BLOCKS(nnz), 256, 0, st>>>((const __half*)vals, idx, nnz, (const __half*)dense, n, mask,
                                                           mask_windows, mask_n, (__half*)out);
      break;
    case SSW_BF16:
      k_add_bias_mask<__nv_bfloat16><<<BLOCKS(nnz), 256, 0, st>>>((const __nv_bfloat16*)vals, idx, nnz,
                                                                  (const __nv_bfloat16*)dense, n, mask, mask_windows,
                                                                  mask_n, (__nv_bfloat16*)out);
      break;
    default: return SSW_E_INVALID;
  }
  SSW_LAUNCH_CHECK("k_add_bias_mask");
  return SSW_OK;
}
