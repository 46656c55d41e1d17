// Residual add + LayerNorm over voxel rows, the element-wise shell of a Swin block
// (sparse_swin/swin3d_base.py:741-782):
//     x  = shortcut + attention(norm1(shortcut))          (forward, :778-780)
//     x  = x + mlp(norm2(x))                               (forward_part2, :772-775, :781)
// Between two GEMMs of that chain there is always the same pair of row operations: add the branch
// output to the running features, then normalise the sum for the next branch.  ssw_add_layernorm
// does both in one pass over the rows: sum = a (+ b), norm = LayerNorm(sum) * gamma + beta, either
// output optional.  HBM bound: each row is read once per input and written once per output.
//
// A row of C elements is handled by a group of 8, 16 or 32 lanes, 16 bytes per lane and step, values
// kept in registers between the statistics and the normalisation (C * elt <= 32 lanes * 16 B * 4
// steps).  Statistics in fp32, two passes over the registers (mean, then the centred second
// moment), biased variance and eps as torch.nn.LayerNorm has them.
#include "ssw_common.cuh"

namespace ssw {

template <typename T>
__device__ __forceinline__ float round_to(float x);
template <>
__device__ __forceinline__ float round_to<float>(float x) { return x; }
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
template <>
__device__ __forceinline__ float round_to<__half>(float x) { return __half2float(__float2half_rn(x)); }

template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 u = *reinterpret_cast<const float4*>(p);
    v[0] = u.x, v[1] = u.y, v[2] = u.z, v[3] = u.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <>
struct Vec16<__half> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __half* p, float* v) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      v[2 * i] = f.x, v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__half* p, const float* v) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// GL lanes per row, STEPS 16-byte chunks per lane; chunk k of a lane is chunk k * GL + lane-in-group
// of the row, so a group's loads of one step are contiguous.
template <typename T, int GL, int STEPS>
__global__ void __launch_bounds__(256) k_add_layernorm(const T* a, const T* b,
                                                       const float* __restrict__ gamma, const float* __restrict__ beta,
                                                       float eps, int64_t n_rows, int C, T* sum_out, T* norm_out) {
  constexpr int V = Vec16<T>::N;
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int gl = lane % GL;
  const int chunks = C / V;
  const int64_t groups_per_block = blockDim.x / GL;
  const int64_t g0 = (int64_t)blockIdx.x * groups_per_block + threadIdx.x / GL;
  const int64_t g_step = (int64_t)gridDim.x * groups_per_block;
  // the affine parameters of this lane's channels stay in registers for all its rows
  float gm[STEPS][V], bt[STEPS][V];
#pragma unroll
  for (int s = 0; s < STEPS; ++s) {
    const int ch = s * GL + gl;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      gm[s][i] = (norm_out && ch < chunks) ? __ldg(gamma + ch * V + i) : 0.f;
      bt[s][i] = (norm_out && ch < chunks) ? __ldg(beta + ch * V + i) : 0.f;
    }
  }
  const float inv_c = 1.0f / (float)C;
  // every lane of a warp runs the same number of iterations, so the group shuffles are convergent
  const int64_t n_iter = (n_rows + g_step - 1) / g_step;
  for (int64_t it = 0; it < n_iter; ++it) {
    const int64_t row = g0 + it * g_step;
    const bool live = row < n_rows;
    float v[STEPS][V];
    float part = 0.f;
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      const int ch = s * GL + gl;
      const bool on = live && ch < chunks;
#pragma unroll
      for (int i = 0; i < V; ++i) v[s][i] = 0.f;
      if (on) {
        Vec16<T>::load(a + row * C + ch * V, v[s]);
        if (b) {
          float w[V];
          Vec16<T>::load(b + row * C + ch * V, w);
#pragma unroll
          for (int i = 0; i < V; ++i) v[s][i] += w[i];
        }
        // With 16-bit rows the sum that is normalised is the rounded sum the caller sees in sum_out
        // (what a separate add followed by LayerNorm would read), not the fp32 value.
        if (b) {
#pragma unroll
          for (int i = 0; i < V; ++i) v[s][i] = round_to<T>(v[s][i]);
        }
        if (sum_out) Vec16<T>::store(sum_out + row * C + ch * V, v[s]);
      }
    }
    if (!norm_out) continue;
#pragma unroll
    for (int s = 0; s < STEPS; ++s)
#pragma unroll
      for (int i = 0; i < V; ++i) part += v[s][i];
#pragma unroll
    for (int o = GL / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    const float mean = part * inv_c;
    float sq = 0.f;
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      const int ch = s * GL + gl;
      if (ch < chunks) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const float d = v[s][i] - mean;
          sq += d * d;
        }
      }
    }
#pragma unroll
    for (int o = GL / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rstd = rsqrtf(sq * inv_c + eps);
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      const int ch = s * GL + gl;
      if (live && ch < chunks) {
        float y[V];
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] = (v[s][i] - mean) * rstd * gm[s][i] + bt[s][i];
        Vec16<T>::store(norm_out + row * C + ch * V, y);
      }
    }
  }
}

template <typename T, int GL, int STEPS>
static int launch_norm(const void* a, const void* b, const float* gamma, const float* beta, float eps, int64_t n, int C,
                       void* sum_out, void* norm_out, cudaStream_t stream) {
  int dev = 0, sms = 0;
  SSW_CUDA_TRY(cudaGetDevice(&dev));
  SSW_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int64_t groups_per_block = 256 / GL;
  int64_t blocks = ceil_div64(n, groups_per_block);
  const int64_t cap = (int64_t)sms * 8;  // eight resident blocks per SM, rows beyond that by striding
  if (blocks > cap) blocks = cap;
  SSW_CUDA_TRY(launch_chained(k_add_layernorm<T, GL, STEPS>, dim3((unsigned)blocks), dim3(256), 0, stream,
                              reinterpret_cast<const T*>(a), reinterpret_cast<const T*>(b), gamma, beta, eps, n, C,
                              reinterpret_cast<T*>(sum_out), reinterpret_cast<T*>(norm_out)));
  SSW_LAUNCH_CHECK("k_add_layernorm");
  return SSW_OK;
}

template <typename T>
static int dispatch_norm(const void* a, const void* b, const float* gamma, const float* beta, float eps, int64_t n, int C,
                         void* sum_out, void* norm_out, cudaStream_t stream) {
  const int chunks = C / Vec16<T>::N;
#define SSW_NORM_CASE(GL, STEPS) \
  if (chunks <= GL * STEPS) return launch_norm<T, GL, STEPS>(a, b, gamma, beta, eps, n, C, sum_out, norm_out, stream)
  SSW_NORM_CASE(8, 1);
  SSW_NORM_CASE(16, 1);
  SSW_NORM_CASE(32, 1);
  SSW_NORM_CASE(32, 2);
  SSW_NORM_CASE(32, 3);
  SSW_NORM_CASE(32, 4);
#undef SSW_NORM_CASE
  return SSW_E_UNSUPPORTED;
}

}  // namespace ssw

using namespace ssw;

extern "C" int ssw_add_layernorm(const void* a, const void* b, const float* gamma, const float* beta, float eps,
                                 int dtype, int64_t n_rows, int32_t channels, void* sum_out, void* norm_out,
                                 void* stream_) {
  if (n_rows < 0 || channels <= 0) return SSW_E_INVALID;
  if (n_rows == 0) return SSW_OK;
  if (!a || (!sum_out && !norm_out) || (norm_out && (!gamma || !beta))) return SSW_E_INVALID;
  if (!b && sum_out && !norm_out) return SSW_E_INVALID;  // a plain copy is not this call's business
  const int elt = dtype == SSW_F32 ? 4 : (dtype == SSW_BF16 || dtype == SSW_F16) ? 2 : 0;
  if (!elt) return SSW_E_INVALID;
  if ((channels * elt) % 16) return SSW_E_UNSUPPORTED;
  const void* ptrs[4] = {a, b, sum_out, norm_out};
  for (const void* q : ptrs)
    if (q && (reinterpret_cast<uintptr_t>(q) & 15)) return SSW_E_INVALID;
  if (n_rows * (int64_t)channels >= (int64_t)1 << 40) return SSW_E_RANGE;
  cudaStream_t stream = (cudaStream_t)stream_;
  switch (dtype) {
    case SSW_F32: return dispatch_norm<float>(a, b, gamma, beta, eps, n_rows, channels, sum_out, norm_out, stream);
    case SSW_BF16: return dispatch_norm<__nv_bfloat16>(a, b, gamma, beta, eps, n_rows, channels, sum_out, norm_out, stream);
    case SSW_F16: return dispatch_norm<__half>(a, b, gamma, beta, eps, n_rows, channels, sum_out, norm_out, stream);
  }
  return SSW_E_INVALID;
}
