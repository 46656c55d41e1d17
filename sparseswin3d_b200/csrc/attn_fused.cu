// Fused window attention for sparse voxel windows: QK^T, relative-position bias, shift mask,
// row softmax (upstream semantics: max starts at 0, denominator + 1e-8) and P.V in one kernel.
//
// CUDA-core path.  One CTA = one work item of the plan: either a *pack* of several windows that
// all hold exactly c voxels (c <= tile), or one tile of query rows of a window with c > tile.
// Thread (h, r) owns query row r of head h: its q row lives in registers, the K|V halves of the
// item's voxel rows are gathered into shared memory with one 1-D bulk (TMA) copy per voxel
// (2*C contiguous elements: k and v sit side by side in the qkv row), and the thread walks the
// keys of its own window with a chunked online softmax.  Scores are accumulated as a sequential
// FMA chain over the head channels, the order upstream's kernel uses (ops.cu:371-375).
#include <math.h>

#include <type_traits>

#include "ssw_common.cuh"

namespace ssw {

struct AttnParams {
  const void* qkv;
  void* out;
  void* attn_vals;
  int32_t* header;
  const int4* pack_desc;
  const int32_t* pack_perm;
  const int32_t* pack_meta;
  const int32_t* pack_win;
  const int32_t* coo_start;
  const float* table;
  int rel_off;
  int H, C, tile;
  float scale;
  int use_mask;
  int row_stride;  // bytes between staged K|V rows in shared memory
};

template <typename T>
struct Elt;
template <>
struct Elt<float> {
  static constexpr int kVec = 4;  // elements per 16-byte vector
  __device__ static void unpack(const uint4& u, float* f) {
    f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y);
    f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
  }
  __device__ static uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  __device__ static float round_trip(float x) { return x; }
};
template <>
struct Elt<__nv_bfloat16> {
  static constexpr int kVec = 8;
  __device__ static void unpack(const uint4& u, float* f) {
    f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xffff0000u);
    f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xffff0000u);
    f[4] = __uint_as_float(u.z << 16); f[5] = __uint_as_float(u.z & 0xffff0000u);
    f[6] = __uint_as_float(u.w << 16); f[7] = __uint_as_float(u.w & 0xffff0000u);
  }
  __device__ static uint32_t pk(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ static uint4 pack(const float* f) {
    return make_uint4(pk(f[0], f[1]), pk(f[2], f[3]), pk(f[4], f[5]), pk(f[6], f[7]));
  }
  __device__ static float round_trip(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};
template <>
struct Elt<__half> {
  static constexpr int kVec = 8;
  __device__ static void up(uint32_t w, float* f) {
    __half2 h = *reinterpret_cast<__half2*>(&w);
    float2 v = __half22float2(h);
    f[0] = v.x; f[1] = v.y;
  }
  __device__ static void unpack(const uint4& u, float* f) {
    up(u.x, f); up(u.y, f + 2); up(u.z, f + 4); up(u.w, f + 6);
  }
  __device__ static uint32_t pk(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ static uint4 pack(const float* f) {
    return make_uint4(pk(f[0], f[1]), pk(f[2], f[3]), pk(f[4], f[5]), pk(f[6], f[7]));
  }
  __device__ static float round_trip(float x) { return __half2float(__float2half_rn(x)); }
};

constexpr int kKeyChunk = 4;

template <typename T, int HD>
__device__ __forceinline__ float dot_row(const float (&q)[HD], const unsigned char* krow) {
  constexpr int V = Elt<T>::kVec;
  float s = 0.f;
#pragma unroll
  for (int d = 0; d < HD; d += V) {
    uint4 u = *reinterpret_cast<const uint4*>(krow + d * sizeof(T));
    float f[V];
    Elt<T>::unpack(u, f);
#pragma unroll
    for (int e = 0; e < V; ++e) s = fmaf(q[d + e], f[e], s);
  }
  return s;
}

template <typename T, int HD, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) k_attn_fused(AttnParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int item = blockIdx.x;
  if (item >= p.header[SSW_H_PACKS]) return;
  const int tile = p.tile;
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem);
  int32_t* kmeta = reinterpret_cast<int32_t*>(smem + 16);
  unsigned char* rows = smem + 16 + ((tile * 4 + 15) & ~15);

  const int4 d = p.pack_desc[item];
  const int c = d.y;
  const bool big = d.z < 0;
  const int h = threadIdx.x / tile;
  const int r = threadIdx.x - h * tile;
  const int q_first = big ? (-d.z - 1) * tile : 0;
  const int q_rows = big ? min(tile, c - q_first) : d.z * c;
  const int keys_total = big ? c : q_rows;
  const bool active = r < q_rows;
  const int wl = big ? 0 : r / c;                  // window inside the pack
  const int kbeg = big ? 0 : wl * c;               // my window's keys, relative to row d.x
  const int kend = kbeg + c;
  const int C = p.C, H = p.H;
  const uint32_t row_bytes = 2u * C * sizeof(T);

  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }

  float q[HD];
  float acc[HD];
  int my_vox = 0, my_rel = 0, my_region = 0;
  if (active) {
    const int row = d.x + q_first + r;
    my_vox = __ldg(p.pack_perm + row);
    const int m = __ldg(p.pack_meta + row);
    my_rel = meta_rel(m) + p.rel_off;
    my_region = meta_region(m);
    const unsigned char* src =
        reinterpret_cast<const unsigned char*>(p.qkv) + ((int64_t)my_vox * 3 * C + h * HD) * sizeof(T);
    constexpr int V = Elt<T>::kVec;
#pragma unroll
    for (int e = 0; e < HD; e += V) {
      uint4 u = __ldg(reinterpret_cast<const uint4*>(src + e * sizeof(T)));
      float f[V];
      Elt<T>::unpack(u, f);
#pragma unroll
      for (int x = 0; x < V; ++x) q[e + x] = f[x] * p.scale;
    }
  }
  const float* table_h = p.table + h;
  __syncthreads();  // barrier initialised

  const int n_tiles = (keys_total + tile - 1) / tile;
  const int n_pass = p.attn_vals ? 2 : 1;
  float m_run = 0.f, l_run = 0.f;  // upstream's row maximum starts from 0 (ops.cu:137)
  float inv_l = 0.f;
  uint32_t phase = 0;
  int64_t coo_base = 0;
  if (n_pass == 2 && active) {
    const int kwin = __ldg(p.pack_win + d.w + wl);
    coo_base = ((int64_t)__ldg(p.coo_start + kwin) * H + (int64_t)h * c * c) +
               (int64_t)(big ? q_first + r : r - wl * c) * c;
  }
#pragma unroll
  for (int e = 0; e < HD; ++e) acc[e] = 0.f;

  for (int pass = 0; pass < n_pass; ++pass) {
    for (int t = 0; t < n_tiles; ++t) {
      const int k0 = t * tile;
      const int rows_t = min(tile, keys_total - k0);
      if (pass == 0 || n_tiles > 1) {
        if (threadIdx.x == 0) mbar_expect_tx(bar, rows_t * row_bytes);
        if ((int)threadIdx.x < rows_t) {
          const int row = d.x + k0 + threadIdx.x;
          const int vj = __ldg(p.pack_perm + row);
          kmeta[threadIdx.x] = __ldg(p.pack_meta + row);
          bulk_g2s(rows + (size_t)threadIdx.x * p.row_stride,
                   reinterpret_cast<const unsigned char*>(p.qkv) + ((int64_t)vj * 3 * C + C) * sizeof(T), row_bytes,
                   bar);
        }
        __syncthreads();  // kmeta visible
        if (!mbar_wait_bounded(bar, phase)) {
          atomicOr(reinterpret_cast<unsigned*>(p.header + SSW_H_ERROR), SSW_DEV_TIMEOUT);
          return;
        }
        phase ^= 1;
      }
      if (active) {
        const int jb = max(kbeg, k0), je = min(kend, k0 + rows_t);
        for (int j = jb; j < je; j += kKeyChunk) {
          float s[kKeyChunk];
#pragma unroll
          for (int u = 0; u < kKeyChunk; ++u) {
            const int jj = min(j + u, je - 1) - k0;
            const unsigned char* krow = rows + (size_t)jj * p.row_stride + h * HD * sizeof(T);
            float sc = dot_row<T, HD>(q, krow);
            const int km = kmeta[jj];
            sc += __ldg(table_h + (my_rel - meta_rel(km)) * H);
            if (p.use_mask && my_region != meta_region(km)) sc += -100.0f;
            s[u] = (j + u < je) ? sc : -INFINITY;
          }
          if (pass == 0) {
            float mc = s[0];
#pragma unroll
            for (int u = 1; u < kKeyChunk; ++u) mc = fmaxf(mc, s[u]);
            if (mc > m_run) {
              const float corr = expf(m_run - mc);
              l_run *= corr;
#pragma unroll
              for (int e = 0; e < HD; ++e) acc[e] *= corr;
              m_run = mc;
            }
#pragma unroll
            for (int u = 0; u < kKeyChunk; ++u) {
              const float pu = expf(s[u] - m_run);
              l_run += pu;
              const int jj = min(j + u, je - 1) - k0;
              const unsigned char* vrow = rows + (size_t)jj * p.row_stride + (C + h * HD) * sizeof(T);
              constexpr int V = Elt<T>::kVec;
#pragma unroll
              for (int e = 0; e < HD; e += V) {
                uint4 uv = *reinterpret_cast<const uint4*>(vrow + e * sizeof(T));
                float f[V];
                Elt<T>::unpack(uv, f);
#pragma unroll
                for (int x = 0; x < V; ++x) acc[e + x] = fmaf(pu, f[x], acc[e + x]);
              }
            }
          } else {
            T* dst = reinterpret_cast<T*>(p.attn_vals) + coo_base + (j - kbeg);
#pragma unroll
            for (int u = 0; u < kKeyChunk; ++u) {
              if (j + u < je) {
                float f = expf(s[u] - m_run) * inv_l;
                if constexpr (sizeof(T) == 4) {
                  reinterpret_cast<float*>(dst)[u] = f;
                } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
                  dst[u] = __float2bfloat16_rn(f);
                } else {
                  dst[u] = __float2half_rn(f);
                }
              }
            }
          }
        }
      }
      if (n_tiles > 1) __syncthreads();  // everyone done with this tile before it is overwritten
    }
    if (pass == 0) inv_l = 1.0f / (l_run + 1e-8f);
  }

  if (active) {
    const float denom = l_run + 1e-8f;  // ops.cu:164
    unsigned char* dst = reinterpret_cast<unsigned char*>(p.out) + ((int64_t)my_vox * C + h * HD) * sizeof(T);
    constexpr int V = Elt<T>::kVec;
#pragma unroll
    for (int e = 0; e < HD; e += V) {
      float f[V];
#pragma unroll
      for (int x = 0; x < V; ++x) f[x] = acc[e + x] / denom;
      *reinterpret_cast<uint4*>(dst + e * sizeof(T)) = Elt<T>::pack(f);
    }
  }
}

template <typename T, int HD>
static int launch_attn(const AttnParams& p, int grid, int threads, size_t smem, cudaStream_t stream) {
  // Two register budgets: up to 256 threads per item (>=3 items per SM) or up to 1024.
  if (threads <= 256) {
    auto kern = k_attn_fused<T, HD, 256, 2>;
    SSW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, threads, smem, stream>>>(p);
  } else {
    auto kern = k_attn_fused<T, HD, 1024, 1>;
    SSW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, threads, smem, stream>>>(p);
  }
  SSW_LAUNCH_CHECK("k_attn_fused");
  return SSW_OK;
}

template <typename T>
static int dispatch_hd(const AttnParams& p, int hd, int grid, int threads, size_t smem, cudaStream_t stream) {
  switch (hd) {
    case 16: return launch_attn<T, 16>(p, grid, threads, smem, stream);
    case 32: return launch_attn<T, 32>(p, grid, threads, smem, stream);
    default: return SSW_E_UNSUPPORTED;
  }
}

}  // namespace ssw

using namespace ssw;

extern "C" int ssw_attn_fused(const void* qkv, int dtype, int32_t heads, int32_t head_dim, const ssw_plan_layout* L,
                              const int32_t* plan, const float* table, const int32_t rpb_window[3], float scale,
                              int use_mask, void* out, void* attn_vals, void* stream_) {
  if (!L || !plan || !table || !rpb_window || heads <= 0 || head_dim <= 0) return SSW_E_INVALID;
  if (L->n_vox == 0) return SSW_OK;
  if (!qkv || !out) return SSW_E_INVALID;
  const int elt = dtype == SSW_F32 ? 4 : (dtype == SSW_BF16 || dtype == SSW_F16) ? 2 : 0;
  if (!elt) return SSW_E_INVALID;
  const int C = heads * head_dim;
  if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return SSW_E_INVALID;
  if ((head_dim * elt) % 16) return SSW_E_UNSUPPORTED;
  const int tile = L->tile_rows;
  const int threads = tile * heads;
  if (threads > 1024) return SSW_E_INVALID;
  AttnParams p;
  p.qkv = qkv;
  p.out = out;
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
  p.row_stride = 2 * C * elt + 16;  // +16 B skews rows across shared-memory banks
  const size_t smem = 16 + ((tile * 4 + 15) & ~15) + (size_t)tile * p.row_stride;
  if (smem > 227 * 1024) return SSW_E_UNSUPPORTED;
  cudaStream_t stream = (cudaStream_t)stream_;
  switch (dtype) {
    case SSW_F32: return dispatch_hd<float>(p, head_dim, L->pack_cap, threads, smem, stream);
    case SSW_BF16: return dispatch_hd<__nv_bfloat16>(p, head_dim, L->pack_cap, threads, smem, stream);
    case SSW_F16: return dispatch_hd<__half>(p, head_dim, L->pack_cap, threads, smem, stream);
  }
  return SSW_E_INVALID;
}
