// Sparse 3-D convolutions over voxel sets, as the layers around the attention stages use them
// (sparse_swin/swin3d_base.py:915-935 patch embedding, :965-970 patch merging, :989-994 patch
// expansion, :1039-1059 residual blocks): submanifold convolution (output sites = input sites),
// strided convolution with kernel = stride (each output cell gathers its 2^3 children) and its
// inverse.  Upstream takes these from the spconv library; here a convolution is
//     rulebook (which input row feeds which output row through which kernel tap)  - integer kernels below
//  -> gathered operand  cols[m, tap * Cin + c] = x[nbr[m, tap], c]  (zero where there is no neighbour)
//  -> one dense GEMM    out = cols @ W.reshape(taps * Cin, Cout)    (a library GEMM, issued by the host side)
// so the arithmetic is a plain contraction and the irregular part is pure data movement: HBM bound,
// 16-byte chunks, one chunk per thread, neighbour ids re-read through L1.
//
// The rulebook of a submanifold convolution comes from a dense cell -> voxel-id table of the scene
// (4 bytes per cell of the grid: 96 MB for 400 x 400 x 150, independent of the channel count and
// shared by every layer over the same coordinates).
#include <type_traits>

#include "ssw_common.cuh"

namespace ssw {

__global__ void k_grid_scatter(const int32_t* __restrict__ coords, int64_t n, int batch, int D, int H, int W,
                               int32_t* __restrict__ grid, int32_t* __restrict__ err) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int4 c = __ldg(reinterpret_cast<const int4*>(coords) + i);  // b, z, y, x
  if ((unsigned)c.x >= (unsigned)batch || (unsigned)c.y >= (unsigned)D || (unsigned)c.z >= (unsigned)H ||
      (unsigned)c.w >= (unsigned)W) {
    if (err) atomicOr(reinterpret_cast<unsigned*>(err), SSW_DEV_BAD_COORD);
    return;
  }
  const int64_t cell = (((int64_t)c.x * D + c.y) * H + c.z) * W + c.w;
  // two voxels in one cell: the larger id stays (deterministic), and the caller is told
  const int prev = atomicMax(grid + cell, (int)i);
  if (prev >= 0 && err) atomicOr(reinterpret_cast<unsigned*>(err), SSW_DEV_DUPLICATE);
}

// nbr[i, t] = id of the voxel at coords[i] + offset(t), t = (dz * K + dy) * K + dx with offsets
// -K/2 .. K/2 (the cross-correlation convention of a dense convolution with padding K/2), or -1
__global__ void k_subm_neighbors(const int32_t* __restrict__ coords, int64_t n, int batch, int D, int H, int W,
                                 const int32_t* __restrict__ grid, int K, int32_t* __restrict__ nbr) {
  const int taps = K * K * K;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n * taps) return;
  const int64_t i = idx / taps;
  const int t = (int)(idx - i * taps);
  const int4 c = __ldg(reinterpret_cast<const int4*>(coords) + i);
  const int r = K / 2;
  const int dz = t / (K * K) - r, dy = (t / K) % K - r, dx = t % K - r;
  const int z = c.y + dz, y = c.z + dy, x = c.w + dx;
  int v = -1;
  if ((unsigned)c.x < (unsigned)batch && (unsigned)z < (unsigned)D && (unsigned)y < (unsigned)H && (unsigned)x < (unsigned)W)
    v = __ldg(grid + ((((int64_t)c.x * D + z) * H + y) * W + x));
  nbr[idx] = v;
}

// cols[m, t * cin + c] = x[nbr[m, t], c] or 0; VEC bytes per thread (16 when the rows allow it)
template <int VEC>
__global__ void k_gather_cols(const unsigned char* __restrict__ x, int64_t m_rows, int taps, int row_bytes,
                              const int32_t* __restrict__ nbr, int64_t n_src, unsigned char* __restrict__ cols) {
  const int chunks = row_bytes / VEC;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= m_rows * taps * chunks) return;
  const int64_t mt = idx / chunks;
  const int ch = (int)(idx - mt * chunks);
  const int j = __ldg(nbr + mt);
  const bool ok = (unsigned)j < (unsigned)n_src;  // a rulebook entry outside the source reads as "no neighbour"
  if constexpr (VEC == 16) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (ok) v = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)j * row_bytes) + ch);
    reinterpret_cast<uint4*>(cols + mt * row_bytes)[ch] = v;
  } else if constexpr (VEC == 4) {
    uint32_t v = 0;
    if (ok) v = __ldg(reinterpret_cast<const uint32_t*>(x + (int64_t)j * row_bytes) + ch);
    reinterpret_cast<uint32_t*>(cols + mt * row_bytes)[ch] = v;
  } else {
    uint16_t v = 0;
    if (ok) v = __ldg(reinterpret_cast<const uint16_t*>(x + (int64_t)j * row_bytes) + ch);
    reinterpret_cast<uint16_t*>(cols + mt * row_bytes)[ch] = v;
  }
}

// out[i, :] = z[parent[i], tap[i] * cout : (tap[i] + 1) * cout], zero where parent[i] < 0
template <int VEC>
__global__ void k_gather_slices(const unsigned char* __restrict__ z, int64_t n, int out_bytes, int z_row_bytes,
                                const int32_t* __restrict__ parent, const int32_t* __restrict__ tap, int64_t n_src,
                                int taps, unsigned char* __restrict__ out) {
  const int chunks = out_bytes / VEC;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n * chunks) return;
  const int64_t i = idx / chunks;
  const int ch = (int)(idx - i * chunks);
  const int pj = __ldg(parent + i), t = __ldg(tap + i);
  const bool ok = (unsigned)pj < (unsigned)n_src && (unsigned)t < (unsigned)taps;
  const unsigned char* src = z + (int64_t)pj * z_row_bytes + (int64_t)t * out_bytes;
  if constexpr (VEC == 16) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (ok) v = __ldg(reinterpret_cast<const uint4*>(src) + ch);
    reinterpret_cast<uint4*>(out + i * out_bytes)[ch] = v;
  } else if constexpr (VEC == 4) {
    uint32_t v = 0;
    if (ok) v = __ldg(reinterpret_cast<const uint32_t*>(src) + ch);
    reinterpret_cast<uint32_t*>(out + i * out_bytes)[ch] = v;
  } else {
    uint16_t v = 0;
    if (ok) v = __ldg(reinterpret_cast<const uint16_t*>(src) + ch);
    reinterpret_cast<uint16_t*>(out + i * out_bytes)[ch] = v;
  }
}

// out[i, :] = base[i, :] + sum of y[slots[p], :] over p in [row_start[i], row_start[i + 1]), summed in
// fp32 in list order (deterministic).  One thread per (row, 16-byte chunk).
template <typename T>
__global__ void k_gather_reduce(const T* __restrict__ base, const T* __restrict__ y, int64_t n_y,
                                const int32_t* __restrict__ row_start, const int32_t* __restrict__ slots, int64_t n_slots,
                                int64_t n, int c, T* __restrict__ out) {
  constexpr int V = 16 / (int)sizeof(T);
  const int chunks = c / V;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n * chunks) return;
  const int64_t i = idx / chunks;
  const int ch = (int)(idx - i * chunks);
  float acc[V];
  auto add = [&](const T* row) {
    if constexpr (sizeof(T) == 4) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(row) + ch);
      acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
    } else {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(row) + ch);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if constexpr (std::is_same<T, __nv_bfloat16>::value) {
          acc[2 * k] += __uint_as_float(w[k] << 16);
          acc[2 * k + 1] += __uint_as_float(w[k] & 0xffff0000u);
        } else {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
          acc[2 * k] += f.x;
          acc[2 * k + 1] += f.y;
        }
      }
    }
  };
#pragma unroll
  for (int k = 0; k < V; ++k) acc[k] = 0.f;
  if (base) add(base + i * c);
  // a list that does not fit its own table (a stale or foreign rulebook) is cut to the table
  const int64_t p0 = max(0, __ldg(row_start + i)), p1 = min((int64_t)__ldg(row_start + i + 1), n_slots);
  for (int64_t q = p0; q < p1; ++q) {
    const int pj = __ldg(slots + q);
    if ((unsigned)pj < (unsigned)n_y) add(y + (int64_t)pj * c);
  }
  if constexpr (sizeof(T) == 4) {
    reinterpret_cast<float4*>(out + i * c)[ch] = make_float4(acc[0], acc[1], acc[2], acc[3]);
  } else {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
        w[k] = *reinterpret_cast<const uint32_t*>(&h);
      } else {
        const __half2 h = __floats2half2_rn(acc[2 * k], acc[2 * k + 1]);
        w[k] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
    reinterpret_cast<uint4*>(out + i * c)[ch] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

static int vec_of(int row_bytes, const void* a, const void* b) {
  const uintptr_t al = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b);
  if (row_bytes % 16 == 0 && (al & 15) == 0) return 16;
  if (row_bytes % 4 == 0 && (al & 3) == 0) return 4;
  return 2;
}

}  // namespace ssw

using namespace ssw;

static int elt_of(int dtype) { return dtype == SSW_F32 ? 4 : (dtype == SSW_BF16 || dtype == SSW_F16) ? 2 : 0; }

extern "C" int ssw_voxel_grid_build(const int32_t* coords, int64_t n, int32_t batch, const int32_t dims[3], int32_t* grid,
                                    int32_t* err, void* stream_) {
  if (n < 0 || batch <= 0 || !dims || !grid || dims[0] <= 0 || dims[1] <= 0 || dims[2] <= 0) return SSW_E_INVALID;
  const int64_t cells = (int64_t)batch * dims[0] * dims[1] * dims[2];
  if (cells >= ((int64_t)1 << 31) || n >= ((int64_t)1 << 31)) return SSW_E_RANGE;
  cudaStream_t stream = (cudaStream_t)stream_;
  SSW_CUDA_TRY(cudaMemsetAsync(grid, 0xff, (size_t)cells * 4, stream));  // every cell -1
  if (n == 0) return SSW_OK;
  if (!coords || (reinterpret_cast<uintptr_t>(coords) & 15)) return SSW_E_INVALID;
  k_grid_scatter<<<(unsigned)ceil_div64(n, 256), 256, 0, stream>>>(coords, n, batch, dims[0], dims[1], dims[2], grid, err);
  SSW_LAUNCH_CHECK("k_grid_scatter");
  return SSW_OK;
}

extern "C" int ssw_subm_neighbors(const int32_t* coords, int64_t n, int32_t batch, const int32_t dims[3],
                                  const int32_t* grid, int32_t ksize, int32_t* nbr, void* stream_) {
  if (n < 0 || batch <= 0 || !dims || !grid || ksize < 1 || ksize > 7 || !(ksize & 1)) return SSW_E_INVALID;
  if (n == 0) return SSW_OK;
  if (!coords || !nbr || (reinterpret_cast<uintptr_t>(coords) & 15)) return SSW_E_INVALID;
  const int64_t total = n * ksize * ksize * ksize;
  if (total >= ((int64_t)1 << 40)) return SSW_E_RANGE;
  k_subm_neighbors<<<(unsigned)ceil_div64(total, 256), 256, 0, (cudaStream_t)stream_>>>(coords, n, batch, dims[0], dims[1],
                                                                                      dims[2], grid, ksize, nbr);
  SSW_LAUNCH_CHECK("k_subm_neighbors");
  return SSW_OK;
}

extern "C" int ssw_gather_cols(const void* x, int dtype, int64_t n_src, int64_t m_rows, int32_t taps, int32_t cin,
                               const int32_t* nbr, void* cols, void* stream_) {
  const int elt = elt_of(dtype);
  if (!elt || m_rows < 0 || n_src < 0 || taps <= 0 || cin <= 0) return SSW_E_INVALID;
  if (m_rows == 0) return SSW_OK;
  if (!nbr || !cols || (n_src > 0 && !x)) return SSW_E_INVALID;
  const int row_bytes = cin * elt;
  const int vec = vec_of(row_bytes, x, cols);
  const int64_t total = m_rows * taps * (row_bytes / vec);
  if (total >= ((int64_t)1 << 40)) return SSW_E_RANGE;
  const unsigned blocks = (unsigned)ceil_div64(total, 256);
  cudaStream_t stream = (cudaStream_t)stream_;
  const unsigned char* xs = reinterpret_cast<const unsigned char*>(x);
  unsigned char* cs = reinterpret_cast<unsigned char*>(cols);
  if (vec == 16) k_gather_cols<16><<<blocks, 256, 0, stream>>>(xs, m_rows, taps, row_bytes, nbr, n_src, cs);
  else if (vec == 4) k_gather_cols<4><<<blocks, 256, 0, stream>>>(xs, m_rows, taps, row_bytes, nbr, n_src, cs);
  else k_gather_cols<2><<<blocks, 256, 0, stream>>>(xs, m_rows, taps, row_bytes, nbr, n_src, cs);
  SSW_LAUNCH_CHECK("k_gather_cols");
  return SSW_OK;
}

extern "C" int ssw_gather_slices(const void* z, int dtype, int64_t n_src, int32_t taps, int32_t cout, int64_t n,
                                 const int32_t* parent, const int32_t* tap, void* out, void* stream_) {
  const int elt = elt_of(dtype);
  if (!elt || n < 0 || n_src < 0 || taps <= 0 || cout <= 0) return SSW_E_INVALID;
  if (n == 0) return SSW_OK;
  if (!parent || !tap || !out || (n_src > 0 && !z)) return SSW_E_INVALID;
  const int out_bytes = cout * elt;
  const int vec = vec_of(out_bytes, z, out);
  const int64_t total = n * (out_bytes / vec);
  const unsigned blocks = (unsigned)ceil_div64(total, 256);
  cudaStream_t stream = (cudaStream_t)stream_;
  const unsigned char* zs = reinterpret_cast<const unsigned char*>(z);
  unsigned char* os = reinterpret_cast<unsigned char*>(out);
  const int zrb = out_bytes * taps;
  if (vec == 16) k_gather_slices<16><<<blocks, 256, 0, stream>>>(zs, n, out_bytes, zrb, parent, tap, n_src, taps, os);
  else if (vec == 4) k_gather_slices<4><<<blocks, 256, 0, stream>>>(zs, n, out_bytes, zrb, parent, tap, n_src, taps, os);
  else k_gather_slices<2><<<blocks, 256, 0, stream>>>(zs, n, out_bytes, zrb, parent, tap, n_src, taps, os);
  SSW_LAUNCH_CHECK("k_gather_slices");
  return SSW_OK;
}

extern "C" int ssw_gather_reduce(const void* base, const void* y, int dtype, int64_t n_y, const int32_t* row_start,
                                 const int32_t* slots, int64_t n_slots, int64_t n, int32_t c, void* out, void* stream_) {
  const int elt = elt_of(dtype);
  if (!elt || n < 0 || n_y < 0 || n_slots < 0 || c <= 0) return SSW_E_INVALID;
  if (n == 0) return SSW_OK;
  if (!out || !row_start || (n_slots > 0 && (!slots || !y))) return SSW_E_INVALID;
  if ((c * elt) % 16) return SSW_E_UNSUPPORTED;
  const void* ptrs[3] = {base, y, out};
  for (const void* q : ptrs)
    if (q && (reinterpret_cast<uintptr_t>(q) & 15)) return SSW_E_INVALID;
  const int64_t total = n * (c * elt / 16);
  const unsigned blocks = (unsigned)ceil_div64(total, 256);
  cudaStream_t stream = (cudaStream_t)stream_;
  switch (dtype) {
    case SSW_F32:
      k_gather_reduce<float><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(base), reinterpret_cast<const float*>(y),
                                                         n_y, row_start, slots, n_slots, n, c, reinterpret_cast<float*>(out));
      break;
    case SSW_BF16:
      k_gather_reduce<__nv_bfloat16><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(base),
                                                                 reinterpret_cast<const __nv_bfloat16*>(y), n_y, row_start, slots,
                                                                 n_slots, n, c, reinterpret_cast<__nv_bfloat16*>(out));
      break;
    default:
      k_gather_reduce<__half><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __half*>(base), reinterpret_cast<const __half*>(y),
                                                          n_y, row_start, slots, n_slots, n, c, reinterpret_cast<__half*>(out));
  }
  SSW_LAUNCH_CHECK("k_gather_reduce");
  return SSW_OK;
}
