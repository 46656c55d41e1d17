// Backward of the fused window attention: gradients of qkv and of the relative-position bias
// table from the gradient of the output, without materialising the attention matrix.
//
// Upstream differentiates the unfused chain (swin3d_base.py:106-138, 177-188; ops.cu:169-194,
// 422-557): d(softmax) = out * (g - sum_row(out * g)) on the stored COO values, then the blocked
// products rc_cr / rr_rc / cr_rr.  Here the probabilities are recomputed from q and k instead of
// stored (the forward keeps nothing but its output), with the forward's exact definition:
//   s_ij = scale * q_i.k_j + bias[rel_i - rel_j] (- 100 if the regions differ)
//   m_i = max(0, max_j s_ij),  p_ij = exp(s_ij - m_i) / (sum_j exp(s_ij - m_i) + 1e-8)
//   dP_ij = dO_i.v_j,  D_i = sum_j p_ij dP_ij,  dS_ij = p_ij (dP_ij - D_i)
//   dq_i = scale * sum_j dS_ij k_j,  dk_j = scale * sum_i dS_ij q_i,  dv_j = sum_i p_ij dO_i,
//   dbias[rel_i - rel_j, h] += dS_ij
//
// Two kernels over the plan's work items, one thread per (row, head), rows read straight from
// global memory (the rows of a window are re-read by its own threads only, so they stay in L1/L2):
//   k_attn_bwd_q : per query row one sweep over the window's keys with an online maximum: the row
//                  statistics and dq (as (A - D B)/(l+1e-8) with A = sum e dP k, B = sum e k);
//                  leaves (m_i, 1/(l_i+1e-8), D_i) per (row, head) for
//   k_attn_bwd_kv: per key row one sweep over the window's queries -> dk, dv and the bias gradient.
// No atomics on the row gradients; the bias gradient is accumulated in a shared-memory copy of the
// table per CTA (when it fits) and flushed with global atomics.
//
// The plan may be stale (the backward runs long after the forward that built it, possibly after
// the caller rebuilt another plan in the same buffer): item counts, descriptors, voxel ids and
// relative-position codes are held to their bounds exactly as in the forward kernels; a violation
// sets SSW_DEV_BAD_PLAN and is replaced by a harmless value.
#include <math.h>

#include "attn_common.cuh"

namespace ssw {

struct BwdParams {
  const void* qkv;
  const void* grad_out;
  void* dqkv;
  float* dtable;
  float* stats;  // [N * H * 4]: m (log2 domain), 1/(l + 1e-8), D, unused
  int32_t* header;
  const int4* pack_desc;
  const int32_t* pack_perm;
  const int32_t* pack_meta;
  const float* table;
  int rel_off, H, C, tile;
  int n_vox, pack_cap;  // bounds the kernels hold the plan's voxel ids and item counts to
  float scale;
  int use_mask;
  int table_floats;  // > 0: the bias gradient is accumulated in shared memory first
};

template <typename T, int HD>
__device__ __forceinline__ void load_row(const T* src, float (&x)[HD]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int e = 0; e < HD / 4; ++e) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(src) + e);
      x[4 * e] = v.x; x[4 * e + 1] = v.y; x[4 * e + 2] = v.z; x[4 * e + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int e = 0; e < HD / 8; ++e) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(src) + e);
      float4 a, b;
      widen8<T>(u, a, b);
      x[8 * e] = a.x; x[8 * e + 1] = a.y; x[8 * e + 2] = a.z; x[8 * e + 3] = a.w;
      x[8 * e + 4] = b.x; x[8 * e + 5] = b.y; x[8 * e + 6] = b.z; x[8 * e + 7] = b.w;
    }
  }
}

template <typename T, int HD>
__device__ __forceinline__ void store_row(T* dst, const float (&x)[HD], float f) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int e = 0; e < HD / 4; ++e)
      reinterpret_cast<float4*>(dst)[e] = make_float4(x[4 * e] * f, x[4 * e + 1] * f, x[4 * e + 2] * f, x[4 * e + 3] * f);
  } else {
#pragma unroll
    for (int e = 0; e < HD / 8; ++e) {
      uint4 u;
      u.x = pack2<T>(x[8 * e] * f, x[8 * e + 1] * f);
      u.y = pack2<T>(x[8 * e + 2] * f, x[8 * e + 3] * f);
      u.z = pack2<T>(x[8 * e + 4] * f, x[8 * e + 5] * f);
      u.w = pack2<T>(x[8 * e + 6] * f, x[8 * e + 7] * f);
      reinterpret_cast<uint4*>(dst)[e] = u;
    }
  }
}

template <int HD>
__device__ __forceinline__ float dot(const float (&a)[HD], const float (&b)[HD]) {
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int e = 0; e < HD; e += 2) {
    s0 = fmaf(a[e], b[e], s0);
    s1 = fmaf(a[e + 1], b[e + 1], s1);
  }
  return s0 + s1;
}

// The rows of work item d this thread's local row t belongs with: its own pack row and the first
// row and length of its window's run.  False when t is beyond the item.
__device__ __forceinline__ bool item_row(const int4& d, int tile, int t, int& row, int& first, int& count) {
  const int c = d.y;
  if (d.z >= 0) {  // pack of d.z windows with c voxels each
    if (t >= d.z * c) return false;
    const int wl = t / c;
    row = d.x + t;
    first = d.x + wl * c;
  } else {  // one tile of rows of a large window
    const int r0 = (-d.z - 1) * tile;
    if (r0 + t >= c || t >= tile) return false;
    row = d.x + r0 + t;
    first = d.x;
  }
  count = c;
  return true;
}
__device__ __forceinline__ int item_rows(const int4& d, int tile) {
  if (d.z >= 0) return d.z * d.y;
  return min(tile, d.y - (-d.z - 1) * tile);
}

// log2-domain score of (query i, key j) from the raw dot product
__device__ __forceinline__ float score2(float qk, float qs, const float* table, int rel_i_off, int meta_i, int meta_j,
                                        int H, int h, bool use_mask) {
  const float b = __ldg(table + (rel_i_off - meta_rel(meta_j)) * H + h);
  const float madd = (use_mask && meta_region(meta_i) != meta_region(meta_j)) ? -100.0f : 0.f;
  return fmaf(qk, qs, (b + madd) * kLog2e);
}

template <typename T, int HD>
__global__ void __launch_bounds__(128) k_attn_bwd_q(BwdParams p) {
  const int H = p.H, C = p.C;
  const int n_items = checked_count(p.header[SSW_H_PACKS], p);
  const int n_small = min(checked_count(p.header[SSW_H_PACKS_SMALL], p), n_items);
  const float qs = p.scale * kLog2e;
  const T* qkv = reinterpret_cast<const T*>(p.qkv);
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int4 d = checked_desc(__ldg(p.pack_desc + item), p, item < n_small);
    const int nrows = item_rows(d, p.tile);
    for (int idx = threadIdx.x; idx < nrows * H; idx += blockDim.x) {
      const int h = idx / nrows, t = idx - h * nrows;
      int row, first, c;
      if (!item_row(d, p.tile, t, row, first, c)) continue;
      const int vi = checked_voxel(__ldg(p.pack_perm + row), p), mi = checked_meta(__ldg(p.pack_meta + row), p);
      const int rel_i_off = meta_rel(mi) + p.rel_off;
      float q[HD], go[HD];
      load_row<T, HD>(qkv + (int64_t)vi * 3 * C + h * HD, q);
      load_row<T, HD>(reinterpret_cast<const T*>(p.grad_out) + (int64_t)vi * C + h * HD, go);
      // One sweep over the window's keys with the running maximum (from 0): denominator l,
      // dn = sum_j e_ij dP_ij, A = sum_j e_ij dP_ij k_j and B = sum_j e_ij k_j, from which
      // D = dn / (l + 1e-8) and dq = (A - D B) / (l + 1e-8).
      float m = 0.f, l = 0.f, dn = 0.f;
      float dq[HD], kb[HD];
#pragma unroll
      for (int e = 0; e < HD; ++e) dq[e] = kb[e] = 0.f;
      for (int j = 0; j < c; ++j) {
        const int vj = checked_voxel(__ldg(p.pack_perm + first + j), p);
        const int mj = checked_meta(__ldg(p.pack_meta + first + j), p);
        float k[HD], v[HD];
        load_row<T, HD>(qkv + (int64_t)vj * 3 * C + C + h * HD, k);
        load_row<T, HD>(qkv + (int64_t)vj * 3 * C + 2 * C + h * HD, v);
        const float s2 = score2(dot<HD>(q, k), qs, p.table, rel_i_off, mi, mj, H, h, p.use_mask != 0);
        const float dp = dot<HD>(go, v);
        if (s2 > m) {
          const float corr = fast_exp2(m - s2);
          l *= corr;
          dn *= corr;
#pragma unroll
          for (int e = 0; e < HD; ++e) { dq[e] *= corr; kb[e] *= corr; }
          m = s2;
        }
        const float ex = fast_exp2(s2 - m);
        const float edp = ex * dp;
        l += ex;
        dn += edp;
#pragma unroll
        for (int e = 0; e < HD; ++e) {
          dq[e] = fmaf(edp, k[e], dq[e]);
          kb[e] = fmaf(ex, k[e], kb[e]);
        }
      }
      const float inv = 1.0f / (l + 1e-8f);
      const float D = dn * inv;
      reinterpret_cast<float4*>(p.stats)[(int64_t)row * H + h] = make_float4(m, inv, D, 0.f);
#pragma unroll
      for (int e = 0; e < HD; ++e) dq[e] = (dq[e] - D * kb[e]) * inv;
      store_row<T, HD>(reinterpret_cast<T*>(p.dqkv) + (int64_t)vi * 3 * C + h * HD, dq, p.scale);
    }
  }
}

template <typename T, int HD>
__global__ void __launch_bounds__(128) k_attn_bwd_kv(BwdParams p) {
  extern __shared__ float dtab_s[];
  const int H = p.H, C = p.C;
  for (int i = threadIdx.x; i < p.table_floats; i += blockDim.x) dtab_s[i] = 0.f;
  __syncthreads();
  grid_dependency_wait();  // the row statistics come from the kernel this one is chained behind
  const int n_items = checked_count(p.header[SSW_H_PACKS], p);
  const int n_small = min(checked_count(p.header[SSW_H_PACKS_SMALL], p), n_items);
  const float qs = p.scale * kLog2e;
  const T* qkv = reinterpret_cast<const T*>(p.qkv);
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int4 d = checked_desc(__ldg(p.pack_desc + item), p, item < n_small);
    const int nrows = item_rows(d, p.tile);
    for (int idx = threadIdx.x; idx < nrows * H; idx += blockDim.x) {
      const int h = idx / nrows, t = idx - h * nrows;
      int row, first, c;
      if (!item_row(d, p.tile, t, row, first, c)) continue;
      const int vj = checked_voxel(__ldg(p.pack_perm + row), p), mj = checked_meta(__ldg(p.pack_meta + row), p);
      float k[HD], v[HD], dk[HD], dv[HD];
      load_row<T, HD>(qkv + (int64_t)vj * 3 * C + C + h * HD, k);
      load_row<T, HD>(qkv + (int64_t)vj * 3 * C + 2 * C + h * HD, v);
#pragma unroll
      for (int e = 0; e < HD; ++e) dk[e] = dv[e] = 0.f;
      for (int i = 0; i < c; ++i) {
        const int vi = checked_voxel(__ldg(p.pack_perm + first + i), p);
        const int mi = checked_meta(__ldg(p.pack_meta + first + i), p);
        float q[HD], go[HD];
        load_row<T, HD>(qkv + (int64_t)vi * 3 * C + h * HD, q);
        load_row<T, HD>(reinterpret_cast<const T*>(p.grad_out) + (int64_t)vi * C + h * HD, go);
        const float4 st = reinterpret_cast<const float4*>(p.stats)[(int64_t)(first + i) * H + h];
        const float s2 = score2(dot<HD>(q, k), qs, p.table, meta_rel(mi) + p.rel_off, mi, mj, H, h, p.use_mask != 0);
        const float pij = fast_exp2(s2 - st.x) * st.y;
        const float ds = pij * (dot<HD>(go, v) - st.z);
#pragma unroll
        for (int e = 0; e < HD; ++e) {
          dk[e] = fmaf(ds, q[e], dk[e]);
          dv[e] = fmaf(pij, go[e], dv[e]);
        }
        const int ti = (meta_rel(mi) + p.rel_off - meta_rel(mj)) * H + h;
        if (p.table_floats > 0) atomicAdd(dtab_s + ti, ds);
        else atomicAdd(p.dtable + ti, ds);
      }
      T* dst = reinterpret_cast<T*>(p.dqkv) + (int64_t)vj * 3 * C + h * HD;
      store_row<T, HD>(dst + C, dk, p.scale);
      store_row<T, HD>(dst + 2 * C, dv, 1.0f);
    }
  }
  if (p.table_floats > 0) {
    __syncthreads();
    for (int i = threadIdx.x; i < p.table_floats; i += blockDim.x) {
      const float g = dtab_s[i];
      if (g != 0.f) atomicAdd(p.dtable + i, g);
    }
  }
}

template <typename T, int HD>
static int launch_bwd(const BwdParams& p, cudaStream_t stream) {
  int dev = 0, sms = 0;
  SSW_CUDA_TRY(cudaGetDevice(&dev));
  SSW_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const size_t smem = (size_t)p.table_floats * 4;
  auto kkv = k_attn_bwd_kv<T, HD>;
  if (smem > 48 * 1024) SSW_CUDA_TRY(cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  k_attn_bwd_q<T, HD><<<sms * 8, 128, 0, stream>>>(p);
  SSW_LAUNCH_CHECK("k_attn_bwd_q");
  SSW_CUDA_TRY(launch_chained(kkv, dim3(sms * 8), dim3(128), smem, stream, p));
  return SSW_OK;
}

}  // namespace ssw

using namespace ssw;

extern "C" int64_t ssw_attn_fused_bwd_workspace_floats(int64_t n_vox, int32_t heads) { return n_vox * heads * 4; }

extern "C" int ssw_attn_fused_bwd(const void* qkv, const void* grad_out, int dtype, int32_t heads, int32_t head_dim,
                                  const ssw_plan_layout* L, const int32_t* plan, const float* table,
                                  const int32_t rpb_window[3], float scale, int use_mask, void* dqkv, float* dtable,
                                  float* workspace, void* stream_) {
  if (!L || !plan || !table || !rpb_window || heads <= 0 || head_dim <= 0) return SSW_E_INVALID;
  if (L->n_vox == 0) return SSW_OK;
  if (!qkv || !grad_out || !dqkv || !dtable || !workspace) return SSW_E_INVALID;
  const int elt = dtype == SSW_F32 ? 4 : (dtype == SSW_BF16 || dtype == SSW_F16) ? 2 : 0;
  if (!elt) return SSW_E_INVALID;
  if ((head_dim * elt) % 16) return SSW_E_UNSUPPORTED;
  const uintptr_t align = reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(grad_out) |
                          reinterpret_cast<uintptr_t>(dqkv) | reinterpret_cast<uintptr_t>(workspace);
  if (align & 15) return SSW_E_INVALID;
  BwdParams p;
  p.qkv = qkv;
  p.grad_out = grad_out;
  p.dqkv = dqkv;
  p.dtable = dtable;
  p.stats = workspace;
  p.header = const_cast<int32_t*>(plan + L->off_header);
  p.n_vox = (int)L->n_vox;
  p.pack_cap = (int)L->pack_cap;
  p.pack_desc = reinterpret_cast<const int4*>(plan + L->off_pack_desc);
  p.pack_perm = plan + L->off_pack_perm;
  p.pack_meta = plan + L->off_pack_meta;
  p.table = table;
  p.rel_off = ((rpb_window[0] - 1) * (2 * rpb_window[1] - 1) + (rpb_window[1] - 1)) * (2 * rpb_window[2] - 1) +
              (rpb_window[2] - 1);
  p.H = heads;
  p.C = heads * head_dim;
  p.tile = L->tile_rows;
  p.scale = scale;
  p.use_mask = use_mask;
  const int64_t tf = (int64_t)(2 * rpb_window[0] - 1) * (2 * rpb_window[1] - 1) * (2 * rpb_window[2] - 1) * heads;
  p.table_floats = tf * 4 <= 96 * 1024 ? (int)tf : 0;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (dtype == SSW_F32) {
    if (head_dim == 16) return launch_bwd<float, 16>(p, stream);
    if (head_dim == 32) return launch_bwd<float, 32>(p, stream);
  } else if (dtype == SSW_BF16) {
    if (head_dim == 16) return launch_bwd<__nv_bfloat16, 16>(p, stream);
    if (head_dim == 32) return launch_bwd<__nv_bfloat16, 32>(p, stream);
  } else {
    if (head_dim == 16) return launch_bwd<__half, 16>(p, stream);
    if (head_dim == 32) return launch_bwd<__half, 32>(p, stream);
  }
  return SSW_E_UNSUPPORTED;
}
