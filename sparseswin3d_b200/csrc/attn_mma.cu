// Fused window attention for 16-bit inputs (bf16 / fp16) on tensor cores.
//
// Same persistent producer/consumer pipeline as the CUDA-core kernel (one CTA per SM, one producer
// warp that gathers whole q|k|v rows with one 1-D bulk (TMA) copy per voxel, `full`/`empty`/`done`
// mbarriers, bulk (TMA) stores of finished rows), but the rows stay 16-bit in shared memory and the
// arithmetic is warp-level MMA (m16n8k16, fp32 accumulation):
//
//   * The plan is *padded*: inside a pack every window gets a run of row slots rounded up to
//     1, 2, 4, 8, 16, 32, 48 or 64, so a 16-slot MMA tile holds whole windows (several when c < 16)
//     or a 16-row slice of one window.  Unused slots keep stale (finite) data; their keys are
//     masked out, their query rows are never stored.
//   * A warp takes (16-slot tile, head) units.  Q comes in as A fragments (ldmatrix), K as B
//     fragments (ldmatrix), S = Q K^T lands in fp32 accumulators whose layout is also the A layout
//     of the next MMA, so P = softmax(S) is packed to 16 bit in registers and multiplied with V
//     (ldmatrix.trans).  Windows longer than 16 loop over 16-key blocks with an online softmax.
//   * Softmax keeps upstream's semantics: the running maximum starts at 0, the denominator gets
//     +1e-8; bias from the shared-memory table (pre-multiplied by log2 e), -100 shift mask.
//   * The output tile overwrites the q slice it came from and leaves through bulk stores.
//
// Windows with more voxels than a pack holds are left to the CUDA-core kernel's second phase.
#include <math.h>
#include <stdlib.h>

#include "attn_common.cuh"

namespace ssw {

constexpr int kMmaGroupWarps = 4;
constexpr int kMmaStageVoxOff = 16;
constexpr int kMmaStageRowsOff = kMmaStageVoxOff + kMaxTile * 4;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

template <typename T, int HD, bool kTableSmem>
__global__ void __launch_bounds__(kMmaGroupWarps * 32 * kMaxGroups + 32, 1) k_attn_mma(AttnParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int tile = p.tile, C = p.C, H = p.H;
  const int S = p.stages, G = p.groups;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + kMaxStages;
  uint64_t* done = empty + kMaxStages;
  float* table_s = reinterpret_cast<float*>(smem + 256);
  unsigned char* stage0 = smem + 256 + (kTableSmem ? ((p.table_floats * 4 + 15) & ~15) : 0);
  const float* table_base = kTableSmem ? table_s : p.table;
  const int gsize = kMmaGroupWarps * 32;
  const int n_cons = gsize * G;
  const bool is_producer = (int)threadIdx.x >= n_cons;
  const int lane = threadIdx.x & 31;
  const int data_bytes = 3 * C * (int)sizeof(T);  // one staged row; its metadata follows
  const float qscale = p.scale * kLog2e;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
      mbar_init(done + s, kMmaGroupWarps);
    }
    mbar_fence_init();
  }
  // unused row slots are read as keys/values (and masked): they must hold finite numbers
  for (int i = threadIdx.x; i < (S * p.stage_bytes) / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(stage0)[i] = make_uint4(0, 0, 0, 0);
  fence_async_smem();  // order the zero fill before the bulk copies that will land in the same rows
  grid_dependency_wait();
  if constexpr (kTableSmem)
    for (int i = threadIdx.x; i < p.table_floats; i += blockDim.x) table_s[i] = __ldg(p.table + i) * kLog2e;
  const int n_small = p.header[SSW_H_PACKS_SMALL];
  __syncthreads();

  const int my_items = n_small > (int)blockIdx.x ? (n_small - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  bool timed_out = false;
  if (is_producer) {
    // slot -> row of the pack: window wl = slot / cpad, i = slot % cpad, valid if wl < nwin && i < c
    int4 d_cur = make_int4(0, 0, 0, 0), d_nxt = make_int4(0, 0, 0, 0);
    int vox[2] = {-1, -1}, km[2] = {0, 0};
    auto fetch = [&](const int4& d, int (&v)[2], int (&m)[2]) {
      const int c = d.y, cpad = slots_of_window(c, 1);
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int slot = lane + 32 * k;
        const int wl = slot / cpad, i = slot - wl * cpad;
        v[k] = -1;
        m[k] = 0;
        if (slot < tile && wl < d.z && i < c) {
          v[k] = __ldg(p.pack_perm + d.x + wl * c + i);
          m[k] = __ldg(p.pack_meta + d.x + wl * c + i);
        }
      }
    };
    if (my_items > 0) d_cur = __ldg(p.pack_desc + blockIdx.x);
    if (my_items > 1) d_nxt = __ldg(p.pack_desc + blockIdx.x + gridDim.x);
    if (my_items > 0) fetch(d_cur, vox, km);
    for (int i = 0; i < my_items; ++i) {
      const int s = i % S;
      const int use = i / S;
      int4 d_nn = make_int4(0, 0, 0, 0);
      if (i + 2 < my_items) d_nn = __ldg(p.pack_desc + blockIdx.x + (size_t)(i + 2) * gridDim.x);
      int vox_n[2] = {-1, -1}, km_n[2] = {0, 0};
      if (i + 1 < my_items) fetch(d_nxt, vox_n, km_n);
      if (use > 0 && !mbar_wait_bounded(empty + s, (use - 1) & 1)) {
        timed_out = true;
        break;
      }
      unsigned char* st = stage0 + (size_t)s * p.stage_bytes;
      if (lane == 0) *reinterpret_cast<int4*>(st) = d_cur;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int slot = lane + 32 * k;
        if (slot < tile) {
          reinterpret_cast<int*>(st + kMmaStageVoxOff)[slot] = vox[k];
          // unused slots get neutral metadata so that their (discarded) scores index inside the table
          *reinterpret_cast<int2*>(st + kMmaStageRowsOff + (size_t)slot * p.row_stride + data_bytes) =
              vox[k] >= 0 ? make_int2(meta_rel(km[k]) * H * 4, meta_region(km[k]) | ((meta_rel(km[k]) + p.rel_off) << 8))
                          : make_int2(0, p.rel_off << 8);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_expect_tx(full + s, (uint32_t)(d_cur.z * d_cur.y) * (uint32_t)data_bytes);
      __syncwarp();
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int slot = lane + 32 * k;
        if (slot < tile && vox[k] >= 0)
          bulk_g2s(st + kMmaStageRowsOff + (size_t)slot * p.row_stride,
                   reinterpret_cast<const T*>(p.qkv) + (int64_t)vox[k] * 3 * C, data_bytes, full + s);
      }
      d_cur = d_nxt;
      d_nxt = d_nn;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        vox[k] = vox_n[k];
        km[k] = km_n[k];
      }
    }
  } else {
    const int g = threadIdx.x / gsize;
    const int wg = (threadIdx.x - g * gsize) >> 5;  // warp inside the group
    const bool store_warp = wg == 0;
    const int qr = lane >> 2, qt = lane & 3;        // fragment coordinates of this lane
    for (int i = g; i < my_items && !timed_out; i += G) {
      const int s = i % S;
      const int use = i / S;
      unsigned char* sp = stage0 + (size_t)s * p.stage_bytes;
      unsigned char* rows = sp + kMmaStageRowsOff;
      if (!mbar_wait_bounded(full + s, use & 1)) {
        timed_out = true;
        break;
      }
      const int4 d = *reinterpret_cast<const int4*>(sp);
      const int c = d.y, nwin = d.z;
      const int cpad = slots_of_window(c, 1);
      const int n_mt = (nwin * cpad + 15) >> 4;
      const int nkb = cpad > 16 ? cpad >> 4 : 1;  // 16-key blocks per window
      for (int u = wg; u < n_mt * H; u += kMmaGroupWarps) {
        const int mt = u / H, h = u - mt * H;
        const int slot_lo = mt * 16 + qr, slot_hi = slot_lo + 8;
        // first key slot of the window(s) this tile belongs to
        const int kbase = cpad > 16 ? (mt * 16 / cpad) * cpad : mt * 16;
        const int2 me_lo = *reinterpret_cast<const int2*>(rows + (size_t)slot_lo * p.row_stride + data_bytes);
        const int2 me_hi = *reinterpret_cast<const int2*>(rows + (size_t)slot_hi * p.row_stride + data_bytes);
        const unsigned char* tab_lo = reinterpret_cast<const unsigned char*>(table_base + (me_lo.y >> 8) * H + h);
        const unsigned char* tab_hi = reinterpret_cast<const unsigned char*>(table_base + (me_hi.y >> 8) * H + h);
        const int reg_lo = me_lo.y & 31, reg_hi = me_hi.y & 31;
        const int win_lo = slot_lo / cpad, win_hi = slot_hi / cpad;  // window of my two query rows

        // Q fragments: HD/16 k-steps
        uint32_t qf[HD / 16][4];
        {
          const int mi = lane >> 3;
          const unsigned char* qp = rows + (size_t)(mt * 16 + (mi & 1) * 8 + (lane & 7)) * p.row_stride +
                                    (h * HD + (mi >> 1) * 8) * sizeof(T);
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) ldmatrix_x4(qf[ks], qp + ks * 16 * sizeof(T));
        }
        float o[HD / 8][4];
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
        float m_lo = 0.f, m_hi = 0.f, l_lo = 0.f, l_hi = 0.f;  // maximum starts from 0 (ops.cu:137)

        for (int kb = 0; kb < nkb; ++kb) {
          const int ks0 = kbase + kb * 16;  // first key slot of this block
          float sacc[2][4];
#pragma unroll
          for (int n = 0; n < 2; ++n) sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
          {
            const int mi = lane >> 3;
            const unsigned char* kp = rows + (size_t)(ks0 + (mi >> 1) * 8 + (lane & 7)) * p.row_stride +
                                      (C + h * HD + (mi & 1) * 8) * sizeof(T);
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
              uint32_t kf[4];
              ldmatrix_x4(kf, kp + ks * 16 * sizeof(T));
              mma16816<T>(sacc[0], qf[ks], kf[0], kf[1]);
              mma16816<T>(sacc[1], qf[ks], kf[2], kf[3]);
            }
          }
          // scores -> log2 domain, bias, masks
          float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
          for (int n = 0; n < 2; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int ks = ks0 + n * 8 + qt * 2 + e;  // key slot of this column
              const int2 km = *reinterpret_cast<const int2*>(rows + (size_t)ks * p.row_stride + data_bytes);
              const int kwin = ks / cpad;
              const bool kvalid = (ks - kwin * cpad) < c && kwin < nwin;
              const float b_lo = kTableSmem ? *reinterpret_cast<const float*>(tab_lo - km.x)
                                            : __ldg(reinterpret_cast<const float*>(tab_lo - km.x)) * kLog2e;
              const float b_hi = kTableSmem ? *reinterpret_cast<const float*>(tab_hi - km.x)
                                            : __ldg(reinterpret_cast<const float*>(tab_hi - km.x)) * kLog2e;
              float s_lo = fmaf(sacc[n][e], qscale, b_lo), s_hi = fmaf(sacc[n][2 + e], qscale, b_hi);
              if (p.use_mask) {
                const int kr = km.y & 31;
                if (reg_lo != kr) s_lo += -100.0f * kLog2e;
                if (reg_hi != kr) s_hi += -100.0f * kLog2e;
              }
              s_lo = (kvalid && kwin == win_lo) ? s_lo : -INFINITY;
              s_hi = (kvalid && kwin == win_hi) ? s_hi : -INFINITY;
              sacc[n][e] = s_lo;
              sacc[n][2 + e] = s_hi;
              mx_lo = fmaxf(mx_lo, s_lo);
              mx_hi = fmaxf(mx_hi, s_hi);
            }
          }
          mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
          mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
          mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
          mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
          if (mx_lo > m_lo) {
            const float corr = fast_exp2(m_lo - mx_lo);
            l_lo *= corr;
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) { o[n][0] *= corr; o[n][1] *= corr; }
            m_lo = mx_lo;
          }
          if (mx_hi > m_hi) {
            const float corr = fast_exp2(m_hi - mx_hi);
            l_hi *= corr;
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) { o[n][2] *= corr; o[n][3] *= corr; }
            m_hi = mx_hi;
          }
          // P in the A-fragment layout of the next MMA
          uint32_t pf[4];
          {
            const float p00 = fast_exp2(sacc[0][0] - m_lo), p01 = fast_exp2(sacc[0][1] - m_lo);
            const float p02 = fast_exp2(sacc[0][2] - m_hi), p03 = fast_exp2(sacc[0][3] - m_hi);
            const float p10 = fast_exp2(sacc[1][0] - m_lo), p11 = fast_exp2(sacc[1][1] - m_lo);
            const float p12 = fast_exp2(sacc[1][2] - m_hi), p13 = fast_exp2(sacc[1][3] - m_hi);
            l_lo += (p00 + p01) + (p10 + p11);
            l_hi += (p02 + p03) + (p12 + p13);
            pf[0] = pack2<T>(p00, p01);
            pf[1] = pack2<T>(p02, p03);
            pf[2] = pack2<T>(p10, p11);
            pf[3] = pack2<T>(p12, p13);
          }
          {
            const int mi = lane >> 3;
            const unsigned char* vp = rows + (size_t)(ks0 + (mi & 1) * 8 + (lane & 7)) * p.row_stride +
                                      (2 * C + h * HD + (mi >> 1) * 8) * sizeof(T);
#pragma unroll
            for (int n = 0; n < HD / 8; n += 2) {
              uint32_t vf[4];
              ldmatrix_x4_trans(vf, vp + n * 8 * sizeof(T));
              mma16816<T>(o[n], pf, vf[0], vf[1]);
              mma16816<T>(o[n + 1], pf, vf[2], vf[3]);
            }
          }
        }
        // row sums live in four lanes each
        l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
        l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
        const float inv_lo = 1.0f / (l_lo + 1e-8f), inv_hi = 1.0f / (l_hi + 1e-8f);  // ops.cu:164
        // the q slice this tile was read from becomes its output slice
        __syncwarp();
        uint32_t* out_lo = reinterpret_cast<uint32_t*>(rows + (size_t)slot_lo * p.row_stride + (h * HD) * sizeof(T)) + qt;
        uint32_t* out_hi = reinterpret_cast<uint32_t*>(rows + (size_t)slot_hi * p.row_stride + (h * HD) * sizeof(T)) + qt;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
          out_lo[n * 4] = pack2<T>(o[n][0] * inv_lo, o[n][1] * inv_lo);
          out_hi[n * 4] = pack2<T>(o[n][2] * inv_hi, o[n][3] * inv_hi);
        }
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(done + s);
      if (store_warp) {
        if (!mbar_wait_bounded(done + s, use & 1)) {
          timed_out = true;
          break;
        }
        const int* svox = reinterpret_cast<const int*>(sp + kMmaStageVoxOff);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int slot = lane + 32 * k;
          if (slot < tile) {
            const int v = svox[slot];
            if (v >= 0)
              bulk_s2g(reinterpret_cast<T*>(p.out) + (int64_t)v * C, rows + (size_t)slot * p.row_stride,
                       C * sizeof(T));
          }
        }
        bulk_commit();
        bulk_wait_read_all();
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
      }
    }
    if (store_warp) bulk_wait_all();
  }
  if (timed_out) atomicOr(reinterpret_cast<unsigned*>(p.header + SSW_H_ERROR), SSW_DEV_TIMEOUT);
  __syncthreads();
}

struct MmaShape {
  int groups, stages, row_stride, stage_bytes, table_floats;
  size_t smem;
};
static MmaShape mma_shape(int tile, int heads, int head_dim, const int32_t rpb_window[3]) {
  MmaShape s;
  const int C = heads * head_dim;
  s.row_stride = 3 * C * 2 + 16;  // +16 B: per-row metadata, and consecutive rows fall on different banks
  s.stage_bytes = kMmaStageRowsOff + tile * s.row_stride;
  const int tf = (2 * rpb_window[0] - 1) * (2 * rpb_window[1] - 1) * (2 * rpb_window[2] - 1) * heads;
  s.table_floats = tf * 4 <= 40 * 1024 ? tf : 0;
  const size_t fixed = 256 + ((s.table_floats * 4 + 15) & ~15);
  int stages = (int)((size_t(226) * 1024 - fixed) / s.stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  int groups = stages - 1;
  if (groups > kMaxGroups) groups = kMaxGroups;
  if (groups < 1) groups = 1;
  if (const char* e = getenv("SSW_STAGES")) {
    const int v = atoi(e);
    if (v >= 2 && v <= stages) stages = v;
  }
  if (const char* e = getenv("SSW_GROUPS")) {
    const int v = atoi(e);
    if (v >= 1 && v <= kMaxGroups && v <= stages) groups = v;
  }
  if (groups > stages) groups = stages;
  s.stages = stages;
  s.groups = groups;
  s.smem = fixed + (size_t)(stages > 0 ? stages : 1) * s.stage_bytes;
  return s;
}

// The largest tile of 64/32/16 slots that leaves at least four pipeline stages.
int mma_default_tile(int heads, int head_dim, const int32_t rpb_window[3]) {
  static const int kTiles[] = {64, 32, 16};
  for (int tile : kTiles)
    if (mma_shape(tile, heads, head_dim, rpb_window).stages >= 4) return tile;
  return 16;
}

template <typename T, int HD>
static int launch_mma(AttnParams p, const MmaShape& s, cudaStream_t stream) {
  int dev = 0, sms = 0;
  SSW_CUDA_TRY(cudaGetDevice(&dev));
  SSW_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int threads = s.groups * kMmaGroupWarps * 32 + 32;
  if (s.table_floats > 0) {
    auto kern = k_attn_mma<T, HD, true>;
    SSW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s.smem));
    SSW_CUDA_TRY(launch_chained(kern, dim3(sms), dim3(threads), s.smem, stream, p));
  } else {
    auto kern = k_attn_mma<T, HD, false>;
    SSW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s.smem));
    SSW_CUDA_TRY(launch_chained(kern, dim3(sms), dim3(threads), s.smem, stream, p));
  }
  return SSW_OK;
}

// Packs of a padded plan, 16-bit inputs.  `p` arrives with the plan pointers, qkv/out/table, H, C,
// tile, scale, use_mask and rel_off filled in.
int run_attn_mma(AttnParams p, int dtype, int head_dim, const int32_t rpb_window[3], cudaStream_t stream) {
  const MmaShape s = mma_shape(p.tile, p.H, head_dim, rpb_window);
  if (s.stages < 2 || s.smem > 227 * 1024) return SSW_E_UNSUPPORTED;
  p.groups = s.groups;
  p.stages = s.stages;
  p.row_stride = s.row_stride;
  p.stage_bytes = s.stage_bytes;
  p.table_floats = s.table_floats;
  if (dtype == SSW_BF16) {
    if (head_dim == 16) return launch_mma<__nv_bfloat16, 16>(p, s, stream);
    if (head_dim == 32) return launch_mma<__nv_bfloat16, 32>(p, s, stream);
  } else if (dtype == SSW_F16) {
    if (head_dim == 16) return launch_mma<__half, 16>(p, s, stream);
    if (head_dim == 32) return launch_mma<__half, 32>(p, s, stream);
  }
  return SSW_E_UNSUPPORTED;
}

}  // namespace ssw
