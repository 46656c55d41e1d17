// Fused window attention for 16-bit inputs (bf16 / fp16) on tensor cores.
//
// Same persistent producer/consumer pipeline as the CUDA-core kernel (one CTA per SM, producer
// warps that gather voxel rows with one 1-D bulk (TMA) copy per row, `full`/`empty` mbarriers with
// bounded waits), but the rows stay 16-bit in shared memory and the arithmetic is warp-level MMA
// (m16n8k16, fp32 accumulation):
//
//   * The plan is *padded*: inside a pack every window gets a run of row slots rounded up to
//     1, 2, 4, 8, 16, 32, 48 or 64, so a 16-slot MMA tile holds whole windows (several when c < 16)
//     or a 16-row slice of one window.  Unused slots keep whatever an earlier item left in their
//     q and k parts (their scores are replaced, not multiplied, so the contents do not matter) and
//     get their v part zeroed by the producer (p = 0 times a stale Inf would be NaN); their query
//     rows are never stored.
//   * Q comes in as A fragments (ldmatrix), K as B fragments (ldmatrix), S = Q K^T lands in fp32
//     accumulators whose layout is also the A layout of the next MMA, so P = softmax(S) is packed
//     to 16 bit in registers and multiplied with V (ldmatrix.trans).
//   * Windows of up to 16 voxels (nine in ten on a surface scene): a warp takes a 16-slot tile and
//     walks all heads inside it, so the per-key metadata, the window / region comparisons and the
//     bias rows (one 16-byte load per (query, key) pair brings four heads) are worked out once per
//     tile.  Larger windows: a unit of work is (16-slot tile, head) looping over 16-key blocks with
//     an online softmax.
//   * Softmax keeps upstream's semantics: the running maximum starts at 0, the denominator gets
//     +1e-8; bias from the shared-memory table (pre-multiplied by log2 e, heads padded to a
//     multiple of four), -100 shift mask.
//   * Outputs go from the accumulator registers straight to the voxels' rows.
//   * Values that are not finite: upstream confines them to their own window; here a v row that
//     holds Inf or NaN also spoils the other windows that share its 16-slot tile (p = 0 for those
//     keys, and 0 * Inf is NaN inside the MMA).
//
// Phase 1 (packs): every consumer group of four warps takes whole work items, one per pipeline
// stage.  Phase 2 (windows with more voxels than a pack holds): a work item is one tile of query
// rows of such a window; its q rows sit in stage 0 while the window's k|v rows stream through the
// other stages tile by tile, and all consumer warps work on the same key tile, each on its own
// (16 query rows, head) unit whose accumulators stay in registers for the whole window.
#include <math.h>

#include "attn_common.cuh"

namespace ssw {

constexpr int kMmaGroupWarps = 4;
constexpr int kMmaStageVoxOff = 16;
constexpr int kMmaStageRowsOff = kMmaStageVoxOff + kMaxTile * 4;
// Layout of a staged row's metadata word .y: region (5 bits), window inside the pack (7 bits: 0..63,
// kMmaPadWindow for unused slots), row of the bias table (from bit 12).
constexpr int kMmaRelShift = 12;
constexpr int kMmaPadWindow = 64;
constexpr int kMmaWindowBits = 127 << 5;

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

// Metadata of a staged row (see kMmaRelShift): what the producer writes behind the row's data.
// .x: the row's relative-position code (its key-side share of a bias-table row index),
// .y: region | window << 5 | (code + rel_off) << 12 (the query-side share).
__device__ __forceinline__ int2 row_meta(int m, int window, int rel_off) {
  return make_int2(meta_rel(m), meta_region(m) | (window << 5) | ((meta_rel(m) + rel_off) << kMmaRelShift));
}
// zero the v part (C elements from byte 2*C*sizeof(T)) of a staged row
template <typename T>
__device__ __forceinline__ void zero_v(unsigned char* row, int C) {
  uint4* v = reinterpret_cast<uint4*>(row + 2 * C * sizeof(T));
  for (int i = 0; i < (C * (int)sizeof(T)) / 16; ++i) v[i] = make_uint4(0, 0, 0, 0);
}
__device__ __forceinline__ int2 pad_meta(int rel_off) {
  return make_int2(0, (kMmaPadWindow << 5) | (rel_off << kMmaRelShift));
}

// Bias of (query row meta .y, key meta .x) for head h, in the log2 domain.  `tstride`: floats per
// table row (heads padded to a multiple of four in shared memory, the caller's H in global memory).
template <bool kTableSmem>
__device__ __forceinline__ float bias_of(const float* table_base, int tstride, int me_y, int km_x, int h) {
  const float* t = table_base + ((me_y >> kMmaRelShift) - km_x) * tstride + h;
  return kTableSmem ? *t : __ldg(t) * kLog2e;
}
// Additive mask of a (query, key) pair from the XOR of their metadata words: -inf across windows
// (bits 5..11), -100 across shift-mask regions (bits 0..4), else 0.
template <bool kMask>
__device__ __forceinline__ float pair_mask(int x) {
  if (x & kMmaWindowBits) return -INFINITY;
  return (kMask && (x & 31)) ? -100.0f * kLog2e : 0.f;
}

// A 16-slot tile whose windows hold at most 16 voxels: the tile's 16 slots are also its keys.  The
// warp walks all heads; everything that does not depend on the head is computed once.
template <typename T, int HD, bool kTableSmem, bool kMask>
__device__ __forceinline__ void tile_all_heads(const unsigned char* rows, int row_stride, int data_bytes, const int* svox,
                                               int slot0, int H, int C, const float* table_base, int tstride,
                                               float qscale, T* out, int lane) {
  const int qr = lane >> 2, qt = lane & 3, mi = lane >> 3;
  const unsigned char* r_lo = rows + (size_t)(slot0 + qr) * row_stride;
  const unsigned char* r_hi = r_lo + 8 * (size_t)row_stride;
  const int me_lo = reinterpret_cast<const int2*>(r_lo + data_bytes)->y;
  const int me_hi = reinterpret_cast<const int2*>(r_hi + data_bytes)->y;
  const int v_lo = svox[slot0 + qr], v_hi = svox[slot0 + qr + 8];
  // column j of this lane: key slot n*8 + qt*2 + e with j = n*2 + e
  float madd_lo[4], madd_hi[4];
  int kx[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int ks = slot0 + (j >> 1) * 8 + qt * 2 + (j & 1);
    const int2 km = *reinterpret_cast<const int2*>(rows + (size_t)ks * row_stride + data_bytes);
    kx[j] = km.x;
    madd_lo[j] = pair_mask<kMask>(km.y ^ me_lo);
    madd_hi[j] = pair_mask<kMask>(km.y ^ me_hi);
  }
  const unsigned char* qp = rows + (size_t)(slot0 + (mi & 1) * 8 + (lane & 7)) * row_stride + (mi >> 1) * 8 * sizeof(T);
  const unsigned char* kp = rows + (size_t)(slot0 + (mi >> 1) * 8 + (lane & 7)) * row_stride + (C + (mi & 1) * 8) * sizeof(T);
  const unsigned char* vp = rows + (size_t)(slot0 + (mi & 1) * 8 + (lane & 7)) * row_stride + (2 * C + (mi >> 1) * 8) * sizeof(T);
  T* o_lo = out + (int64_t)(v_lo < 0 ? 0 : v_lo) * C + qt * 2;
  T* o_hi = out + (int64_t)(v_hi < 0 ? 0 : v_hi) * C + qt * 2;
  for (int h0 = 0; h0 < H; h0 += 4) {
    // biases of the lane's eight (row, column) pairs for four heads at a time
    float4 b_lo[4], b_hi[4];
    if constexpr (kTableSmem) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        b_lo[j] = *reinterpret_cast<const float4*>(table_base + ((me_lo >> kMmaRelShift) - kx[j]) * tstride + h0);
        b_hi[j] = *reinterpret_cast<const float4*>(table_base + ((me_hi >> kMmaRelShift) - kx[j]) * tstride + h0);
      }
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int h = h0 + t;
      if (h >= H) break;
      const int hoff = h * HD * (int)sizeof(T);
      float sacc[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n) sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        uint32_t qf[4], kf[4];
        ldmatrix_x4(qf, qp + hoff + ks * 16 * sizeof(T));
        ldmatrix_x4(kf, kp + hoff + ks * 16 * sizeof(T));
        mma16816<T>(sacc[0], qf, kf[0], kf[1]);
        mma16816<T>(sacc[1], qf, kf[2], kf[3]);
      }
      float s_lo[4], s_hi[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float bl, bh;
        if constexpr (kTableSmem) {
          bl = t == 0 ? b_lo[j].x : t == 1 ? b_lo[j].y : t == 2 ? b_lo[j].z : b_lo[j].w;
          bh = t == 0 ? b_hi[j].x : t == 1 ? b_hi[j].y : t == 2 ? b_hi[j].z : b_hi[j].w;
        } else {
          bl = bias_of<false>(table_base, tstride, me_lo, kx[j], h);
          bh = bias_of<false>(table_base, tstride, me_hi, kx[j], h);
        }
        s_lo[j] = fmaf(sacc[j >> 1][j & 1], qscale, bl) + madd_lo[j];
        s_hi[j] = fmaf(sacc[j >> 1][2 + (j & 1)], qscale, bh) + madd_hi[j];
      }
      // the row maximum starts from 0 (ops.cu:137)
      float m_lo = fmaxf(fmaxf(s_lo[0], s_lo[1]), fmaxf(s_lo[2], s_lo[3]));
      float m_hi = fmaxf(fmaxf(s_hi[0], s_hi[1]), fmaxf(s_hi[2], s_hi[3]));
      m_lo = fmaxf(m_lo, __shfl_xor_sync(0xffffffffu, m_lo, 1));
      m_hi = fmaxf(m_hi, __shfl_xor_sync(0xffffffffu, m_hi, 1));
      m_lo = fmaxf(fmaxf(m_lo, __shfl_xor_sync(0xffffffffu, m_lo, 2)), 0.f);
      m_hi = fmaxf(fmaxf(m_hi, __shfl_xor_sync(0xffffffffu, m_hi, 2)), 0.f);
      float p_lo[4], p_hi[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        p_lo[j] = fast_exp2(s_lo[j] - m_lo);
        p_hi[j] = fast_exp2(s_hi[j] - m_hi);
      }
      float l_lo = (p_lo[0] + p_lo[1]) + (p_lo[2] + p_lo[3]);
      float l_hi = (p_hi[0] + p_hi[1]) + (p_hi[2] + p_hi[3]);
      l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
      l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
      l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
      l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
      uint32_t pf[4];
      pf[0] = pack2<T>(p_lo[0], p_lo[1]);
      pf[1] = pack2<T>(p_hi[0], p_hi[1]);
      pf[2] = pack2<T>(p_lo[2], p_lo[3]);
      pf[3] = pack2<T>(p_hi[2], p_hi[3]);
      const float inv_lo = 1.0f / (l_lo + 1e-8f), inv_hi = 1.0f / (l_hi + 1e-8f);  // ops.cu:164
#pragma unroll
      for (int n = 0; n < HD / 8; n += 2) {
        uint32_t vf[4];
        float oa[4] = {0.f, 0.f, 0.f, 0.f}, ob[4] = {0.f, 0.f, 0.f, 0.f};
        ldmatrix_x4_trans(vf, vp + hoff + n * 8 * sizeof(T));
        mma16816<T>(oa, pf, vf[0], vf[1]);
        mma16816<T>(ob, pf, vf[2], vf[3]);
        if (v_lo >= 0) {
          *reinterpret_cast<uint32_t*>(o_lo + h * HD + n * 8) = pack2<T>(oa[0] * inv_lo, oa[1] * inv_lo);
          *reinterpret_cast<uint32_t*>(o_lo + h * HD + n * 8 + 8) = pack2<T>(ob[0] * inv_lo, ob[1] * inv_lo);
        }
        if (v_hi >= 0) {
          *reinterpret_cast<uint32_t*>(o_hi + h * HD + n * 8) = pack2<T>(oa[2] * inv_hi, oa[3] * inv_hi);
          *reinterpret_cast<uint32_t*>(o_hi + h * HD + n * 8 + 8) = pack2<T>(ob[2] * inv_hi, ob[3] * inv_hi);
        }
      }
    }
  }
}

// One (16 query rows, head) unit of a window that spans several 16-key blocks: the q fragments, the
// two rows' metadata, the running softmax and the output accumulators of this lane (rows lane/4 and
// lane/4 + 8 of the tile).
template <int HD>
struct MmaUnit {
  uint32_t qf[HD / 16][4];
  float o[HD / 8][4];
  float m_lo, m_hi, l_lo, l_hi;
  int me_lo_y, me_hi_y;
};

// Start a unit on query slots [slot0, slot0 + 16) of the staged rows, head h.
template <typename T, int HD>
__device__ __forceinline__ void unit_begin(MmaUnit<HD>& u, const unsigned char* rows, int row_stride, int data_bytes,
                                           int slot0, int h, int lane) {
  const int qr = lane >> 2, mi = lane >> 3;
  u.me_lo_y = reinterpret_cast<const int2*>(rows + (size_t)(slot0 + qr) * row_stride + data_bytes)->y;
  u.me_hi_y = reinterpret_cast<const int2*>(rows + (size_t)(slot0 + qr + 8) * row_stride + data_bytes)->y;
  const unsigned char* qp =
      rows + (size_t)(slot0 + (mi & 1) * 8 + (lane & 7)) * row_stride + (h * HD + (mi >> 1) * 8) * sizeof(T);
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) ldmatrix_x4(u.qf[ks], qp + ks * 16 * sizeof(T));
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) u.o[n][0] = u.o[n][1] = u.o[n][2] = u.o[n][3] = 0.f;
  u.m_lo = u.m_hi = 0.f;  // the maximum starts from 0 (ops.cu:137)
  u.l_lo = u.l_hi = 0.f;
}

// One block of 16 key slots starting at ks0: S = Q K^T, bias and masks, online softmax, O += P V.
// k_off / v_off: byte offsets of this head's k and v slices inside a staged row.
template <typename T, int HD, bool kTableSmem, bool kMask>
__device__ __forceinline__ void unit_key_block(MmaUnit<HD>& u, const unsigned char* rows, int row_stride, int data_bytes,
                                               int ks0, int k_off, int v_off, const float* table_base, int tstride, int h,
                                               float qscale, int lane) {
  const int qt = lane & 3, mi = lane >> 3;
  float sacc[2][4];
#pragma unroll
  for (int n = 0; n < 2; ++n) sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
  const unsigned char* kp = rows + (size_t)(ks0 + (mi >> 1) * 8 + (lane & 7)) * row_stride + k_off + (mi & 1) * 8 * sizeof(T);
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    uint32_t kf[4];
    ldmatrix_x4(kf, kp + ks * 16 * sizeof(T));
    mma16816<T>(sacc[0], u.qf[ks], kf[0], kf[1]);
    mma16816<T>(sacc[1], u.qf[ks], kf[2], kf[3]);
  }
  // scores -> log2 domain, bias, masks
  float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
  for (int n = 0; n < 2; ++n) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int ks = ks0 + n * 8 + qt * 2 + e;  // key slot of this column
      const int2 km = *reinterpret_cast<const int2*>(rows + (size_t)ks * row_stride + data_bytes);
      const float s_lo = fmaf(sacc[n][e], qscale, bias_of<kTableSmem>(table_base, tstride, u.me_lo_y, km.x, h)) +
                         pair_mask<kMask>(km.y ^ u.me_lo_y);
      const float s_hi = fmaf(sacc[n][2 + e], qscale, bias_of<kTableSmem>(table_base, tstride, u.me_hi_y, km.x, h)) +
                         pair_mask<kMask>(km.y ^ u.me_hi_y);
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
  if (mx_lo > u.m_lo) {
    const float corr = fast_exp2(u.m_lo - mx_lo);
    u.l_lo *= corr;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) { u.o[n][0] *= corr; u.o[n][1] *= corr; }
    u.m_lo = mx_lo;
  }
  if (mx_hi > u.m_hi) {
    const float corr = fast_exp2(u.m_hi - mx_hi);
    u.l_hi *= corr;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) { u.o[n][2] *= corr; u.o[n][3] *= corr; }
    u.m_hi = mx_hi;
  }
  // P in the A-fragment layout of the next MMA
  const float p00 = fast_exp2(sacc[0][0] - u.m_lo), p01 = fast_exp2(sacc[0][1] - u.m_lo);
  const float p02 = fast_exp2(sacc[0][2] - u.m_hi), p03 = fast_exp2(sacc[0][3] - u.m_hi);
  const float p10 = fast_exp2(sacc[1][0] - u.m_lo), p11 = fast_exp2(sacc[1][1] - u.m_lo);
  const float p12 = fast_exp2(sacc[1][2] - u.m_hi), p13 = fast_exp2(sacc[1][3] - u.m_hi);
  u.l_lo += (p00 + p01) + (p10 + p11);
  u.l_hi += (p02 + p03) + (p12 + p13);
  uint32_t pf[4];
  pf[0] = pack2<T>(p00, p01);
  pf[1] = pack2<T>(p02, p03);
  pf[2] = pack2<T>(p10, p11);
  pf[3] = pack2<T>(p12, p13);
  const unsigned char* vp = rows + (size_t)(ks0 + (mi & 1) * 8 + (lane & 7)) * row_stride + v_off + (mi >> 1) * 8 * sizeof(T);
#pragma unroll
  for (int n = 0; n < HD / 8; n += 2) {
    uint32_t vf[4];
    ldmatrix_x4_trans(vf, vp + n * 8 * sizeof(T));
    mma16816<T>(u.o[n], pf, vf[0], vf[1]);
    mma16816<T>(u.o[n + 1], pf, vf[2], vf[3]);
  }
}

// Normalise the unit's output and store it from the accumulator registers to the voxels' rows
// (each lane owns two adjacent channels per 8-channel block of rows lane/4 and lane/4 + 8).
// `svox`: voxel of every slot, -1 for unused.
template <typename T, int HD>
__device__ __forceinline__ void unit_finish(const MmaUnit<HD>& u, const int* svox, int slot0, int h, int C, T* out,
                                            int lane) {
  const int qr = lane >> 2, qt = lane & 3;
  // row sums live in four lanes each
  float ll = u.l_lo, lh = u.l_hi;
  ll += __shfl_xor_sync(0xffffffffu, ll, 1);
  ll += __shfl_xor_sync(0xffffffffu, ll, 2);
  lh += __shfl_xor_sync(0xffffffffu, lh, 1);
  lh += __shfl_xor_sync(0xffffffffu, lh, 2);
  const float inv_lo = 1.0f / (ll + 1e-8f), inv_hi = 1.0f / (lh + 1e-8f);  // ops.cu:164
  const int v_lo = svox[slot0 + qr], v_hi = svox[slot0 + qr + 8];
  if (v_lo >= 0) {
    T* o = out + (int64_t)v_lo * C + h * HD + qt * 2;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) *reinterpret_cast<uint32_t*>(o + n * 8) = pack2<T>(u.o[n][0] * inv_lo, u.o[n][1] * inv_lo);
  }
  if (v_hi >= 0) {
    T* o = out + (int64_t)v_hi * C + h * HD + qt * 2;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) *reinterpret_cast<uint32_t*>(o + n * 8) = pack2<T>(u.o[n][2] * inv_hi, u.o[n][3] * inv_hi);
  }
}

template <typename T, int HD, bool kTableSmem, bool kMask>
__global__ void __launch_bounds__(kMmaGroupWarps * 32 * kMaxGroups + 32 * kMaxProducerWarps, 1) k_attn_mma(AttnParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int tile = p.tile, C = p.C, H = p.H;
  const int S = p.stages, G = p.groups;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);  // phase 1: data of a stage landed
  uint64_t* empty = full + kMaxStages;                  // phase 1: stage may be refilled
  uint64_t* dfull = empty + kMaxStages;                 // phase 2: key tile landed
  uint64_t* dempty = dfull + kMaxStages;                // phase 2: key stage may be refilled
  uint64_t* qfull = dempty + kMaxStages;                // phase 2: query tile landed
  uint64_t* qempty = qfull + 1;                         // phase 2: query stage may be refilled
  uint64_t* tbar = reinterpret_cast<uint64_t*>(smem) + 30;  // bias table landed
  float* table_s = reinterpret_cast<float*>(smem + 256);
  unsigned char* stage0 = smem + 256 + (kTableSmem ? ((p.table_floats * 4 + 15) & ~15) : 0);
  const float* table_base = kTableSmem ? table_s : p.table;
  const int tstride = kTableSmem ? ((H + 3) & ~3) : H;  // floats per bias-table row
  const int gsize = kMmaGroupWarps * 32;
  const int n_cons = gsize * G;
  const int n_cons_warps = G * kMmaGroupWarps;
  const bool is_producer = (int)threadIdx.x >= n_cons;
  const int lane = threadIdx.x & 31;
  const int PW = p.prod_warps, pw = ((int)threadIdx.x - n_cons) >> 5;
  const int data_bytes = 3 * C * (int)sizeof(T);  // one staged row; its metadata follows
  const float qscale = p.scale * kLog2e;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full + s, PW);               // one arrive (with its byte count) per producer warp
      mbar_init(empty + s, kMmaGroupWarps);  // every warp of the consuming group hands the stage back
      mbar_init(dfull + s, PW);
      mbar_init(dempty + s, n_cons_warps);   // every consumer warp works on every key tile
    }
    mbar_init(qfull, PW);
    mbar_init(qempty, n_cons_warps);
    mbar_fence_init();
  }
  __syncthreads();
  grid_dependency_wait();
  const int n_items = checked_count(p.header[SSW_H_PACKS], p);
  const int n_small = min(checked_count(p.header[SSW_H_PACKS_SMALL], p), n_items);
  if constexpr (kTableSmem) {
    if (!is_producer) {  // the producers are already gathering the first items
      stage_table_padded(table_s, p.table, p.table_floats / tstride, H, tstride, threadIdx.x, n_cons);
      consumer_sync(n_cons);
    }
  }

  // ------------------------------------------------------------------------------------------
  // Phase 1: packs
  // ------------------------------------------------------------------------------------------
  const int my_items = n_small > (int)blockIdx.x ? (n_small - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  bool timed_out = false;
  int issued = 0;  // producer warps: phase-1 items whose row copies this warp has submitted
  if (is_producer) {
    // slot -> row of the pack: window wl = slot / cpad, i = slot % cpad, valid if wl < nwin && i < c.
    // Register pipeline, three items deep: the descriptor of item i+5 and the voxel ids / metadata
    // of item i+3 (whose descriptor arrived an iteration ago) are requested while item i is issued,
    // so no iteration waits on a global load.
    // The rows of an item are dealt round-robin to the producer warps: a warp submits its bulk
    // copies one lane after the other, so several warps submit several rows at a time.
    constexpr int kAhead = 3;
    // The plan lists packs by ascending occupancy; walking the list backwards puts the long items
    // first and leaves the short ones for the tail of the kernel.
    auto item_index = [&](int k) { return n_small - 1 - ((int)blockIdx.x + k * (int)gridDim.x); };
    int4 dq[kAhead + 2];
    int vox[kAhead][2], km[kAhead][2];
    auto fetch = [&](const int4& d, int (&v)[2], int (&m)[2]) {
      const int c = d.y, cpad = slots_of_window(c > 0 ? c : 1, 1);
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int slot = (lane + 32 * k) * PW + pw;
        const int wl = slot / cpad, i = slot - wl * cpad;
        v[k] = -1;
        m[k] = 0;
        if (slot < tile && wl < d.z && i < c) {
          v[k] = __ldg(p.pack_perm + d.x + wl * c + i);
          // the in-window position is not needed here: its bits carry the window's index in the pack
          m[k] = (__ldg(p.pack_meta + d.x + wl * c + i) & ~1023) | wl;
        }
      }
    };
#pragma unroll
    for (int a = 0; a <= kAhead + 1; ++a)
      dq[a] = a < my_items ? __ldg(p.pack_desc + item_index(a)) : make_int4(0, 0, 0, 0);
#pragma unroll
    for (int a = 0; a < kAhead; ++a) {
      if (a < my_items) dq[a] = checked_desc(dq[a], p, true);
      fetch(dq[a], vox[a], km[a]);
    }
    for (int i = 0; i < my_items; ++i) {
      const int s = i % S;
      const int use = i / S;
      const int4 d_new = i + kAhead + 2 < my_items
                             ? __ldg(p.pack_desc + item_index(i + kAhead + 2))
                             : make_int4(0, 0, 0, 0);
      int vox_n[2], km_n[2];
      // the descriptor of item i + kAhead arrived iterations ago: checking it here waits for nothing
      if (i + kAhead < my_items) dq[kAhead] = checked_desc(dq[kAhead], p, true);
      fetch(dq[kAhead], vox_n, km_n);  // (an all-zero descriptor fetches nothing)
      if (use > 0 && !mbar_wait_bounded(empty + s, (use - 1) & 1)) {
        timed_out = true;
        break;
      }
      unsigned char* st = stage0 + (size_t)s * p.stage_bytes;
      const int4 d_cur = dq[0];
      if (lane == 0 && pw == 0) *reinterpret_cast<int4*>(st) = d_cur;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int slot = (lane + 32 * k) * PW + pw;
        if (slot < tile) {
          if (vox[0][k] >= 0) {  // loaded three items ago: no wait
            vox[0][k] = checked_voxel(vox[0][k], p);
            km[0][k] = checked_meta(km[0][k], p);
          }
          reinterpret_cast<int*>(st + kMmaStageVoxOff)[slot] = vox[0][k];
          // Unused slots form a window of their own with neutral codes, so their (discarded) scores
          // index inside the bias table; their v part must not hold a stale Inf or NaN.
          unsigned char* row = st + kMmaStageRowsOff + (size_t)slot * p.row_stride;
          *reinterpret_cast<int2*>(row + data_bytes) =
              vox[0][k] >= 0 ? row_meta(km[0][k], km[0][k] & 1023, p.rel_off) : pad_meta(p.rel_off);
          if (vox[0][k] < 0) zero_v<T>(row, C);
        }
      }
      const int my_rows = __popc(__ballot_sync(0xffffffffu, vox[0][0] >= 0)) + __popc(__ballot_sync(0xffffffffu, vox[0][1] >= 0));
      // Zeroed v parts were written through the generic proxy; a later item's bulk copy may land on
      // them.  The arrive releases the stage to the consumers: every lane's stores come before it,
      // and the warp's copies after the byte count they complete against is announced.
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_expect_tx(full + s, (uint32_t)my_rows * (uint32_t)data_bytes);
      __syncwarp();
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int slot = (lane + 32 * k) * PW + pw;
        if (slot < tile && vox[0][k] >= 0)
          bulk_g2s(st + kMmaStageRowsOff + (size_t)slot * p.row_stride,
                   reinterpret_cast<const T*>(p.qkv) + (int64_t)vox[0][k] * 3 * C, data_bytes, full + s);
      }
      issued = i + 1;
#pragma unroll
      for (int a = 0; a <= kAhead; ++a) dq[a] = dq[a + 1];
      dq[kAhead + 1] = d_new;
#pragma unroll
      for (int a = 0; a + 1 < kAhead; ++a) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          vox[a][k] = vox[a + 1][k];
          km[a][k] = km[a + 1][k];
        }
      }
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        vox[kAhead - 1][k] = vox_n[k];
        km[kAhead - 1][k] = km_n[k];
      }
    }
  } else {
    const int g = threadIdx.x / gsize;
    const int wg = (threadIdx.x - g * gsize) >> 5;  // warp inside the group
    for (int i = g; i < my_items && !timed_out; i += G) {
      const int s = i % S;
      const int use = i / S;
      unsigned char* sp = stage0 + (size_t)s * p.stage_bytes;
      unsigned char* rows = sp + kMmaStageRowsOff;
      const int* svox = reinterpret_cast<const int*>(sp + kMmaStageVoxOff);
      if (!mbar_wait_bounded(full + s, use & 1)) {
        timed_out = true;
        break;
      }
      const int4 d = *reinterpret_cast<const int4*>(sp);
      const int c = d.y, nwin = d.z;
      const int cpad = slots_of_window(c, 1);
      const int n_mt = (nwin * cpad + 15) >> 4;
      if (cpad <= 16) {
        // windows of at most 16 voxels: a tile's slots are its keys; one warp per tile, all heads
        for (int mt = wg; mt < n_mt; mt += kMmaGroupWarps)
          tile_all_heads<T, HD, kTableSmem, kMask>(rows, p.row_stride, data_bytes, svox, mt * 16, H, C, table_base,
                                                   tstride, qscale, reinterpret_cast<T*>(p.out), lane);
      } else {
        const int nkb = cpad >> 4;  // 16-key blocks per window
        for (int un = wg; un < n_mt * H; un += kMmaGroupWarps) {
          const int mt = un / H, h = un - mt * H;
          const int kbase = (mt * 16 / cpad) * cpad;  // first key slot of the window this tile belongs to
          MmaUnit<HD> u;
          unit_begin<T, HD>(u, rows, p.row_stride, data_bytes, mt * 16, h, lane);
          for (int kb = 0; kb < nkb; ++kb)
            unit_key_block<T, HD, kTableSmem, kMask>(u, rows, p.row_stride, data_bytes, kbase + kb * 16,
                                                     (C + h * HD) * (int)sizeof(T), (2 * C + h * HD) * (int)sizeof(T),
                                                     table_base, tstride, h, qscale, lane);
          unit_finish<T, HD>(u, svox, mt * 16, h, C, reinterpret_cast<T*>(p.out), lane);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty + s);
    }
  }
  if (timed_out) atomicOr(reinterpret_cast<unsigned*>(p.header + SSW_H_ERROR), SSW_DEV_TIMEOUT);
  // A timed-out role leaves; the other roles then time out on their own bounded waits.
  if (__syncthreads_or(timed_out)) {
    // Nobody consumes what is still in flight, but the CTA must not retire under copies that
    // target its shared memory: each producer warp waits, bounded, for the last use of every stage
    // it submitted copies to (whether the phase completes or not, the wait outlasts any copy).
    if (is_producer && lane == 0)
      for (int j = max(0, issued - S); j < issued; ++j) mbar_wait_bounded(full + j % S, (j / S) & 1);
    return;
  }
  if (n_items <= n_small) return;

  // ------------------------------------------------------------------------------------------
  // Phase 2: windows with c > tile.  Stage 0 holds the item's query rows (q slices), stages
  // 1..S-1 form a ring for the window's key tiles (k|v slices).
  // ------------------------------------------------------------------------------------------
  const int R = S - 1;                           // key stages
  const int n_mt_tile = tile >> 4;               // 16-row tiles per query tile
  const int heads_per_round = n_cons_warps / n_mt_tile;
  const int rounds = (H + heads_per_round - 1) / heads_per_round;
  const uint32_t q_bytes = (uint32_t)C * sizeof(T), kv_bytes = 2u * C * sizeof(T);
  unsigned char* q_stage = stage0;
  unsigned char* q_rows = q_stage + kMmaStageRowsOff;
  int kseq = 0, qseq = 0;  // key tiles / query tiles handled so far by this CTA
  int q_issued = 0, k_issued = 0;  // producer warps: query / key tiles whose copies this warp has submitted
  for (int item = n_small + blockIdx.x; item < n_items && !timed_out; item += gridDim.x, ++qseq) {
    const int4 d = checked_desc(__ldg(p.pack_desc + item), p, false);
    const int c = d.y;
    const int q_first = (-d.z - 1) * tile;
    const int n_q = min(tile, c - q_first);
    const int n_kt = (c + tile - 1) / tile;
    if (is_producer) {
      // query tile
      int qv[2], qm[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int slot = (lane + 32 * k) * PW + pw;
        qv[k] = -1;
        qm[k] = 0;
        if (slot < n_q) {
          qv[k] = checked_voxel(__ldg(p.pack_perm + d.x + q_first + slot), p);
          qm[k] = checked_meta(__ldg(p.pack_meta + d.x + q_first + slot), p);
        }
      }
      if (qseq > 0 && !mbar_wait_bounded(qempty, (qseq - 1) & 1)) {
        timed_out = true;
        break;
      }
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int slot = (lane + 32 * k) * PW + pw;
        if (slot < tile) {
          reinterpret_cast<int*>(q_stage + kMmaStageVoxOff)[slot] = qv[k];
          *reinterpret_cast<int2*>(q_rows + (size_t)slot * p.row_stride + data_bytes) =
              qv[k] >= 0 ? row_meta(qm[k], 0, p.rel_off) : pad_meta(p.rel_off);
        }
      }
      {
        const int my_rows = __popc(__ballot_sync(0xffffffffu, qv[0] >= 0)) + __popc(__ballot_sync(0xffffffffu, qv[1] >= 0));
        __syncwarp();  // every lane's metadata stores before the arrive that releases them
        if (lane == 0) mbar_expect_tx(qfull, (uint32_t)my_rows * q_bytes);
        __syncwarp();
      }
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int slot = (lane + 32 * k) * PW + pw;
        if (slot < tile && qv[k] >= 0)
          bulk_g2s(q_rows + (size_t)slot * p.row_stride, reinterpret_cast<const T*>(p.qkv) + (int64_t)qv[k] * 3 * C,
                   q_bytes, qfull);
      }
      q_issued = qseq + 1;
      // key tiles, once per round of heads
      for (int rt = 0; rt < rounds * n_kt && !timed_out; ++rt, ++kseq) {
        const int kt = rt % n_kt;
        const int k0 = kt * tile, n_k = min(tile, c - k0);
        int kv[2], kmeta[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int slot = (lane + 32 * k) * PW + pw;
          kv[k] = -1;
          kmeta[k] = 0;
          if (slot < n_k) {
            kv[k] = checked_voxel(__ldg(p.pack_perm + d.x + k0 + slot), p);
            kmeta[k] = checked_meta(__ldg(p.pack_meta + d.x + k0 + slot), p);
          }
        }
        const int s = 1 + kseq % R, use = kseq / R;
        if (use > 0 && !mbar_wait_bounded(dempty + s, (use - 1) & 1)) {
          timed_out = true;
          break;
        }
        unsigned char* krows = stage0 + (size_t)s * p.stage_bytes + kMmaStageRowsOff;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int slot = (lane + 32 * k) * PW + pw;
          if (slot < tile) {
            unsigned char* row = krows + (size_t)slot * p.row_stride;
            *reinterpret_cast<int2*>(row + data_bytes) =
                kv[k] >= 0 ? row_meta(kmeta[k], 0, p.rel_off) : pad_meta(p.rel_off);
            if (kv[k] < 0) zero_v<T>(row, C);  // p = 0 times a stale Inf would be NaN
          }
        }
        const int my_rows = __popc(__ballot_sync(0xffffffffu, kv[0] >= 0)) + __popc(__ballot_sync(0xffffffffu, kv[1] >= 0));
        fence_async_smem();  // the zeroed v parts (generic proxy) against later bulk copies onto them
        __syncwarp();        // every lane's stores before the arrive that releases them
        if (lane == 0) mbar_expect_tx(dfull + s, (uint32_t)my_rows * kv_bytes);
        __syncwarp();
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int slot = (lane + 32 * k) * PW + pw;
          if (slot < tile && kv[k] >= 0)
            bulk_g2s(krows + (size_t)slot * p.row_stride + q_bytes,
                     reinterpret_cast<const T*>(p.qkv) + (int64_t)kv[k] * 3 * C + C, kv_bytes, dfull + s);
        }
        k_issued = kseq + 1;
      }
    } else {
      const int cw = threadIdx.x >> 5;  // consumer warp
      const int mt = cw % n_mt_tile, hsel = cw / n_mt_tile;
      if (!mbar_wait_bounded(qfull, qseq & 1)) {
        timed_out = true;
        break;
      }
      for (int r = 0; r < rounds && !timed_out; ++r) {
        const int h = r * heads_per_round + hsel;
        const bool active = hsel < heads_per_round && h < H && mt * 16 < n_q;
        MmaUnit<HD> u;
        if (active) unit_begin<T, HD>(u, q_rows, p.row_stride, data_bytes, mt * 16, h, lane);
        for (int kt = 0; kt < n_kt; ++kt, ++kseq) {
          const int s = 1 + kseq % R, use = kseq / R;
          if (!mbar_wait_bounded(dfull + s, use & 1)) {
            timed_out = true;
            break;
          }
          if (active) {
            const unsigned char* krows = stage0 + (size_t)s * p.stage_bytes + kMmaStageRowsOff;
            const int n_k = min(tile, c - kt * tile);
            for (int kb = 0; kb * 16 < n_k; ++kb)
              unit_key_block<T, HD, kTableSmem, kMask>(u, krows, p.row_stride, data_bytes, kb * 16,
                                                       (C + h * HD) * (int)sizeof(T), (2 * C + h * HD) * (int)sizeof(T),
                                                       table_base, tstride, h, qscale, lane);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(dempty + s);
        }
        if (active && !timed_out)
          unit_finish<T, HD>(u, reinterpret_cast<const int*>(q_stage + kMmaStageVoxOff), mt * 16, h, C,
                             reinterpret_cast<T*>(p.out), lane);
      }
      __syncwarp();
      if (lane == 0 && !timed_out) mbar_arrive(qempty);
    }
  }
  if (timed_out) atomicOr(reinterpret_cast<unsigned*>(p.header + SSW_H_ERROR), SSW_DEV_TIMEOUT);
  if (__syncthreads_or(timed_out) && is_producer && lane == 0) {
    // drain what this warp submitted and nobody will consume (bounded, see phase 1)
    if (q_issued > 0) mbar_wait_bounded(qfull, (q_issued - 1) & 1);
    for (int j = max(0, k_issued - R); j < k_issued; ++j) mbar_wait_bounded(dfull + 1 + j % R, (j / R) & 1);
  }
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
  // in shared memory the table's rows are padded to a multiple of four heads (one 16-byte load
  // then brings the biases of four heads)
  const int tf = (2 * rpb_window[0] - 1) * (2 * rpb_window[1] - 1) * (2 * rpb_window[2] - 1) * ((heads + 3) & ~3);
  // The bias table goes to shared memory when four stages still fit beside it (look-ups from global
  // memory cost a dense window about a quarter of its time); otherwise it stays in global memory.
  const size_t budget = size_t(226) * 1024;
  const size_t tbytes = ((size_t)tf * 4 + 15) & ~size_t(15);
  const bool table_smem = 256 + tbytes + 4 * (size_t)s.stage_bytes <= budget;
  s.table_floats = table_smem ? tf : 0;
  const size_t fixed = 256 + (table_smem ? tbytes : 0);
  int stages = (int)((budget - fixed) / s.stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  int groups = stages - 1;
  if (groups > kMaxGroups) groups = kMaxGroups;
  if (groups < 1) groups = 1;
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
  p.prod_warps = 4;  // 16-bit rows are short: the copy submission rate, not the bytes, bounds the producer
  const int threads = p.groups * kMmaGroupWarps * 32 + 32 * p.prod_warps;
  // four variants: bias table in shared memory or not, shift mask or not
  void (*kern)(AttnParams) =
      s.table_floats > 0 ? (p.use_mask ? k_attn_mma<T, HD, true, true> : k_attn_mma<T, HD, true, false>)
                         : (p.use_mask ? k_attn_mma<T, HD, false, true> : k_attn_mma<T, HD, false, false>);
  SSW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s.smem));
  SSW_CUDA_TRY(launch_chained(kern, dim3(sms), dim3(threads), s.smem, stream, p));
  SSW_LAUNCH_CHECK("k_attn_mma");
  return SSW_OK;
}

// Padded plan, 16-bit inputs: packs and larger windows.  `p` arrives with the plan pointers,
// qkv/out/table, H, C, tile, scale, use_mask and rel_off filled in.
int run_attn_mma(AttnParams p, int dtype, int head_dim, const int32_t rpb_window[3], cudaStream_t stream) {
  const MmaShape s = mma_shape(p.tile, p.H, head_dim, rpb_window);
  // three stages at least: the second phase keeps the query tile in one and needs two for key tiles
  if (s.stages < 3 || s.smem > 227 * 1024) return SSW_E_UNSUPPORTED;
  if (p.tile & 15) return SSW_E_INVALID;
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
