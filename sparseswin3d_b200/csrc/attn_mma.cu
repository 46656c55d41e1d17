// Fused window attention for 16-bit inputs (bf16 / fp16) on tensor cores.
//
// Same persistent producer/consumer pipeline as the CUDA-core kernel (one CTA per SM, producer
// warps that gather voxel rows with one 1-D bulk (TMA) copy per row, `full`/`empty` mbarriers with
// bounded waits), but the rows stay 16-bit in shared memory and the arithmetic is warp-level MMA
// (m16n8k16, fp32 accumulation):
//
//   * The plan is *padded*: inside a pack every window gets a run of row slots rounded up to
//     1, 2, 4, 8, 16, 32, 48 or 64, so a 16-slot MMA tile holds whole windows (several when c < 16)
//     or a 16-row slice of one window.  Unused slots keep whatever an earlier item left in them;
//     as keys they are never read: the ldmatrix row addresses of unused slots point at a row of
//     zeros instead (their scores then get -inf and their probabilities are 0; -inf plus a NaN
//     score or 0 times a stale Inf would be NaN).  As queries they give rows that are never stored.
//   * Q comes in as A fragments (ldmatrix), K as B fragments (ldmatrix), S = Q K^T lands in fp32
//     accumulators whose layout is also the A layout of the next MMA, so P = softmax(S) is packed
//     to 16 bit in registers and multiplied with V (ldmatrix.trans).
//   * A unit of work is (16-slot tile, head).  Windows of up to 16 voxels (nine in ten on a surface
//     scene) see one block of 16 keys: scores, row maximum (from 0), probabilities and the output
//     in one straight pass.  Larger windows loop over 16-key blocks with an online softmax.
//   * All consumer warps work on the same item, each on its own units, so an item's stage is held
//     for about one unit's time and the other stages of the ring are copies in flight: what bounds
//     this kernel is how far the row gathers run ahead, not the arithmetic.
//   * Softmax keeps upstream's semantics: the running maximum starts at 0, the denominator gets
//     +1e-8; bias from the shared-memory table (pre-multiplied by log2 e), -100 shift mask.
//   * Outputs go from the accumulator registers straight to the voxels' rows.
//   * Values that are not finite: upstream confines them to their own window; here a v row that
//     holds Inf or NaN also spoils the other windows that share its 16-slot tile (p = 0 for those
//     keys, and 0 * Inf is NaN inside the MMA).
//
// Phase 1 (packs): one work item per pipeline stage.  Phase 2 (windows with more voxels than a pack holds): a work item is one tile of query
// rows of such a window; its q rows sit in stage 0 while the window's k|v rows stream through the
// other stages tile by tile, and all consumer warps work on the same key tile, each on its own
// (16 query rows, head) unit whose accumulators stay in registers for the whole window.
#include <math.h>

#include "attn_common.cuh"

namespace ssw {

constexpr int kMmaGroupWarps = 4;
constexpr int kMmaGroups = 3;  // 12 consumer warps: with up to six producer warps 576 threads, 96 registers each

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
__device__ __forceinline__ int2 pad_meta(int rel_off) {
  return make_int2(0, (kMmaPadWindow << 5) | (rel_off << kMmaRelShift));
}
__device__ __forceinline__ bool is_pad_meta(int me_y) { return ((me_y >> 5) & 127) == kMmaPadWindow; }
// Where ldmatrix reads slot `slot` as a key (k and v slices): the staged row, or a row of zeros for
// an unused slot.
__device__ __forceinline__ const unsigned char* key_row(const unsigned char* rows, int row_stride, int data_bytes, int slot,
                                                        const unsigned char* zero_row) {
  const unsigned char* r = rows + (size_t)slot * row_stride;
  return is_pad_meta(reinterpret_cast<const int2*>(r + data_bytes)->y) ? zero_row : r;
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

// One (16-slot tile, head) unit whose windows hold at most 16 voxels: the tile's 16 slots are also
// its keys, so there is one block of scores and no running state.
template <typename T, int HD, bool kTableSmem, bool kMask>
__device__ __forceinline__ void tile_head(const unsigned char* rows, int row_stride, int data_bytes, const int* svox,
                                          const unsigned char* zero_row, int slot0, int h, int C, const float* table_base,
                                          int tstride, float qscale, const OutSet& outs, int lane) {
  const int qr = lane >> 2, qt = lane & 3, mi = lane >> 3;
  const unsigned char* r_lo = rows + (size_t)(slot0 + qr) * row_stride;
  const unsigned char* r_hi = r_lo + 8 * (size_t)row_stride;
  const int me_lo = reinterpret_cast<const int2*>(r_lo + data_bytes)->y;
  const int me_hi = reinterpret_cast<const int2*>(r_hi + data_bytes)->y;
  const int hoff = h * HD * (int)sizeof(T);
  const unsigned char* qp =
      rows + (size_t)(slot0 + (mi & 1) * 8 + (lane & 7)) * row_stride + hoff + (mi >> 1) * 8 * sizeof(T);
  const unsigned char* kp = key_row(rows, row_stride, data_bytes, slot0 + (mi >> 1) * 8 + (lane & 7), zero_row) + hoff +
                            (C + (mi & 1) * 8) * sizeof(T);
  const unsigned char* vp = key_row(rows, row_stride, data_bytes, slot0 + (mi & 1) * 8 + (lane & 7), zero_row) + hoff +
                            (2 * C + (mi >> 1) * 8) * sizeof(T);
  float sacc[2][4];
#pragma unroll
  for (int n = 0; n < 2; ++n) sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    uint32_t qf[4], kf[4];
    ldmatrix_x4(qf, qp + ks * 16 * sizeof(T));
    ldmatrix_x4(kf, kp + ks * 16 * sizeof(T));
    mma16816<T>(sacc[0], qf, kf[0], kf[1]);
    mma16816<T>(sacc[1], qf, kf[2], kf[3]);
  }
  // the V fragments do not depend on the scores: request them before the softmax arithmetic
  uint32_t vf[HD / 16][4];
#pragma unroll
  for (int n = 0; n < HD / 16; ++n) ldmatrix_x4_trans(vf[n], vp + n * 16 * sizeof(T));
  // column j of this lane: key slot n*8 + qt*2 + e with j = n*2 + e
  float s_lo[4], s_hi[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int ks = slot0 + (j >> 1) * 8 + qt * 2 + (j & 1);
    const int2 km = *reinterpret_cast<const int2*>(rows + (size_t)ks * row_stride + data_bytes);
    s_lo[j] = fmaf(sacc[j >> 1][j & 1], qscale, bias_of<kTableSmem>(table_base, tstride, me_lo, km.x, h)) +
              pair_mask<kMask>(km.y ^ me_lo);
    s_hi[j] = fmaf(sacc[j >> 1][2 + (j & 1)], qscale, bias_of<kTableSmem>(table_base, tstride, me_hi, km.x, h)) +
              pair_mask<kMask>(km.y ^ me_hi);
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
  // bf16 keeps 8 bits of a probability: the rounding residual goes through a second MMA (see
  // unit_key_block)
  constexpr bool kSplitP = std::is_same<T, __nv_bfloat16>::value;
  uint32_t pl[4];
  if constexpr (kSplitP) {
    pl[0] = pack2<T>(p_lo[0] - __uint_as_float(pf[0] << 16), p_lo[1] - __uint_as_float(pf[0] & 0xffff0000u));
    pl[1] = pack2<T>(p_hi[0] - __uint_as_float(pf[1] << 16), p_hi[1] - __uint_as_float(pf[1] & 0xffff0000u));
    pl[2] = pack2<T>(p_lo[2] - __uint_as_float(pf[2] << 16), p_lo[3] - __uint_as_float(pf[2] & 0xffff0000u));
    pl[3] = pack2<T>(p_hi[2] - __uint_as_float(pf[3] << 16), p_hi[3] - __uint_as_float(pf[3] & 0xffff0000u));
  }
  const float inv_lo = __frcp_rn(l_lo + 1e-8f), inv_hi = __frcp_rn(l_hi + 1e-8f);  // ops.cu:164
  const int v_lo = svox[slot0 + qr], v_hi = svox[slot0 + qr + 8];
  const int64_t off_lo = (int64_t)(v_lo < 0 ? 0 : v_lo) * C + h * HD + qt * 2;
  const int64_t off_hi = (int64_t)(v_hi < 0 ? 0 : v_hi) * C + h * HD + qt * 2;
#pragma unroll
  for (int n = 0; n < HD / 16; ++n) {
    float oa[4] = {0.f, 0.f, 0.f, 0.f}, ob[4] = {0.f, 0.f, 0.f, 0.f};
    mma16816<T>(oa, pf, vf[n][0], vf[n][1]);
    mma16816<T>(ob, pf, vf[n][2], vf[n][3]);
    if constexpr (kSplitP) {
      mma16816<T>(oa, pl, vf[n][0], vf[n][1]);
      mma16816<T>(ob, pl, vf[n][2], vf[n][3]);
    }
    const uint32_t a_lo = pack2<T>(oa[0] * inv_lo, oa[1] * inv_lo), b_lo = pack2<T>(ob[0] * inv_lo, ob[1] * inv_lo);
    const uint32_t a_hi = pack2<T>(oa[2] * inv_hi, oa[3] * inv_hi), b_hi = pack2<T>(ob[2] * inv_hi, ob[3] * inv_hi);
    for (int d = 0; d < outs.n; ++d) {
      T* out = reinterpret_cast<T*>(outs.base[d]);
      if (v_lo >= 0) {
        *reinterpret_cast<uint32_t*>(out + off_lo + n * 16) = a_lo;
        *reinterpret_cast<uint32_t*>(out + off_lo + n * 16 + 8) = b_lo;
      }
      if (v_hi >= 0) {
        *reinterpret_cast<uint32_t*>(out + off_hi + n * 16) = a_hi;
        *reinterpret_cast<uint32_t*>(out + off_hi + n * 16 + 8) = b_hi;
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
                                               const unsigned char* zero_row, int ks0, int k_off, int v_off,
                                               const float* table_base, int tstride, int h, float qscale, int lane) {
  const int qt = lane & 3, mi = lane >> 3;
  float sacc[2][4];
#pragma unroll
  for (int n = 0; n < 2; ++n) sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
  const unsigned char* kp =
      key_row(rows, row_stride, data_bytes, ks0 + (mi >> 1) * 8 + (lane & 7), zero_row) + k_off + (mi & 1) * 8 * sizeof(T);
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
  // bf16 keeps 8 bits of a probability.  The absolute error that leaves in an output is bounded by
  // 2^-8 * sum p|v|, which a row that averages hundreds of keys (small output, by cancellation) does
  // not forgive.  The rounding residual goes through a second MMA (the tensor pipe is far from
  // busy), which leaves the output rounding as the only 16-bit step after the scores.
  constexpr bool kSplitP = std::is_same<T, __nv_bfloat16>::value;
  uint32_t pl[4];
  if constexpr (kSplitP) {
    pl[0] = pack2<T>(p00 - __uint_as_float(pf[0] << 16), p01 - __uint_as_float(pf[0] & 0xffff0000u));
    pl[1] = pack2<T>(p02 - __uint_as_float(pf[1] << 16), p03 - __uint_as_float(pf[1] & 0xffff0000u));
    pl[2] = pack2<T>(p10 - __uint_as_float(pf[2] << 16), p11 - __uint_as_float(pf[2] & 0xffff0000u));
    pl[3] = pack2<T>(p12 - __uint_as_float(pf[3] << 16), p13 - __uint_as_float(pf[3] & 0xffff0000u));
  }
  const unsigned char* vp =
      key_row(rows, row_stride, data_bytes, ks0 + (mi & 1) * 8 + (lane & 7), zero_row) + v_off + (mi >> 1) * 8 * sizeof(T);
#pragma unroll
  for (int n = 0; n < HD / 8; n += 2) {
    uint32_t vf[4];
    ldmatrix_x4_trans(vf, vp + n * 8 * sizeof(T));
    mma16816<T>(u.o[n], pf, vf[0], vf[1]);
    mma16816<T>(u.o[n + 1], pf, vf[2], vf[3]);
    if constexpr (kSplitP) {
      mma16816<T>(u.o[n], pl, vf[0], vf[1]);
      mma16816<T>(u.o[n + 1], pl, vf[2], vf[3]);
    }
  }
}

// Normalise the unit's output and store it from the accumulator registers to the voxels' rows
// (each lane owns two adjacent channels per 8-channel block of rows lane/4 and lane/4 + 8).
// `svox`: voxel of every slot, -1 for unused.
template <typename T, int HD>
__device__ __forceinline__ void unit_finish(const MmaUnit<HD>& u, const int* svox, int slot0, int h, int C,
                                            const OutSet& outs, int lane) {
  const int qr = lane >> 2, qt = lane & 3;
  // row sums live in four lanes each
  float ll = u.l_lo, lh = u.l_hi;
  ll += __shfl_xor_sync(0xffffffffu, ll, 1);
  ll += __shfl_xor_sync(0xffffffffu, ll, 2);
  lh += __shfl_xor_sync(0xffffffffu, lh, 1);
  lh += __shfl_xor_sync(0xffffffffu, lh, 2);
  const float inv_lo = __frcp_rn(ll + 1e-8f), inv_hi = __frcp_rn(lh + 1e-8f);  // ops.cu:164
  const int v_lo = svox[slot0 + qr], v_hi = svox[slot0 + qr + 8];
  for (int d = 0; d < outs.n; ++d) {
    T* out = reinterpret_cast<T*>(outs.base[d]);
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
}

template <typename T, int HD, bool kTableSmem, bool kMask>
__global__ void __launch_bounds__(kMmaGroupWarps * 32 * kMmaGroups + 32 * kMaxProducerWarps, 1) k_attn_mma(AttnParams p) {
  // p.prod_warps == p.stages: one producer warp per pipeline stage
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
  // [barriers 256 B][plan-prefetch rings of the producer warps][row of zeros, row_stride B][bias table][stages]
  unsigned char* prod_scratch = smem + 256;
  unsigned char* zero_row = prod_scratch + p.prod_warps * producer_scratch_bytes(p.tile);
  float* table_s = reinterpret_cast<float*>(zero_row + p.row_stride);
  bool table_ok = true;
  unsigned char* stage0 = reinterpret_cast<unsigned char*>(table_s) + (kTableSmem ? ((p.table_floats * 4 + 15) & ~15) : 0);
  const float* table_base = kTableSmem ? table_s : p.table;
  const int tstride = H;  // floats per bias-table row
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
      mbar_init(full + s, 1);                // one producer warp gathers an item: its arrive carries the byte count
      mbar_init(empty + s, n_cons_warps);    // every consumer warp hands the stage back
      mbar_init(dfull + s, PW);
      mbar_init(dempty + s, n_cons_warps);   // every consumer warp works on every key tile
    }
    mbar_init(qfull, PW);
    mbar_init(qempty, n_cons_warps);
    mbar_init(tbar, 1);
    mbar_fence_init();
  }
  for (int i = threadIdx.x; i < p.row_stride / 16; i += blockDim.x) reinterpret_cast<uint4*>(zero_row)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  grid_dependency_wait();
  const int n_items = checked_count(p.header[SSW_H_PACKS], p);
  const int n_small = min(checked_count(p.header[SSW_H_PACKS_SMALL], p), n_items);
  if constexpr (kTableSmem) {
    if (!is_producer) {  // the producers are already gathering the first items
      table_ok = stage_table(table_s, p.table, p.table_floats, threadIdx.x, n_cons, tbar);
      consumer_sync(n_cons);
    }
  }

  // ------------------------------------------------------------------------------------------
  // Phase 1: packs
  // ------------------------------------------------------------------------------------------
  const int my_items = n_small > (int)blockIdx.x ? (n_small - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  bool timed_out = !table_ok;
  int issued = 0;  // producer warps: how many of its phase-1 items this warp has submitted row copies for
  if (is_producer) {
    // slot -> row of the pack: window wl = slot / cpad, i = slot % cpad, valid if wl < nwin && i < c.
    // This warp gathers the items pw, pw + S, ... of the CTA into stage pw (PW == S), lane l looking
    // after slots l and l + 32; descriptors, voxel ids and metadata come through the warp's
    // plan-prefetch rings.
    unsigned char* pscr = prod_scratch + (size_t)pw * producer_scratch_bytes(tile);
    int4* dring = reinterpret_cast<int4*>(pscr);
    int2* vring = reinterpret_cast<int2*>(pscr + kDescRing * 16);  // [kVoxRing][tile] {voxel id, metadata}
    // The plan lists packs by ascending occupancy; walking the list backwards puts the long items
    // first and leaves the short ones for the tail of the kernel.
    auto item_index = [&](int k) { return n_small - 1 - ((int)blockIdx.x + k * (int)gridDim.x); };
    const int n_mine = my_items > pw ? (my_items - pw + PW - 1) / PW : 0;
    for (int t = -kDescAhead; t < n_mine; ++t) {
      const int td = t + kDescAhead;
      if (lane == 0 && td < n_mine) cp_async16(dring + (td & (kDescRing - 1)), p.pack_desc + item_index(pw + td * PW));
      // every iteration commits one group; what was requested kVoxAhead iterations ago has landed
      // once at most kVoxAhead - 1 groups are pending: the descriptor of item t + kVoxAhead (asked for
      // kDescAhead - kVoxAhead iterations before that) and the ids / metadata of item t
      cp_async_wait<kVoxAhead - 1>();
      __syncwarp();
      const int tv = t + kVoxAhead;
      if (tv >= 0 && tv < n_mine) {
        const int4 d = checked_desc(dring[tv & (kDescRing - 1)], p, true);
        const int c = d.y, cpad = slots_of_window(c, 1);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int slot = lane + 32 * k;
          const int wl = slot / cpad, ii = slot - wl * cpad;
          if (slot < tile && wl < d.z && ii < c) {
            int2* dst = vring + (tv & (kVoxRing - 1)) * tile + slot;
            cp_async4(&dst->x, p.pack_perm + d.x + wl * c + ii);
            cp_async4(&dst->y, p.pack_meta + d.x + wl * c + ii);
          }
        }
      }
      cp_async_commit();
      if (t < 0) continue;
      const int s = pw, use = t;  // item pw + t * S
      const int4 d_cur = checked_desc(dring[t & (kDescRing - 1)], p, true);
      int vox[2], km[2];
      {
        const int c = d_cur.y, cpad = slots_of_window(c, 1);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int slot = lane + 32 * k;
          const int wl = slot / cpad, ii = slot - wl * cpad;
          vox[k] = -1;
          km[k] = 0;
          if (slot < tile && wl < d_cur.z && ii < c) {
            const int2 e = vring[(t & (kVoxRing - 1)) * tile + slot];
            vox[k] = checked_voxel(e.x, p);
            // the in-window position is not needed here: its bits carry the window's index in the pack
            km[k] = (checked_meta(e.y, p) & ~1023) | wl;
          }
        }
      }
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
          // Unused slots form a window of their own with neutral codes, so their (discarded) scores
          // index inside the bias table.
          *reinterpret_cast<int2*>(st + kMmaStageRowsOff + (size_t)slot * p.row_stride + data_bytes) =
              vox[k] >= 0 ? row_meta(km[k], km[k] & 1023, p.rel_off) : pad_meta(p.rel_off);
        }
      }
      const int my_rows = __popc(__ballot_sync(0xffffffffu, vox[0] >= 0)) + __popc(__ballot_sync(0xffffffffu, vox[1] >= 0));
      // The arrive releases the stage to the consumers: every lane's metadata stores come before
      // it, and the warp's copies after the byte count they complete against is announced.
      __syncwarp();
      if (lane == 0) mbar_expect_tx(full + s, (uint32_t)my_rows * (uint32_t)data_bytes);
      __syncwarp();
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int slot = lane + 32 * k;
        if (slot < tile && vox[k] >= 0)
          bulk_g2s(st + kMmaStageRowsOff + (size_t)slot * p.row_stride,
                   reinterpret_cast<const T*>(p.qkv) + (int64_t)vox[k] * 3 * C, data_bytes, full + s);
      }
      issued = t + 1;
    }
    cp_async_wait<0>();  // nothing of the plan prefetch may still be under way towards this CTA's shared memory
  } else {
    // Every consumer warp visits every item and takes the units un = warp, warp + n_cons_warps, ...
    // of its (16-slot tile, head) grid; a warp without a unit hands the stage back at once.
    const int cw = threadIdx.x >> 5;
    for (int i = 0; i < my_items && !timed_out; ++i) {
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
        // windows of at most 16 voxels: a tile's slots are its keys
        for (int un = cw; un < n_mt * H; un += n_cons_warps) {
          const int h = un / n_mt, mt = un - h * n_mt;
          tile_head<T, HD, kTableSmem, kMask>(rows, p.row_stride, data_bytes, svox, zero_row, mt * 16, h, C, table_base,
                                              tstride, qscale, p.outs, lane);
        }
      } else {
        const int nkb = cpad >> 4;  // 16-key blocks per window
        for (int un = cw; un < n_mt * H; un += n_cons_warps) {
          const int h = un / n_mt, mt = un - h * n_mt;
          const int kbase = (mt * 16 / cpad) * cpad;  // first key slot of the window this tile belongs to
          MmaUnit<HD> u;
          unit_begin<T, HD>(u, rows, p.row_stride, data_bytes, mt * 16, h, lane);
          for (int kb = 0; kb < nkb; ++kb)
            unit_key_block<T, HD, kTableSmem, kMask>(u, rows, p.row_stride, data_bytes, zero_row, kbase + kb * 16,
                                                     (C + h * HD) * (int)sizeof(T), (2 * C + h * HD) * (int)sizeof(T),
                                                     table_base, tstride, h, qscale, lane);
          unit_finish<T, HD>(u, svox, mt * 16, h, C, p.outs, lane);
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
    if (is_producer && lane == 0) drain_producer(full, pw, PW, S, issued);
    if (kTableSmem && threadIdx.x == 0 && !table_ok) mbar_wait_bounded(tbar, 0);
    return;
  }
  if (n_items <= n_small || p.skip_big) return;

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
          if (slot < tile)
            *reinterpret_cast<int2*>(krows + (size_t)slot * p.row_stride + data_bytes) =
                kv[k] >= 0 ? row_meta(kmeta[k], 0, p.rel_off) : pad_meta(p.rel_off);
        }
        const int my_rows = __popc(__ballot_sync(0xffffffffu, kv[0] >= 0)) + __popc(__ballot_sync(0xffffffffu, kv[1] >= 0));
        __syncwarp();        // every lane's metadata stores before the arrive that releases them
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
              unit_key_block<T, HD, kTableSmem, kMask>(u, krows, p.row_stride, data_bytes, zero_row, kb * 16,
                                                       (C + h * HD) * (int)sizeof(T), (2 * C + h * HD) * (int)sizeof(T),
                                                       table_base, tstride, h, qscale, lane);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(dempty + s);
        }
        if (active && !timed_out)
          unit_finish<T, HD>(u, reinterpret_cast<const int*>(q_stage + kMmaStageVoxOff), mt * 16, h, C,
                             p.outs, lane);
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
  const int tf = (2 * rpb_window[0] - 1) * (2 * rpb_window[1] - 1) * (2 * rpb_window[2] - 1) * heads;
  // The bias table goes to shared memory when four stages still fit beside it (look-ups from global
  // memory cost a dense window about a quarter of its time); otherwise it stays in global memory.
  const size_t budget = size_t(226) * 1024;
  const size_t tbytes = ((size_t)tf * 4 + 15) & ~size_t(15);
  // Barriers, the row of zeros, the table (when four stages still fit beside it: look-ups from global
  // memory cost a dense window about a quarter of its time) and, per stage, the stage itself plus the
  // plan-prefetch rings of its producer warp.
  const size_t base = 256 + (size_t)s.row_stride;
  const size_t per_stage = (size_t)s.stage_bytes + producer_scratch_bytes(tile);
  const bool table_smem = base + tbytes + 4 * per_stage <= budget;
  s.table_floats = table_smem ? tf : 0;
  const size_t fixed = base + (table_smem ? tbytes : 0);
  int stages = (int)((budget - fixed) / per_stage);
  if (stages > kMaxStages) stages = kMaxStages;
  s.stages = stages;
  s.groups = kMmaGroups;  // consumer warps = 4 per group; they all work on the same item
  s.smem = fixed + (size_t)(stages > 0 ? stages : 1) * per_stage;
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
  p.prod_warps = s.stages;
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

static int run_attn_mma_packs(AttnParams p, int dtype, int head_dim, const int32_t rpb_window[3], cudaStream_t stream);

// Padded plan, 16-bit inputs: packs and larger windows.  `p` arrives with the plan pointers,
// qkv/out/table, H, C, tile, scale, use_mask and rel_off filled in.
int run_attn_dense(const AttnParams& a, const int32_t* bins, const int32_t* win_start, const int32_t* win_pstart,
                   int n_per_window, int dtype, const int32_t rpb_window[3], cudaStream_t stream);
bool attn_dense_supported(int head_dim, int n_per_window, const int32_t rpb_window[3]);

int run_attn_mma(AttnParams p, int dtype, int head_dim, const int32_t rpb_window[3], const int32_t* bins,
                 const int32_t* win_start, const int32_t* win_pstart, int n_per_window, cudaStream_t stream) {
  // Windows beyond a pack: the tcgen05 kernel where it serves the shape (and the window size allows
  // such windows at all), else the second phase of this kernel.
  const bool dense = n_per_window > p.tile && attn_dense_supported(head_dim, n_per_window, rpb_window);
  p.skip_big = dense ? 1 : 0;
  const int st = run_attn_mma_packs(p, dtype, head_dim, rpb_window, stream);
  if (st != SSW_OK || !dense) return st;
  return run_attn_dense(p, bins, win_start, win_pstart, n_per_window, dtype, rpb_window, stream);
}

static int run_attn_mma_packs(AttnParams p, int dtype, int head_dim, const int32_t rpb_window[3], cudaStream_t stream) {
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
