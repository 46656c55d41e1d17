// Fused window attention for 16-bit inputs (bf16 / fp16) on tensor cores.
//
// Same persistent producer/consumer pipeline as the CUDA-core kernel (one CTA per SM, one producer
// warp that gathers whole q|k|v rows with one 1-D bulk (TMA) copy per voxel, `full`/`empty`
// mbarriers), but the rows stay 16-bit in shared memory and the
// arithmetic is warp-level MMA (m16n8k16, fp32 accumulation):
//
//   * The plan is *padded*: inside a pack every window gets a run of row slots rounded up to
//     1, 2, 4, 8, 16, 32, 48 or 64, so a 16-slot MMA tile holds whole windows (several when c < 16)
//     or a 16-row slice of one window.  Unused slots keep stale (finite) data; their keys are
//     masked out, their query rows are never stored.
//   * A warp takes (16-slot tile, up to three heads) units and interleaves the heads.  Q comes in as A fragments (ldmatrix), K as B
//     fragments (ldmatrix), S = Q K^T lands in fp32 accumulators whose layout is also the A layout
//     of the next MMA, so P = softmax(S) is packed to 16 bit in registers and multiplied with V
//     (ldmatrix.trans).  Windows longer than 16 loop over 16-key blocks with an online softmax.
//   * Softmax keeps upstream's semantics: the running maximum starts at 0, the denominator gets
//     +1e-8; bias from the shared-memory table (pre-multiplied by log2 e), -100 shift mask.
//   * The output tile overwrites the q slice it came from; the warp then copies it out with
//     coalesced 16-byte stores.
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

// Layout of a staged row's metadata word .y: region (5 bits), window inside the pack (7 bits: 0..63,
// kMmaPadWindow for unused slots), row of the bias table (from bit 12).
constexpr int kMmaRelShift = 12;
constexpr int kMmaPadWindow = 64;
constexpr int kMmaWindowBits = 127 << 5;

template <typename T, int HD, int HU, bool kTableSmem>
__global__ void __launch_bounds__(kMmaGroupWarps * 32 * (HU == 3 ? 3 : kMaxGroups) + 32 * kMaxProducerWarps, 1) k_attn_mma(AttnParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int tile = p.tile, C = p.C, H = p.H;
  const int S = p.stages, G = p.groups;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + kMaxStages;
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
      mbar_init(full + s, p.prod_warps);       // one arrive (with its byte count) per producer warp
      mbar_init(empty + s, kMmaGroupWarps);  // every warp of the consuming group hands the stage back
    }
    mbar_fence_init();
  }
  // unused row slots are read as keys/values (and masked): they must hold finite numbers
  for (int i = threadIdx.x; i < (S * p.stage_bytes) / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(stage0)[i] = make_uint4(0, 0, 0, 0);
  fence_async_smem();  // order the zero fill before the bulk copies that will land in the same rows
  grid_dependency_wait();
  if constexpr (kTableSmem) stage_table(table_s, p.table, p.table_floats);
  const int n_small = p.header[SSW_H_PACKS_SMALL];
  __syncthreads();

  const int my_items = n_small > (int)blockIdx.x ? (n_small - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  bool timed_out = false;
  if (is_producer) {
    // slot -> row of the pack: window wl = slot / cpad, i = slot % cpad, valid if wl < nwin && i < c.
    // Register pipeline, three items deep: the descriptor of item i+5 and the voxel ids / metadata
    // of item i+3 (whose descriptor arrived an iteration ago) are requested while item i is issued,
    // so no iteration waits on a global load.
    // The rows of an item are dealt round-robin to the producer warps: a warp submits its bulk
    // copies one lane after the other, so several warps submit several rows at a time.
    constexpr int kAhead = 3;
    const int PW = p.prod_warps, pw = ((int)threadIdx.x - n_cons) >> 5;
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
    for (int a = 0; a < kAhead; ++a) fetch(dq[a], vox[a], km[a]);
    for (int i = 0; i < my_items; ++i) {
      const int s = i % S;
      const int use = i / S;
      const int4 d_new = i + kAhead + 2 < my_items
                             ? __ldg(p.pack_desc + item_index(i + kAhead + 2))
                             : make_int4(0, 0, 0, 0);
      int vox_n[2], km_n[2];
      fetch(dq[kAhead], vox_n, km_n);  // item i + kAhead (an all-zero descriptor fetches nothing)
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
          reinterpret_cast<int*>(st + kMmaStageVoxOff)[slot] = vox[0][k];
          // Row metadata: .x = byte offset of the row's relative-position code in the bias table,
          // .y = region | window-in-pack << 5 | table row << 12.  Unused slots form a window of their
          // own (kMmaPadWindow) with neutral codes, so their (discarded) scores index inside the table.
          *reinterpret_cast<int2*>(st + kMmaStageRowsOff + (size_t)slot * p.row_stride + data_bytes) =
              vox[0][k] >= 0 ? make_int2(meta_rel(km[0][k]) * H * 4,
                                         meta_region(km[0][k]) | ((km[0][k] & 1023) << 5) |
                                             ((meta_rel(km[0][k]) + p.rel_off) << kMmaRelShift))
                             : make_int2(0, (kMmaPadWindow << 5) | (p.rel_off << kMmaRelShift));
        }
      }
      const int my_rows = __popc(__ballot_sync(0xffffffffu, vox[0][0] >= 0)) + __popc(__ballot_sync(0xffffffffu, vox[0][1] >= 0));
      if (lane == 0) mbar_expect_tx(full + s, (uint32_t)my_rows * (uint32_t)data_bytes);
      __syncwarp();
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int slot = (lane + 32 * k) * PW + pw;
        if (slot < tile && vox[0][k] >= 0)
          bulk_g2s(st + kMmaStageRowsOff + (size_t)slot * p.row_stride,
                   reinterpret_cast<const T*>(p.qkv) + (int64_t)vox[0][k] * 3 * C, data_bytes, full + s);
      }
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
      // A unit is (16-slot tile, HU consecutive heads); the HU heads are independent instruction
      // streams that the unrolled code interleaves, which hides the ldmatrix / MMA / exp latencies.
      const int n_hg = H / HU;
      for (int u = wg; u < n_mt * n_hg; u += kMmaGroupWarps) {
        const int mt = u / n_hg, h0 = (u - mt * n_hg) * HU;
        const int slot_lo = mt * 16 + qr, slot_hi = slot_lo + 8;
        // first key slot of the window(s) this tile belongs to
        const int kbase = cpad > 16 ? (mt * 16 / cpad) * cpad : mt * 16;
        const int2 me_lo = *reinterpret_cast<const int2*>(rows + (size_t)slot_lo * p.row_stride + data_bytes);
        const int2 me_hi = *reinterpret_cast<const int2*>(rows + (size_t)slot_hi * p.row_stride + data_bytes);
        const unsigned char* tab_lo =
            reinterpret_cast<const unsigned char*>(table_base + (me_lo.y >> kMmaRelShift) * H + h0);
        const unsigned char* tab_hi =
            reinterpret_cast<const unsigned char*>(table_base + (me_hi.y >> kMmaRelShift) * H + h0);
        const int mi = lane >> 3;
        const int region_bits = p.use_mask ? 31 : 0;

        uint32_t qf[HU][HD / 16][4];
        float o[HU][HD / 8][4];
        float m_lo[HU], m_hi[HU], l_lo[HU], l_hi[HU];
#pragma unroll
        for (int x = 0; x < HU; ++x) {
          const unsigned char* qp = rows + (size_t)(mt * 16 + (mi & 1) * 8 + (lane & 7)) * p.row_stride +
                                    ((h0 + x) * HD + (mi >> 1) * 8) * sizeof(T);
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) ldmatrix_x4(qf[x][ks], qp + ks * 16 * sizeof(T));
#pragma unroll
          for (int n = 0; n < HD / 8; ++n) o[x][n][0] = o[x][n][1] = o[x][n][2] = o[x][n][3] = 0.f;
          m_lo[x] = m_hi[x] = 0.f;  // maximum starts from 0 (ops.cu:137)
          l_lo[x] = l_hi[x] = 0.f;
        }

        for (int kb = 0; kb < nkb; ++kb) {
          const int ks0 = kbase + kb * 16;  // first key slot of this block
          float sacc[HU][2][4];
#pragma unroll
          for (int x = 0; x < HU; ++x) {
#pragma unroll
            for (int n = 0; n < 2; ++n) sacc[x][n][0] = sacc[x][n][1] = sacc[x][n][2] = sacc[x][n][3] = 0.f;
            const unsigned char* kp = rows + (size_t)(ks0 + (mi >> 1) * 8 + (lane & 7)) * p.row_stride +
                                      (C + (h0 + x) * HD + (mi & 1) * 8) * sizeof(T);
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
              uint32_t kf[4];
              ldmatrix_x4(kf, kp + ks * 16 * sizeof(T));
              mma16816<T>(sacc[x][0], qf[x][ks], kf[0], kf[1]);
              mma16816<T>(sacc[x][1], qf[x][ks], kf[2], kf[3]);
            }
          }
          // scores -> log2 domain, bias, masks (key metadata is shared by the HU heads)
          float mx_lo[HU], mx_hi[HU];
#pragma unroll
          for (int x = 0; x < HU; ++x) mx_lo[x] = mx_hi[x] = -INFINITY;
#pragma unroll
          for (int n = 0; n < 2; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int ks = ks0 + n * 8 + qt * 2 + e;  // key slot of this column
              const int2 km = *reinterpret_cast<const int2*>(rows + (size_t)ks * p.row_stride + data_bytes);
              // one XOR per (query row, key) tells both: same window (bits 5..11), same region (bits 0..4)
              const int x_lo = km.y ^ me_lo.y, x_hi = km.y ^ me_hi.y;
              const bool ok_lo = (x_lo & kMmaWindowBits) == 0, ok_hi = (x_hi & kMmaWindowBits) == 0;
              const float madd_lo = (x_lo & region_bits) ? -100.0f * kLog2e : 0.f;
              const float madd_hi = (x_hi & region_bits) ? -100.0f * kLog2e : 0.f;
#pragma unroll
              for (int x = 0; x < HU; ++x) {
                const float b_lo = kTableSmem ? *reinterpret_cast<const float*>(tab_lo - km.x + x * 4)
                                              : __ldg(reinterpret_cast<const float*>(tab_lo - km.x + x * 4)) * kLog2e;
                const float b_hi = kTableSmem ? *reinterpret_cast<const float*>(tab_hi - km.x + x * 4)
                                              : __ldg(reinterpret_cast<const float*>(tab_hi - km.x + x * 4)) * kLog2e;
                float s_lo = fmaf(sacc[x][n][e], qscale, b_lo) + madd_lo;
                float s_hi = fmaf(sacc[x][n][2 + e], qscale, b_hi) + madd_hi;
                s_lo = ok_lo ? s_lo : -INFINITY;
                s_hi = ok_hi ? s_hi : -INFINITY;
                sacc[x][n][e] = s_lo;
                sacc[x][n][2 + e] = s_hi;
                mx_lo[x] = fmaxf(mx_lo[x], s_lo);
                mx_hi[x] = fmaxf(mx_hi[x], s_hi);
              }
            }
          }
          uint32_t pf[HU][4];
#pragma unroll
          for (int x = 0; x < HU; ++x) {
            mx_lo[x] = fmaxf(mx_lo[x], __shfl_xor_sync(0xffffffffu, mx_lo[x], 1));
            mx_lo[x] = fmaxf(mx_lo[x], __shfl_xor_sync(0xffffffffu, mx_lo[x], 2));
            mx_hi[x] = fmaxf(mx_hi[x], __shfl_xor_sync(0xffffffffu, mx_hi[x], 1));
            mx_hi[x] = fmaxf(mx_hi[x], __shfl_xor_sync(0xffffffffu, mx_hi[x], 2));
            if (mx_lo[x] > m_lo[x]) {
              const float corr = fast_exp2(m_lo[x] - mx_lo[x]);
              l_lo[x] *= corr;
#pragma unroll
              for (int n = 0; n < HD / 8; ++n) { o[x][n][0] *= corr; o[x][n][1] *= corr; }
              m_lo[x] = mx_lo[x];
            }
            if (mx_hi[x] > m_hi[x]) {
              const float corr = fast_exp2(m_hi[x] - mx_hi[x]);
              l_hi[x] *= corr;
#pragma unroll
              for (int n = 0; n < HD / 8; ++n) { o[x][n][2] *= corr; o[x][n][3] *= corr; }
              m_hi[x] = mx_hi[x];
            }
            // P in the A-fragment layout of the next MMA
            const float p00 = fast_exp2(sacc[x][0][0] - m_lo[x]), p01 = fast_exp2(sacc[x][0][1] - m_lo[x]);
            const float p02 = fast_exp2(sacc[x][0][2] - m_hi[x]), p03 = fast_exp2(sacc[x][0][3] - m_hi[x]);
            const float p10 = fast_exp2(sacc[x][1][0] - m_lo[x]), p11 = fast_exp2(sacc[x][1][1] - m_lo[x]);
            const float p12 = fast_exp2(sacc[x][1][2] - m_hi[x]), p13 = fast_exp2(sacc[x][1][3] - m_hi[x]);
            l_lo[x] += (p00 + p01) + (p10 + p11);
            l_hi[x] += (p02 + p03) + (p12 + p13);
            pf[x][0] = pack2<T>(p00, p01);
            pf[x][1] = pack2<T>(p02, p03);
            pf[x][2] = pack2<T>(p10, p11);
            pf[x][3] = pack2<T>(p12, p13);
          }
#pragma unroll
          for (int x = 0; x < HU; ++x) {
            const unsigned char* vp = rows + (size_t)(ks0 + (mi & 1) * 8 + (lane & 7)) * p.row_stride +
                                      (2 * C + (h0 + x) * HD + (mi >> 1) * 8) * sizeof(T);
#pragma unroll
            for (int n = 0; n < HD / 8; n += 2) {
              uint32_t vf[4];
              ldmatrix_x4_trans(vf, vp + n * 8 * sizeof(T));
              mma16816<T>(o[x][n], pf[x], vf[0], vf[1]);
              mma16816<T>(o[x][n + 1], pf[x], vf[2], vf[3]);
            }
          }
        }
        __syncwarp();
#pragma unroll
        for (int x = 0; x < HU; ++x) {
          // row sums live in four lanes each
          float ll = l_lo[x], lh = l_hi[x];
          ll += __shfl_xor_sync(0xffffffffu, ll, 1);
          ll += __shfl_xor_sync(0xffffffffu, ll, 2);
          lh += __shfl_xor_sync(0xffffffffu, lh, 1);
          lh += __shfl_xor_sync(0xffffffffu, lh, 2);
          const float inv_lo = 1.0f / (ll + 1e-8f), inv_hi = 1.0f / (lh + 1e-8f);  // ops.cu:164
          // the q slice this tile was read from becomes its output slice
          uint32_t* out_lo =
              reinterpret_cast<uint32_t*>(rows + (size_t)slot_lo * p.row_stride + ((h0 + x) * HD) * sizeof(T)) + qt;
          uint32_t* out_hi =
              reinterpret_cast<uint32_t*>(rows + (size_t)slot_hi * p.row_stride + ((h0 + x) * HD) * sizeof(T)) + qt;
#pragma unroll
          for (int n = 0; n < HD / 8; ++n) {
            out_lo[n * 4] = pack2<T>(o[x][n][0] * inv_lo, o[x][n][1] * inv_lo);
            out_hi[n * 4] = pack2<T>(o[x][n][2] * inv_hi, o[x][n][3] * inv_hi);
          }
        }
        // The tile's 16 x (HU*HD) outputs now sit in shared memory in row order: copy them out with
        // 16-byte stores, a run of HU*HD elements per voxel row (bulk stores of whole rows were
        // tried; one bulk operation per row is what bounds them).
        __syncwarp();
        {
          constexpr int kChunks = HU * HD / 8;  // 16-byte chunks per row segment
          const int* svox = reinterpret_cast<const int*>(sp + kMmaStageVoxOff);
          for (int idx = lane; idx < 16 * kChunks; idx += 32) {
            const int rr = idx / kChunks, cc = idx - rr * kChunks;
            const int slot = mt * 16 + rr;
            const int v = svox[slot];
            if (v >= 0)
              *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.out) + (int64_t)v * C + h0 * HD + cc * 8) =
                  *reinterpret_cast<const uint4*>(rows + (size_t)slot * p.row_stride + (h0 * HD + cc * 8) * sizeof(T));
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty + s);
    }
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

template <typename T, int HD, int HU>
static int launch_mma(AttnParams p, const MmaShape& s, cudaStream_t stream) {
  int dev = 0, sms = 0;
  SSW_CUDA_TRY(cudaGetDevice(&dev));
  SSW_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (HU == 3 && p.groups > 3) p.groups = 3;  // three interleaved heads need the larger register budget
  p.prod_warps = 4;  // 576-byte rows: the copy submission rate, not the bytes, bounds the producer
  if (const char* e = getenv("SSW_PROD_WARPS")) {  // tuning override (experiments only)
    const int v = atoi(e);
    if (v >= 1 && v <= kMaxProducerWarps) p.prod_warps = v;
  }
  const int threads = p.groups * kMmaGroupWarps * 32 + 32 * p.prod_warps;
  if (s.table_floats > 0) {
    auto kern = k_attn_mma<T, HD, HU, true>;
    SSW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s.smem));
    SSW_CUDA_TRY(launch_chained(kern, dim3(sms), dim3(threads), s.smem, stream, p));
  } else {
    auto kern = k_attn_mma<T, HD, HU, false>;
    SSW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s.smem));
    SSW_CUDA_TRY(launch_chained(kern, dim3(sms), dim3(threads), s.smem, stream, p));
  }
  return SSW_OK;
}

// One head per consumer unit: interleaving two or three heads in a unit was measured slower (more
// registers, fewer units to spread over the warps of a group).
template <typename T, int HD>
static int launch_mma_heads(const AttnParams& p, const MmaShape& s, cudaStream_t stream) {
  return launch_mma<T, HD, 1>(p, s, stream);
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
    if (head_dim == 16) return launch_mma_heads<__nv_bfloat16, 16>(p, s, stream);
    if (head_dim == 32) return launch_mma_heads<__nv_bfloat16, 32>(p, s, stream);
  } else if (dtype == SSW_F16) {
    if (head_dim == 16) return launch_mma_heads<__half, 16>(p, s, stream);
    if (head_dim == 32) return launch_mma_heads<__half, 32>(p, s, stream);
  }
  return SSW_E_UNSUPPORTED;
}

}  // namespace ssw
