// Fused window attention for windows that hold more voxels than one pack (c > tile), 16-bit inputs,
// head_dim 32: the dense contraction of the path, on the fifth-generation tensor cores (tcgen05,
// accumulators in tensor memory).
//
// Upstream computes such a window like every other: one thread per output element of the c x c
// score block and of the c x hd output block (ops.cu:344-418).  Here a unit of work is one
// (window, head).  Its k and v slices (c x 64 bytes each) are gathered once into shared memory in
// the tensor cores' operand layout and stay there while the window's query rows pass in tiles of
// 128:
//
//   S[128 x 64]  = Q_tile K_tile^T       tcgen05.mma, operands from shared memory, S in tensor memory
//   P            = exp2(S*scale + bias + mask - m)   one thread per query row (tcgen05.ld gives a
//                  thread its row of S), running maximum from 0 and +1e-8 as upstream (ops.cu:137,
//                  164); P goes back to shared memory in the input type.  bf16 keeps 8 bits of a
//                  probability, and a row that averages hundreds of keys loses more than the
//                  tolerance with that, so for bf16 the rounding residual is stored beside P and
//                  multiplied with the same V tile (A and B of an MMA must have the same 16-bit
//                  type: an fp16 P against a bf16 V is an illegal instruction)
//   O_part[128 x 32] = P V_tile          tcgen05.mma, added into fp32 registers by the row's thread
//                  with the correction factor of the running maximum
//
// Warp roles (384 threads, one CTA per SM): warp 0 issues the MMAs (one elected lane) and owns the
// tensor-memory allocation; warps 1-3 gather rows (plain 16-byte loads by voxel id, stored with the
// 64-byte swizzle the operand descriptors name); warps 4-11 are the softmax rows: a warp may touch
// the 32 tensor-memory lanes warp_id % 4 selects, so two warps share each quarter of the query
// rows, one for the first 32 keys of a tile and the first 16 output channels, one for the rest
// (they exchange their partial row maxima per tile and their row sums per query tile through shared
// memory): two warps per scheduler instead of one.  Everything is handed over through mbarriers
// with bounded waits; on expiry the kernel sets SSW_DEV_TIMEOUT, lets the tensor cores drain and
// frees its tensor memory before it returns.
#include <math.h>

#include "attn_common.cuh"

namespace ssw {

constexpr int kDQ = 128;       // query rows per tile = MMA M
constexpr int kDK = 64;        // keys per tile
constexpr int kDHD = 32;       // head_dim
constexpr int kDRowB = 64;     // bytes of one q / k / v head slice (32 x 16 bit)
constexpr int kDMaxKT = 16;    // key tiles per window at most (1024 keys)
constexpr int kDProd = 3;      // producer warps
constexpr int kDParts = 2;     // softmax threads per query row, in different warps (2 or 4; measured equal)
constexpr int kDSoftWarps = 4 * kDParts;
constexpr int kDThreads = 128 + 32 * kDSoftWarps;
constexpr int kDHalf = kDK / kDParts;  // keys of a tile one softmax thread looks after
constexpr int kDCpt = kDHD / kDParts;  // output channels one softmax thread accumulates
constexpr int kDOutPitch = kDRowB + 16;  // bytes between rows of the output staging tile (skewed across banks)
constexpr int kTmemCols = 256; // S: 2 x 64 columns, O_part: 2 x 32 columns
constexpr int kTmemS = 0, kTmemO = 128;

struct DenseParams {
  const void* qkv;
  OutSet outs;
  int32_t* header;
  const int32_t* bins;        // per-occupancy tables of the plan
  const int32_t* pack_win;
  const int32_t* win_start;
  const int32_t* win_pstart;
  const int32_t* pack_perm;
  const int32_t* pack_meta;
  const float* table;
  int rel_off, H, C, tile, n_per_window, table_rows;
  int n_vox, w_cap;
  int c_cap;                  // rows the shared-memory buffers are sized for (multiple of 64)
  float scale;
  int use_mask;
};

// ---- tcgen05 wrappers -----------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] (+)= A[smem] * B[smem], 128 x N x 16, 16-bit inputs, fp32 accumulation
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  const uint32_t zero = 0;  // no output lane is disabled
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(zero)
      : "memory");
}
// the mbarrier gets one arrival when every MMA issued by this thread so far has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
      "%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ldn(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
__device__ __forceinline__ void tmem_ldn(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_ldn(uint32_t taddr, uint32_t (&r)[8]) { tmem_ld8(taddr, r); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory operand descriptor (version 1): start address, leading / stride byte offsets in
// 16-byte units, swizzle mode (2 = 128-byte, 4 = 64-byte).  K-major tiles: rows of `swizzle` bytes,
// eight-row groups `sbo` bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t sbo_bytes, uint32_t layout_type) {
  uint64_t d = (uint64_t)((saddr >> 4) & 0x3fff);
  d |= (uint64_t)1 << 16;                              // leading byte offset: unused by swizzled layouts
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;    // stride byte offset
  d |= (uint64_t)1 << 46;                              // descriptor version
  d |= (uint64_t)layout_type << 61;
  return d;
}
// Instruction descriptor, kind::f16: fp32 accumulator, A/B formats (0 = f16, 1 = bf16), B major
// (0 = K, 1 = MN), N / 8 at bit 17, M / 16 at bit 24.
__device__ __forceinline__ uint32_t instr_desc(int a_fmt, int b_fmt, int b_mn_major, int n) {
  return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)b_mn_major << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kDQ >> 4) << 24);
}

// shared-memory accesses by 32-bit shared address (the softmax loop does one bias look-up per
// score: address arithmetic in 32 bits and loads that are certain to take the shared-memory path)
__device__ __forceinline__ float lds_f32(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ int4 lds_v4(uint32_t a) {
  int4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts_v4(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

__device__ __forceinline__ uint32_t f2h2(float a, float b) {  // two floats -> packed fp16 pair
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Shared memory (byte offsets from a 1024-byte aligned base):
//   [0, 1024)        mbarriers and the tensor-memory address
//   [1024, 1024 + 2 * kDParts * 512)  partial row maxima / sums the softmax threads of a row exchange
//   K  c_cap x 64    V  c_cap x 64    (64-byte swizzle; key tile j = rows [64 j, 64 j + 64))
//   Q  2 x 128 x 64  (64-byte swizzle)          P  128 x 128 (128-byte swizzle) twice: P and its bf16 residual
//   per unit (double buffered): the bias slice of its head, (2Wz-1)(2Wy-1)(2Wx-1) floats
//   pre-multiplied by log2 e; per row of its window the voxel id, 4 x relative-position code, region
struct DenseSmem {
  uint32_t k, v, q, p, bias, bias_floats, vox, rel4, reg, ostage, total;
};
__host__ __device__ inline DenseSmem dense_smem(int c_cap, int table_rows) {
  DenseSmem s;
  uint32_t o = 1024u + 2u * kDParts * 512u;
  s.k = o; o += (uint32_t)c_cap * kDRowB;
  s.v = o; o += (uint32_t)c_cap * kDRowB;
  s.q = o; o += 2u * kDQ * kDRowB;
  s.p = o; o += 2u * kDQ * 128u;
  s.bias_floats = ((uint32_t)table_rows + 3u) & ~3u;
  s.bias = o; o += 2u * s.bias_floats * 4u;
  s.vox = o; o += 2u * (uint32_t)c_cap * 4u;
  s.rel4 = o; o += 2u * (uint32_t)c_cap * 4u;
  s.reg = o; o += 2u * (uint32_t)c_cap * 4u;
  s.ostage = o; o += (uint32_t)kDQ * kDOutPitch;
  s.total = o;
  return s;
}

template <typename T, bool kMask>
__global__ void __launch_bounds__(kDThreads, 1) k_attn_dense(DenseParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // the operand layouts want 1024-byte aligned tiles: align the base by hand
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const DenseSmem L = dense_smem(p.c_cap, p.table_rows);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  uint64_t* kv_full = bars;                    // [kDMaxKT] key tile j of the unit is in shared memory
  uint64_t* kv_empty = bars + kDMaxKT;         // [kDMaxKT] the unit's last MMA on key tile j is done
  uint64_t* q_full = bars + 2 * kDMaxKT;       // [2]
  uint64_t* q_empty = q_full + 2;              // [2]
  uint64_t* s_full = q_empty + 2;              // [2] S tile in tensor memory
  uint64_t* s_empty = s_full + 2;              // [2] S tile read out
  uint64_t* p_full = s_empty + 2;              // [2] P tile in shared memory
  uint64_t* pv_done = p_full + 2;              // [2] P V of the tile done: O_part ready, P buffer free
  uint64_t* o_empty = pv_done + 2;             // [2] O_part read out
  uint64_t* meta_full = o_empty + 2;           // [2] a unit's header: voxel ids, metadata, bias slice of its head
  uint64_t* meta_empty = meta_full + 2;        // [2]
  uint64_t* drain_bar = meta_empty + 2;        // [1]
  uint64_t* xbar = drain_bar + 1;              // [4] the two warps of a row quarter have posted their partial values
  uint64_t* obar = xbar + 4;                   // [1] output staging tile: written by all / read by all
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(obar + 1);
  float* xch = reinterpret_cast<float*>(smem + 1024);  // [2 buffers][kDParts][128 rows] partial maxima / sums
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int H = p.H, C = p.C;

  // Whether there is any window beyond a pack is a device-side count: a launch that finds none
  // (the usual case on surface-sparse scenes) leaves before it sets anything up.
  grid_dependency_wait();
  {
    BinTables bins0(const_cast<int32_t*>(p.bins), p.n_per_window);
    const int W0 = min(max(p.header[SSW_H_W], 0), p.w_cap);
    const int first = p.tile + 1 <= p.n_per_window + 1 ? min(max(bins0.wstart[p.tile + 1], 0), W0) : W0;
    if (first >= W0) return;
  }
  if (threadIdx.x == 0) {
    for (int j = 0; j < kDMaxKT; ++j) {
      mbar_init(kv_full + j, kDProd);
      mbar_init(kv_empty + j, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(q_full + b, kDProd);
      mbar_init(q_empty + b, 1);
      mbar_init(s_full + b, 1);
      mbar_init(s_empty + b, kDSoftWarps);
      mbar_init(p_full + b, kDSoftWarps);
      mbar_init(pv_done + b, 1);
      mbar_init(o_empty + b, kDSoftWarps);
      mbar_init(meta_full + b, kDProd);
      mbar_init(meta_empty + b, kDSoftWarps);
    }
    for (int x = 0; x < 4; ++x) mbar_init(xbar + x, kDParts);
    mbar_init(obar, kDSoftWarps);
    mbar_init(drain_bar, 1);
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // the windows beyond a pack, heaviest first: window slots [ws0, W) of the plan's pack order
  BinTables bins(const_cast<int32_t*>(p.bins), p.n_per_window);
  const int W = min(max(p.header[SSW_H_W], 0), p.w_cap);
  const int ws0 = p.tile + 1 <= p.n_per_window + 1 ? min(max(bins.wstart[p.tile + 1], 0), W) : W;
  const int n_units = (W - ws0) * H;
  bool timed_out = false;
  // every role walks the same unit list; window geometry is read from the plan by each
  auto unit_window = [&](int u, int& first, int& c, int& h) {
    const int ws = W - 1 - u / H;
    h = u % H;
    const int k = min(max(__ldg(p.pack_win + ws), 0), p.w_cap - 1);
    first = __ldg(p.win_pstart + k);
    c = __ldg(p.win_start + k + 1) - __ldg(p.win_start + k);
    const bool ok = c > p.tile && c <= p.c_cap && first >= 0 && first <= p.n_vox - c;
    if (!ok) {
      atomicOr(reinterpret_cast<unsigned*>(p.header + SSW_H_ERROR), SSW_DEV_BAD_PLAN);
      first = 0;
      c = 0;
    }
  };
  const int a_fmt_qk = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr bool kSplitP = std::is_same<T, __nv_bfloat16>::value;

  if (warp == 0) {
    // =========================================== MMA issuer ===================================
    const uint32_t sK = smem_u32(smem + L.k), sV = smem_u32(smem + L.v), sQ = smem_u32(smem + L.q), sP = smem_u32(smem + L.p);
    uint32_t g = 0;          // key tiles issued so far (S / P / O_part buffer = g & 1)
    uint32_t qn = 0;         // query tiles so far (Q buffer = qn & 1)
    int un = 0;              // units so far
    for (int u = blockIdx.x; u < n_units && !timed_out; u += gridDim.x, ++un) {
      int first, c, h;
      unit_window(u, first, c, h);
      const int nkt = (c + kDK - 1) / kDK, nqt = (c + kDQ - 1) / kDQ;
      for (int t = 0; t < nqt && !timed_out; ++t, ++qn) {
        const uint32_t qb = qn & 1;
        if (!mbar_wait_bounded(q_full + qb, (qn >> 1) & 1)) { timed_out = true; break; }
        // software pipeline: S of tile j is issued before P V of tile j - 1, so the tensor cores
        // work on the next scores while the softmax rows are busy with the current ones
        for (int j = 0; j <= nkt && !timed_out; ++j) {
          if (j < nkt) {
            const uint32_t b = g & 1;
            const int nk16 = (min(kDK, c - j * kDK) + 15) & ~15;
            if (t == 0 && !mbar_wait_bounded(kv_full + j, un & 1)) { timed_out = true; break; }
            if (g >= 2 && !mbar_wait_bounded(s_empty + b, ((g >> 1) - 1) & 1)) { timed_out = true; break; }
            tc_fence_after();
            if (lane == 0) {
              const uint32_t idesc = instr_desc(a_fmt_qk, a_fmt_qk, 0, nk16);
#pragma unroll
              for (int ks = 0; ks < kDHD / 16; ++ks)
                umma_ss(tmem + kTmemS + b * kDK, smem_desc(sQ + qb * (kDQ * kDRowB) + ks * 32, 512, 4),
                        smem_desc(sK + j * (kDK * kDRowB) + ks * 32, 512, 4), idesc, ks > 0);
              umma_commit(s_full + b);
            }
            __syncwarp();
            ++g;
          }
          if (j > 0) {
            const uint32_t gp = g - (j < nkt ? 2 : 1);  // the tile whose P is multiplied now
            const uint32_t b = gp & 1;
            const int jp = j - 1;
            const int nk16 = (min(kDK, c - jp * kDK) + 15) & ~15;
            if (!mbar_wait_bounded(p_full + b, (gp >> 1) & 1)) { timed_out = true; break; }
            if (gp >= 2 && !mbar_wait_bounded(o_empty + b, ((gp >> 1) - 1) & 1)) { timed_out = true; break; }
            tc_fence_after();
            if (lane == 0) {
              const uint32_t idesc = instr_desc(a_fmt_qk, a_fmt_qk, 1, kDHD);  // A = P, B = V (MN-major)
              for (int part = 0; part < (kSplitP ? 2 : 1); ++part)   // P, then its rounding residual
                for (int ks = 0; ks < nk16 / 16; ++ks)
                  umma_ss(tmem + kTmemO + b * kDHD, smem_desc(sP + part * (kDQ * 128) + ks * 32, 1024, 2),
                          smem_desc(sV + jp * (kDK * kDRowB) + ks * (16 * kDRowB), 512, 4), idesc, (part | ks) > 0);
              umma_commit(pv_done + b);
              if (t == nqt - 1) umma_commit(kv_empty + jp);  // the window's last use of key tile jp
            }
            __syncwarp();
          }
        }
        if (lane == 0) umma_commit(q_empty + qb);  // every S of this query tile has been computed
        __syncwarp();
      }
      // Key tiles this window does not have: their barriers advance one phase per unit all the
      // same, so that a unit's number gives every barrier's phase whatever the windows' sizes.
      if (lane == 0)
        for (int j = nkt; j < kDMaxKT; ++j) umma_commit(kv_empty + j);
      __syncwarp();
    }
    // let the tensor cores finish whatever was issued before the tensor memory is given back
    if (lane == 0) umma_commit(drain_bar);
    __syncwarp();
    mbar_wait_bounded(drain_bar, 0);
  } else if (warp <= kDProd) {
    // =========================================== producers ====================================
    const int pw = warp - 1;
    const int chunk = lane & 3, rsub = lane >> 2;
    const T* qkv = reinterpret_cast<const T*>(p.qkv);
    // rows [r0, r0 + n_rows) of the window -> tile at `dst` (64-byte rows, 64-byte swizzle); rows
    // from `c` on are zero.  `part`: 0 q, 1 k, 2 v.  Row groups of eight are dealt to the warps.
    auto gather = [&](unsigned char* dst, const int* wvox, int r0, int n_rows, int c, int part, int h) {
      const int n_groups = (n_rows + 7) >> 3;
      for (int g0 = pw; g0 < n_groups; g0 += kDProd * 4) {
        uint4 val[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const int gi = g0 + x * kDProd, rl = gi * 8 + rsub, r = r0 + rl;
          val[x] = make_uint4(0, 0, 0, 0);
          if (gi < n_groups && rl < n_rows && r < c) {
            const int vx = wvox[r];
            val[x] = __ldg(reinterpret_cast<const uint4*>(qkv + (int64_t)vx * 3 * C + part * C + h * kDHD) + chunk);
          }
        }
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const int gi = g0 + x * kDProd, rl = gi * 8 + rsub;
          if (gi < n_groups && rl < n_rows)
            *reinterpret_cast<uint4*>(dst + (size_t)rl * kDRowB + ((chunk ^ ((rl >> 1) & 3)) << 4)) = val[x];
        }
      }
    };
    uint32_t qn = 0;
    int un = 0;
    for (int u = blockIdx.x; u < n_units && !timed_out; u += gridDim.x, ++un) {
      int first, c, h;
      unit_window(u, first, c, h);
      const int nkt = (c + kDK - 1) / kDK, nqt = (c + kDQ - 1) / kDQ;
      const int mb = un & 1;
      int* wvox = reinterpret_cast<int*>(smem + L.vox) + mb * p.c_cap;
      int* wrel4 = reinterpret_cast<int*>(smem + L.rel4) + mb * p.c_cap;
      int* wreg = reinterpret_cast<int*>(smem + L.reg) + mb * p.c_cap;
      // ---- the window's voxel ids and metadata
      if (un >= 2 && !mbar_wait_bounded(meta_empty + mb, ((un >> 1) - 1) & 1)) { timed_out = true; break; }
      for (int r = pw * 32 + lane; r < nkt * kDK; r += kDProd * 32) {  // (rows from c on: neutral entries)
        int vx = 0, m = 0;
        if (r < c) {
          vx = __ldg(p.pack_perm + first + r);
          m = __ldg(p.pack_meta + first + r);
        }
        const bool ok = (unsigned)vx < (unsigned)p.n_vox && meta_rel(m) <= p.rel_off;
        if (!ok) atomicOr(reinterpret_cast<unsigned*>(p.header + SSW_H_ERROR), SSW_DEV_BAD_PLAN);
        wvox[r] = ok ? vx : 0;
        wrel4[r] = ok ? meta_rel(m) * 4 : 0;
        wreg[r] = ok ? meta_region(m) : 0;
      }
      // ---- the head's bias slice (rows of the table are [code][head])
      {
        float* bs = reinterpret_cast<float*>(smem + L.bias) + (size_t)mb * L.bias_floats;
        for (int i = pw * 32 + lane; i < p.table_rows; i += kDProd * 32) bs[i] = __ldg(p.table + (int64_t)i * H + h) * kLog2e;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(meta_full + mb);
      // the other producer warps' ids are needed for the gathers below
      if (!mbar_wait_bounded(meta_full + mb, (un >> 1) & 1)) { timed_out = true; break; }
      // ---- key tiles (k and v), the first query tile in between so that the MMAs can start early
      for (int j = 0; j < nkt && !timed_out; ++j) {
        if (un >= 1 && !mbar_wait_bounded(kv_empty + j, (un - 1) & 1)) { timed_out = true; break; }
        const int n_rows = (min(kDK, c - j * kDK) + 15) & ~15;
        gather(smem + L.k + (size_t)j * kDK * kDRowB, wvox, j * kDK, n_rows, c, 1, h);
        gather(smem + L.v + (size_t)j * kDK * kDRowB, wvox, j * kDK, n_rows, c, 2, h);
        fence_async_smem();  // the tensor cores read shared memory through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(kv_full + j);
        if (j == 0 || j == nkt - 1) {
          // query tiles: the first right after key tile 0, the others once all keys are in
          const int t_lo = j == 0 ? 0 : 1, t_hi = j == 0 ? 1 : nqt;
          for (int t = (nkt == 1 ? 0 : t_lo); t < (nkt == 1 ? nqt : t_hi) && !timed_out; ++t) {
            const uint32_t qi = qn + t, qb = qi & 1;
            if (qi >= 2 && !mbar_wait_bounded(q_empty + qb, ((qi >> 1) - 1) & 1)) { timed_out = true; break; }
            gather(smem + L.q + (size_t)qb * kDQ * kDRowB, wvox, t * kDQ, kDQ, c, 0, h);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_full + qb);
          }
        }
      }
      // key tiles this window does not have (see the MMA warp)
      for (int j = nkt; j < kDMaxKT && !timed_out; ++j) {
        if (un >= 1 && !mbar_wait_bounded(kv_empty + j, (un - 1) & 1)) { timed_out = true; break; }
        if (lane == 0) mbar_arrive(kv_full + j);
      }
      qn += nqt;
    }
  } else {
    // =========================================== softmax rows =================================
    const int half = (warp - 4) >> 2;          // which part of a tile's keys / of the output channels (0 .. kDParts-1)
    const int sw = warp & 3;                   // tensor-memory lanes [32 sw, 32 sw + 32)
    const int row_in_tile = sw * 32 + lane;
    const uint32_t t_lane = (uint32_t)(sw * 32) << 16;
    const float qscale = p.scale * kLog2e;
    uint32_t g = 0;    // key tiles so far
    uint32_t xn = 0;   // exchanges with the partner warp so far
    int un = 0;
    // post a value for the other threads of the row (same row, other key parts) and combine theirs:
    // the maximum of the others' values, or their sum
    auto exchange = [&](float mine, float& theirs, bool take_max) -> bool {
      float* slot = xch + (xn & 1) * (kDParts * 128);
      slot[half * 128 + row_in_tile] = mine;
      __syncwarp();
      if (lane == 0) mbar_arrive(xbar + sw);
      const bool ok = mbar_wait_bounded(xbar + sw, xn & 1);
      float acc = take_max ? -INFINITY : 0.f;
#pragma unroll
      for (int o2 = 1; o2 < kDParts; ++o2) {
        const float v = slot[((half + o2) % kDParts) * 128 + row_in_tile];
        acc = take_max ? fmaxf(acc, v) : acc + v;
      }
      theirs = acc;
      ++xn;
      return ok;
    };
    uint32_t on = 0;  // query tiles this thread has put through the output staging tile
    for (int u = blockIdx.x; u < n_units && !timed_out; u += gridDim.x, ++un) {
      int first, c, h;
      unit_window(u, first, c, h);
      const int nkt = (c + kDK - 1) / kDK, nqt = (c + kDQ - 1) / kDQ;
      const int mb = un & 1;
      const int* wvox = reinterpret_cast<const int*>(smem + L.vox) + mb * p.c_cap;
      const int* wrel4 = reinterpret_cast<const int*>(smem + L.rel4) + mb * p.c_cap;
      const int* wreg = reinterpret_cast<const int*>(smem + L.reg) + mb * p.c_cap;
      const uint32_t bias_a = smem_u32(smem + L.bias) + (uint32_t)mb * L.bias_floats * 4u;
      const uint32_t rel4_a = smem_u32(wrel4) + half * kDHalf * 4, reg_a = smem_u32(wreg) + half * kDHalf * 4;
      if (!mbar_wait_bounded(meta_full + mb, (un >> 1) & 1)) { timed_out = true; break; }
      for (int t = 0; t < nqt && !timed_out; ++t) {
        const int qrow = t * kDQ + row_in_tile;
        const bool live = qrow < c;
        // bias of (me, key j) = slice[(code_me + rel_off) - code_j]: my row's base, minus 4 * code_j
        const uint32_t my_bias = bias_a + (uint32_t)(live ? wrel4[qrow] : 0) + (uint32_t)p.rel_off * 4u;
        const int my_region = live ? wreg[qrow] : 0;
        float m = 0.f, l = 0.f, corr_prev = 1.f;   // the maximum starts from 0 (ops.cu:137)
        float o[kDCpt];
#pragma unroll
        for (int e = 0; e < kDCpt; ++e) o[e] = 0.f;
        for (int j = 0; j <= nkt && !timed_out; ++j) {
          const uint32_t gp = g - 1, bp = gp & 1;
          if (j < nkt) {
            const uint32_t b = g & 1;
            const int nk = min(kDK, c - j * kDK) - half * kDHalf;  // valid keys among this thread's 32
            if (!mbar_wait_bounded(s_full + b, (g >> 1) & 1)) { timed_out = true; break; }
            tc_fence_after();
            uint32_t sr[kDHalf];
            tmem_ldn(tmem + t_lane + kTmemS + b * kDK + half * kDHalf, sr);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_empty + b);
            // scores in the log2 domain: bias from the head's slice, -100 across regions, -inf beyond c
            float s[kDHalf];
#pragma unroll
            for (int q4 = 0; q4 < kDHalf / 4; ++q4) {
              const int4 kr = lds_v4(rel4_a + (uint32_t)(j * kDK + q4 * 4) * 4u);
              const int krv[4] = {kr.x, kr.y, kr.z, kr.w};
              int kgv[4] = {0, 0, 0, 0};
              if constexpr (kMask) {
                const int4 kg = lds_v4(reg_a + (uint32_t)(j * kDK + q4 * 4) * 4u);
                kgv[0] = kg.x; kgv[1] = kg.y; kgv[2] = kg.z; kgv[3] = kg.w;
              }
#pragma unroll
              for (int x = 0; x < 4; ++x) {
                const int jj = q4 * 4 + x;
                float v = fmaf(__uint_as_float(sr[jj]), qscale, lds_f32(my_bias - (uint32_t)krv[x]));
                if (kMask && kgv[x] != my_region) v += -100.0f * kLog2e;
                s[jj] = v;
              }
            }
            if (nk < kDHalf) {  // the window's last key tile: nothing beyond its last voxel
#pragma unroll
              for (int jj = 0; jj < kDHalf; ++jj) s[jj] = jj < nk ? s[jj] : -INFINITY;
            }
            float mx;
            {  // four interleaved partial maxima keep the dependency chain short
              float m4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
              for (int jj = 4; jj < kDHalf; ++jj) m4[jj & 3] = fmaxf(m4[jj & 3], s[jj]);
              mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            }
            float mx_other;
            if (!exchange(mx, mx_other, true)) { timed_out = true; break; }
            const float m_new = fmaxf(m, fmaxf(mx, mx_other));
            const float corr = fast_exp2(m - m_new);
            m = m_new;
            // The one P buffer was last read by the P V of the tile before; the same completion says
            // that tile's O_part is in tensor memory.
            if (g >= 1 && !mbar_wait_bounded(pv_done + bp, (gp >> 1) & 1)) { timed_out = true; break; }
            const uint32_t prow = smem_u32(smem + L.p) + (uint32_t)row_in_tile * 128u;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};  // partial row sums, one per pair position
#pragma unroll
            for (int ch = 0; ch < kDHalf / 8; ++ch) {
              uint32_t hi[4], lo[4];
#pragma unroll
              for (int x = 0; x < 4; ++x) {
                const float p0 = fast_exp2(s[8 * ch + 2 * x] - m), p1 = fast_exp2(s[8 * ch + 2 * x + 1] - m);
                sum4[x] += p0 + p1;
                hi[x] = pack2<T>(p0, p1);
                if constexpr (kSplitP)
                  lo[x] = pack2<T>(p0 - __uint_as_float(hi[x] << 16), p1 - __uint_as_float(hi[x] & 0xffff0000u));
              }
              const int chg = half * (kDHalf / 8) + ch;  // 16-byte chunk of the tile's 128-byte row
              sts_v4(prow + ((chg ^ (row_in_tile & 7)) << 4), hi[0], hi[1], hi[2], hi[3]);
              if constexpr (kSplitP) sts_v4(prow + kDQ * 128 + ((chg ^ (row_in_tile & 7)) << 4), lo[0], lo[1], lo[2], lo[3]);
            }
            l = l * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + b);
            // fold the previous tile's O_part in with the factor its maximum update gave
            if (j > 0) {
              tc_fence_after();
              uint32_t orr[kDCpt];
              tmem_ldn(tmem + t_lane + kTmemO + bp * kDHD + half * kDCpt, orr);
              tmem_ld_wait();
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(o_empty + bp);
#pragma unroll
              for (int e = 0; e < kDCpt; ++e) o[e] = fmaf(o[e], corr_prev, __uint_as_float(orr[e]));
            }
            corr_prev = corr;
            ++g;
          } else {
            if (!mbar_wait_bounded(pv_done + bp, (gp >> 1) & 1)) { timed_out = true; break; }
            tc_fence_after();
            uint32_t orr[kDCpt];
            tmem_ldn(tmem + t_lane + kTmemO + bp * kDHD + half * kDCpt, orr);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_empty + bp);
#pragma unroll
            for (int e = 0; e < kDCpt; ++e) o[e] = fmaf(o[e], corr_prev, __uint_as_float(orr[e]));
          }
        }
        // the row's sum is the two halves' sums (both were kept relative to the same running maximum)
        float l_other = 0.f;
        if (!timed_out && !exchange(l, l_other, false)) timed_out = true;
        // The tile's output goes out through a staging tile in shared memory, so that the four lanes
        // that write one row's 64-byte head slice sit side by side in one store instruction (a thread
        // owns only half a slice, and its partner is in another warp).  Whole 64-byte segments matter
        // for the destinations on peer GPUs, where every store instruction's segments cross NVLink as
        // packets of their own.  The staging tile is guarded by one barrier of the eight softmax warps
        // with two phases per query tile: all have written / all have read.
        if (timed_out) break;
        if (on > 0 && !mbar_wait_bounded(obar, 1)) { timed_out = true; break; }
        if (live) {
          const float inv = __frcp_rn(l + l_other + 1e-8f);  // ops.cu:164
          const uint32_t dst = smem_u32(smem + L.ostage) + (uint32_t)row_in_tile * kDOutPitch + (uint32_t)half * (kDRowB / kDParts);
#pragma unroll
          for (int e = 0; e < kDCpt / 8; ++e) {
            uint32_t ww[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) ww[x] = pack2<T>(o[8 * e + 2 * x] * inv, o[8 * e + 2 * x + 1] * inv);
            sts_v4(dst + 16u * e, ww[0], ww[1], ww[2], ww[3]);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(obar);
        if (!mbar_wait_bounded(obar, 0)) { timed_out = true; break; }
#pragma unroll
        for (int k2 = 0; k2 < (kDQ * kDRowB / 16) / (32 * kDSoftWarps); ++k2) {
          const int id = (int)threadIdx.x - 128 + 32 * kDSoftWarps * k2;  // softmax threads are threads 128 and up
          const int orow = id >> 2, piece = id & 3;
          if (t * kDQ + orow < c) {
            const int4 w = lds_v4(smem_u32(smem + L.ostage) + (uint32_t)orow * kDOutPitch + 16u * piece);
            const int64_t off = (int64_t)wvox[t * kDQ + orow] * C + h * kDHD + piece * 8;
            for (int d = 0; d < p.outs.n; ++d)
              *reinterpret_cast<int4*>(reinterpret_cast<T*>(p.outs.base[d]) + off) = w;
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(obar);
        ++on;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(meta_empty + mb);
    }
  }
  if (timed_out) atomicOr(reinterpret_cast<unsigned*>(p.header + SSW_H_ERROR), SSW_DEV_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

int run_attn_dense(const AttnParams& a, const int32_t* bins, const int32_t* win_start, const int32_t* win_pstart,
                   int n_per_window, int dtype, const int32_t rpb_window[3], cudaStream_t stream) {
  DenseParams p = {};
  p.qkv = a.qkv;
  p.outs = a.outs;
  p.header = a.header;
  p.bins = bins;
  p.pack_win = a.pack_win;
  p.win_start = win_start;
  p.win_pstart = win_pstart;
  p.pack_perm = a.pack_perm;
  p.pack_meta = a.pack_meta;
  p.table = a.table;
  p.rel_off = a.rel_off;
  p.H = a.H;
  p.C = a.C;
  p.tile = a.tile;
  p.n_per_window = n_per_window;
  p.table_rows = (2 * rpb_window[0] - 1) * (2 * rpb_window[1] - 1) * (2 * rpb_window[2] - 1);
  p.n_vox = a.n_vox;
  p.w_cap = a.w_cap;
  p.c_cap = (n_per_window + kDK - 1) / kDK * kDK;
  p.scale = a.scale;
  p.use_mask = a.use_mask;
  if (p.c_cap > kDMaxKT * kDK) return SSW_E_UNSUPPORTED;
  const DenseSmem L = dense_smem(p.c_cap, p.table_rows);
  const size_t smem = (size_t)L.total + 1024;  // slack for the 1024-byte alignment of the base
  if (smem > 227 * 1024) return SSW_E_UNSUPPORTED;
  int dev = 0, sms = 0;
  SSW_CUDA_TRY(cudaGetDevice(&dev));
  SSW_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  void (*kern)(DenseParams) =
      dtype == SSW_BF16 ? (p.use_mask ? k_attn_dense<__nv_bfloat16, true> : k_attn_dense<__nv_bfloat16, false>)
                        : (p.use_mask ? k_attn_dense<__half, true> : k_attn_dense<__half, false>);
  SSW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  SSW_CUDA_TRY(launch_chained(kern, dim3(sms), dim3(kDThreads), smem, stream, p));
  SSW_LAUNCH_CHECK("k_attn_dense");
  return SSW_OK;
}

// Whether run_attn_dense serves this configuration (otherwise the windows beyond a pack stay with
// the second phase of the mma.sync kernel).
bool attn_dense_supported(int head_dim, int n_per_window, const int32_t rpb_window[3]) {
  if (head_dim != kDHD) return false;
  const int c_cap = (n_per_window + kDK - 1) / kDK * kDK;
  if (c_cap > kDMaxKT * kDK) return false;
  const int rows = (2 * rpb_window[0] - 1) * (2 * rpb_window[1] - 1) * (2 * rpb_window[2] - 1);
  return (size_t)dense_smem(c_cap, rows).total + 1024 <= 227 * 1024;
}

}  // namespace ssw
