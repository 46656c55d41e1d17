// Window bucketing: a device-side int32 counting sort of voxels by (window, pos), the segment
// offsets of every non-empty window, and the work list of the fused attention kernel grouped
// by window occupancy.  No key wider than 32 bits is ever formed and the host never waits for
// a device value.
//
// Pipeline (all on the caller's stream):
//   zero scratch + header + bin tables
//   k_count    : per voxel, count[w]++ and set bit `pos` of window w's occupancy bitmap
//   k_reduce   : per 2048-window block, totals of (non-empty, c, c^2); last block scans them
//   k_compact  : exclusive scan -> compact window list, row starts, c^2 starts, histogram of c;
//                last block turns the histogram into per-occupancy starts and the item count
//   k_order    : window -> slot inside its occupancy bin; work-item descriptors
//   k_scatter  : per voxel, rank inside its window = popcount of lower bitmap bits -> perm,
//                inverse perm, pack-order perm and per-row metadata
#include <stdio.h>

#include "ssw_common.cuh"

namespace ssw {

struct KeySrc {
  const int32_t* coords;   // [N,4] or null
  const int32_t* indices;  // [N,2] or null
  const int8_t* mask;      // [mask_windows, n_per_window] or null
  int mask_windows;
  int batch, shifted;
  int dims[3], dims_p[3], ws[3], ss[3], nwin[3];
  int n_per_window, n_windows;
  int rpbw[3];
  int win_lo, win_hi;      // only voxels of windows [win_lo, win_hi) are bucketed
};

// (window, pos, region) of voxel v; false when the row is outside the grid / tables.
__device__ __forceinline__ bool load_key(const KeySrc& s, int64_t v, int& w, int& pos, int& region) {
  region = 0;
  if (s.coords) {
    int4 c = __ldg(reinterpret_cast<const int4*>(s.coords) + v);
    int b = c.x, z = c.y, y = c.z, x = c.w;
    if ((unsigned)b >= (unsigned)s.batch || (unsigned)z >= (unsigned)s.dims[0] ||
        (unsigned)y >= (unsigned)s.dims[1] || (unsigned)x >= (unsigned)s.dims[2])
      return false;
    if (s.shifted) {
      z -= s.ss[0]; if (z < 0) z += s.dims_p[0];
      y -= s.ss[1]; if (y < 0) y += s.dims_p[1];
      x -= s.ss[2]; if (x < 0) x += s.dims_p[2];
      int rz = s.ss[0] == 0 ? 2 : (z >= s.dims_p[0] - s.ws[0]) + (z >= s.dims_p[0] - s.ss[0]);
      int ry = s.ss[1] == 0 ? 2 : (y >= s.dims_p[1] - s.ws[1]) + (y >= s.dims_p[1] - s.ss[1]);
      int rx = s.ss[2] == 0 ? 2 : (x >= s.dims_p[2] - s.ws[2]) + (x >= s.dims_p[2] - s.ss[2]);
      region = 9 * rz + 3 * ry + rx;
    }
    int wz = z / s.ws[0], wy = y / s.ws[1], wx = x / s.ws[2];
    w = ((b * s.nwin[0] + wz) * s.nwin[1] + wy) * s.nwin[2] + wx;
    pos = ((z - wz * s.ws[0]) * s.ws[1] + (y - wy * s.ws[1])) * s.ws[2] + (x - wx * s.ws[2]);
    return true;
  }
  int2 k = __ldg(reinterpret_cast<const int2*>(s.indices) + v);
  w = k.x;
  pos = k.y;
  if ((unsigned)w >= (unsigned)s.n_windows || (unsigned)pos >= (unsigned)s.n_per_window) return false;
  if (s.mask) region = __ldg(s.mask + (int64_t)(w % s.mask_windows) * s.n_per_window + pos) & 31;
  return true;
}

__global__ void k_window_keys(KeySrc s, int64_t n, int32_t* __restrict__ indices, int8_t* __restrict__ region,
                              int32_t* __restrict__ dev_error) {
  int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= n) return;
  int w, pos, r;
  bool ok = load_key(s, v, w, pos, r);
  if (!ok) {
    if (dev_error) atomicOr(reinterpret_cast<unsigned*>(dev_error), SSW_DEV_BAD_COORD);
    w = 0; pos = 0; r = 0;
  }
  reinterpret_cast<int2*>(indices)[v] = make_int2(w, pos);
  if (region) region[v] = (int8_t)r;
}

__global__ void k_count(KeySrc s, int64_t n, int words, int32_t* __restrict__ count, uint32_t* __restrict__ bitmap,
                        int32_t* __restrict__ header) {
  grid_dependency_wait();
  int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= n) return;
  int w, pos, r;
  if (!load_key(s, v, w, pos, r)) {
    atomicOr(reinterpret_cast<unsigned*>(header + SSW_H_ERROR), SSW_DEV_BAD_COORD);
    return;
  }
  if (w < s.win_lo || w >= s.win_hi) return;  // another shard's window
  uint32_t bit = 1u << (pos & 31);
  uint32_t old = atomicOr(bitmap + (int64_t)w * words + (pos >> 5), bit);
  if (old & bit) {
    atomicOr(reinterpret_cast<unsigned*>(header + SSW_H_ERROR), SSW_DEV_DUPLICATE);
    return;
  }
  atomicAdd(count + w, 1);
}

constexpr int kScanThreads = 256;
constexpr int kScanItems = 8;
constexpr int kScanBlock = kScanThreads * kScanItems;

struct Tri {
  int flags;
  int rows;
  unsigned long long sq;
};
__device__ __forceinline__ Tri tri_add(Tri a, Tri b) { return Tri{a.flags + b.flags, a.rows + b.rows, a.sq + b.sq}; }

// Block-wide exclusive scan of one Tri per thread (256 threads); returns the exclusive prefix,
// `total` gets the block total.
__device__ Tri block_excl_scan(Tri v, Tri& total) {
  __shared__ Tri warp_tot[kScanThreads / 32];
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  Tri inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int f = __shfl_up_sync(0xffffffffu, inc.flags, o);
    int r = __shfl_up_sync(0xffffffffu, inc.rows, o);
    unsigned long long q = __shfl_up_sync(0xffffffffu, inc.sq, o);
    if (lane >= o) { inc.flags += f; inc.rows += r; inc.sq += q; }
  }
  if (lane == 31) warp_tot[wid] = inc;
  __syncthreads();
  Tri base{0, 0, 0ull};
  Tri tot{0, 0, 0ull};
#pragma unroll
  for (int i = 0; i < kScanThreads / 32; ++i) {
    if (i < wid) base = tri_add(base, warp_tot[i]);
    tot = tri_add(tot, warp_tot[i]);
  }
  total = tot;
  __syncthreads();
  return Tri{base.flags + inc.flags - v.flags, base.rows + inc.rows - v.rows, base.sq + inc.sq - v.sq};
}

// partials: 4 ints per block {flags, rows, sq_lo, sq_hi}; after the last block's pass they hold
// the exclusive prefix over blocks.
__global__ void __launch_bounds__(kScanThreads) k_reduce(const int32_t* __restrict__ count, int n_windows,
                                                         int32_t* __restrict__ partials, int32_t* __restrict__ header,
                                                         int n_blocks) {
  grid_dependency_wait();
  int base = blockIdx.x * kScanBlock + threadIdx.x * kScanItems;
  Tri t{0, 0, 0ull};
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    int w = base + i;
    int c = w < n_windows ? count[w] : 0;
    t.flags += c > 0;
    t.rows += c;
    t.sq += (unsigned long long)c * (unsigned long long)c;
  }
  Tri tot;
  block_excl_scan(t, tot);
  __shared__ bool last;
  if (threadIdx.x == 0) {
    int4 p = make_int4(tot.flags, tot.rows, (int)(tot.sq & 0xffffffffull), (int)(tot.sq >> 32));
    reinterpret_cast<int4*>(partials)[blockIdx.x] = p;
    __threadfence();
    int ticket = atomicAdd(header + SSW_H_TICKET_A, 1);
    last = ticket == n_blocks - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  // exclusive scan of the block totals, 256 at a time with a running carry
  Tri carry{0, 0, 0ull};
  for (int b0 = 0; b0 < n_blocks; b0 += kScanThreads) {
    int b = b0 + threadIdx.x;
    Tri v{0, 0, 0ull};
    if (b < n_blocks) {
      int4 p = __ldcg(reinterpret_cast<const int4*>(partials) + b);
      v = Tri{p.x, p.y, ((unsigned long long)(unsigned)p.w << 32) | (unsigned)p.z};
    }
    Tri tot2;
    Tri ex = block_excl_scan(v, tot2);
    ex = tri_add(ex, carry);
    if (b < n_blocks) {
      reinterpret_cast<int4*>(partials)[b] =
          make_int4(ex.flags, ex.rows, (int)(ex.sq & 0xffffffffull), (int)(ex.sq >> 32));
    }
    carry = tri_add(carry, tot2);
  }
  if (threadIdx.x == 0) {
    header[SSW_H_W] = carry.flags;
    header[SSW_H_N] = carry.rows;
    header[SSW_H_SUMC2_LO] = (int)(carry.sq & 0xffffffffull);
    header[SSW_H_SUMC2_HI] = (int)(carry.sq >> 32);
  }
}

__global__ void __launch_bounds__(kScanThreads) k_compact(int32_t* __restrict__ count, int n_windows,
                                                          const int32_t* __restrict__ partials,
                                                          int32_t* __restrict__ header, int32_t* __restrict__ win_id,
                                                          int32_t* __restrict__ win_start,
                                                          int32_t* __restrict__ coo_start, int32_t* __restrict__ bins_base,
                                                          int n_per_window, int tile, int padded, int n_blocks,
                                                          int pack_cap) {
  extern __shared__ int32_t hist[];  // n_per_window + 2
  BinTables bins(bins_base, n_per_window);
  for (int i = threadIdx.x; i < n_per_window + 2; i += blockDim.x) hist[i] = 0;
  grid_dependency_wait();
  __syncthreads();
  int base = blockIdx.x * kScanBlock + threadIdx.x * kScanItems;
  int c[kScanItems];
  Tri t{0, 0, 0ull};
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    int w = base + i;
    c[i] = w < n_windows ? count[w] : 0;
    t.flags += c[i] > 0;
    t.rows += c[i];
    t.sq += (unsigned long long)c[i] * (unsigned long long)c[i];
  }
  Tri tot;
  Tri ex = block_excl_scan(t, tot);
  int4 p = __ldcg(reinterpret_cast<const int4*>(partials) + blockIdx.x);
  ex = tri_add(ex, Tri{p.x, p.y, ((unsigned long long)(unsigned)p.w << 32) | (unsigned)p.z});
  int cmax = 0;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    int w = base + i;
    if (w < n_windows) {
      if (c[i] > 0) {
        win_id[ex.flags] = w;
        win_start[ex.flags] = ex.rows;
        coo_start[ex.flags] = (int)ex.sq;
        count[w] = ex.flags;
        atomicAdd(&hist[c[i] <= n_per_window ? c[i] : n_per_window + 1], 1);
        cmax = max(cmax, c[i]);
        ex.flags += 1;
        ex.rows += c[i];
        ex.sq += (unsigned long long)c[i] * (unsigned long long)c[i];
      } else {
        count[w] = -1;
      }
    }
  }
  cmax = max(cmax, __shfl_xor_sync(0xffffffffu, cmax, 16));
  cmax = max(cmax, __shfl_xor_sync(0xffffffffu, cmax, 8));
  cmax = max(cmax, __shfl_xor_sync(0xffffffffu, cmax, 4));
  cmax = max(cmax, __shfl_xor_sync(0xffffffffu, cmax, 2));
  cmax = max(cmax, __shfl_xor_sync(0xffffffffu, cmax, 1));
  if ((threadIdx.x & 31) == 0 && cmax > 0) atomicMax(header + SSW_H_CMAX, cmax);
  __syncthreads();
  for (int i = threadIdx.x; i < n_per_window + 2; i += blockDim.x)
    if (hist[i]) atomicAdd(bins.cnt + i, hist[i]);
  __shared__ bool last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    int ticket = atomicAdd(header + SSW_H_TICKET_B, 1);
    last = ticket == n_blocks - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  // Per-occupancy starts: exclusive scans over c = 0..n_per_window of (windows, rows, items).
  int W = __ldcg(header + SSW_H_W);
  int N = __ldcg(header + SSW_H_N);
  unsigned long long sq = ((unsigned long long)(unsigned)__ldcg(header + SSW_H_SUMC2_HI) << 32) |
                          (unsigned)__ldcg(header + SSW_H_SUMC2_LO);
  Tri carry{0, 0, 0ull};  // flags = windows, rows = rows, sq = work items
  for (int c0 = 0; c0 < n_per_window + 2; c0 += kScanThreads) {
    int cc = c0 + threadIdx.x;
    int cnt = cc < n_per_window + 2 ? __ldcg(bins.cnt + cc) : 0;
    Tri v{cnt, cnt * cc, (unsigned long long)packs_of_bin(cc, cnt, tile, padded)};
    Tri tot2;
    Tri e2 = block_excl_scan(v, tot2);
    e2 = tri_add(e2, carry);
    if (cc < n_per_window + 2) {
      bins.wstart[cc] = e2.flags;
      bins.rowstart[cc] = e2.rows;
      bins.packstart[cc] = (int)e2.sq;
      bins.fill[cc] = 0;
      if (cc == tile + 1) header[SSW_H_PACKS_SMALL] = (int)e2.sq;
    }
    carry = tri_add(carry, tot2);
  }
  __syncthreads();  // PACKS_SMALL (written by whichever thread owns c = tile + 1) before thread 0 may clear it
  if (threadIdx.x == 0) {
    win_start[W] = N;
    coo_start[W] = (int)sq;
    // The descriptor array holds pack_cap items (an upper bound for every occupancy histogram the
    // layout call could foresee).  Should a count ever exceed it, the plan is declared empty and
    // flagged rather than written past its end.
    const bool fits = carry.sq <= (unsigned long long)pack_cap;
    if (!fits) atomicOr(reinterpret_cast<unsigned*>(header + SSW_H_ERROR), SSW_DEV_BAD_PLAN);
    header[SSW_H_PACKS] = fits ? (int)carry.sq : 0;
    if (!fits) header[SSW_H_PACKS_SMALL] = 0;
    else if (tile + 1 > n_per_window + 1) header[SSW_H_PACKS_SMALL] = (int)carry.sq;
    header[SSW_H_TILE] = tile;
    header[SSW_H_PADDED] = padded;
    if (sq >= (1ull << 31)) atomicOr(reinterpret_cast<unsigned*>(header + SSW_H_ERROR), SSW_DEV_COO_RANGE);
  }
}

// Blocks [0, w_blocks): one thread per non-empty window, claims a slot in its occupancy bin.
// Blocks [w_blocks, ...): one thread per work item, locates its bin and writes the descriptor.
__global__ void k_order(const int32_t* __restrict__ header, const int32_t* __restrict__ win_start,
                        int32_t* __restrict__ win_pstart, int32_t* __restrict__ pack_win,
                        int32_t* __restrict__ pack_desc, int32_t* __restrict__ bins_base, int n_per_window, int tile,
                        int padded, int w_blocks, int pack_cap) {
  BinTables bins(bins_base, n_per_window);
  grid_dependency_wait();
  if ((int)blockIdx.x < w_blocks) {
    int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= header[SSW_H_W]) return;
    int c = win_start[k + 1] - win_start[k];
    int slot = atomicAdd(bins.fill + c, 1);
    win_pstart[k] = bins.rowstart[c] + slot * c;
    pack_win[bins.wstart[c] + slot] = k;
    return;
  }
  int p = (blockIdx.x - w_blocks) * blockDim.x + threadIdx.x;
  if (p >= header[SSW_H_PACKS] || p >= pack_cap) return;
  // largest c with packstart[c] <= p and a non-empty bin: binary search on the monotone table
  int lo = 1, hi = n_per_window;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (bins.packstart[mid] <= p) lo = mid; else hi = mid - 1;
  }
  int c = lo;
  int q = p - bins.packstart[c];
  int cnt = bins.cnt[c];
  int4 d;
  if (c <= tile) {
    int wpp = windows_per_pack(c, tile, padded);
    int first = q * wpp;
    d = make_int4(bins.rowstart[c] + first * c, c, min(wpp, cnt - first), bins.wstart[c] + first);
  } else {
    int tiles = (c + tile - 1) / tile;
    int wl = q / tiles, qt = q - wl * tiles;
    d = make_int4(bins.rowstart[c] + wl * c, c, -(qt + 1), bins.wstart[c] + wl);
  }
  reinterpret_cast<int4*>(pack_desc)[p] = d;
}

__global__ void k_scatter(KeySrc s, int64_t n, int words, const int32_t* __restrict__ compact,
                          const uint32_t* __restrict__ bitmap, const int32_t* __restrict__ win_start,
                          const int32_t* __restrict__ win_pstart, int32_t* __restrict__ perm,
                          int32_t* __restrict__ inv_perm, int32_t* __restrict__ pack_perm,
                          int32_t* __restrict__ pack_meta) {
  int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int w = 0, pos = 0, r = 0;
  const bool ok = v < n && load_key(s, v, w, pos, r);  // coordinates are an input, not a product of the chain
  grid_dependency_wait();
  if (!ok || w < s.win_lo || w >= s.win_hi) return;
  int k = compact[w];
  if (k < 0) return;
  const uint32_t* bm = bitmap + (int64_t)w * words;
  int rank = 0;
  int full = pos >> 5;
  for (int i = 0; i < full; ++i) rank += __popc(__ldg(bm + i));
  rank += __popc(__ldg(bm + full) & ((1u << (pos & 31)) - 1u));
  int dst = win_start[k] + rank;
  perm[dst] = (int)v;
  inv_perm[v] = dst;
  int pdst = win_pstart[k] + rank;
  pack_perm[pdst] = (int)v;
  int wyx = s.rpbw[1] * s.rpbw[2];
  int pz = pos / wyx, rem = pos - pz * wyx;
  int py = rem / s.rpbw[2], px = rem - py * s.rpbw[2];
  int rel = (pz * (2 * s.rpbw[1] - 1) + py) * (2 * s.rpbw[2] - 1) + px;
  pack_meta[pdst] = pos | (r << kMetaRegionShift) | (rel << kMetaRelShift);
}

static void fill_keysrc(KeySrc& s, const int32_t* coords, const ssw_geometry* g, const int32_t* indices,
                        const int8_t* mask, int mask_windows, const int32_t* rpbw, int n_windows, int n_per_window) {
  s.coords = coords;
  s.indices = indices;
  s.mask = mask;
  s.mask_windows = mask_windows > 0 ? mask_windows : 1;
  s.batch = 1;
  s.shifted = 0;
  for (int i = 0; i < 3; ++i) {
    s.dims[i] = s.dims_p[i] = s.ws[i] = s.nwin[i] = 1;
    s.ss[i] = 0;
    s.rpbw[i] = rpbw ? rpbw[i] : 1;
  }
  if (g) {
    s.batch = g->batch;
    s.shifted = g->shifted;
    for (int i = 0; i < 3; ++i) {
      s.dims[i] = g->dims[i];
      s.dims_p[i] = g->dims_p[i];
      s.ws[i] = g->ws[i];
      s.ss[i] = g->ss[i];
      s.nwin[i] = g->nwin[i];
    }
  }
  s.n_windows = n_windows;
  s.n_per_window = n_per_window;
  s.win_lo = 0;
  s.win_hi = 0x7fffffff;
}

}  // namespace ssw

using namespace ssw;

static inline int64_t align4(int64_t x) { return (x + 3) & ~int64_t(3); }

extern "C" int ssw_geometry_resolve(ssw_geometry* g) {
  if (!g || g->batch <= 0) return SSW_E_INVALID;
  int64_t nw = g->batch, n = 1;
  g->shifted = 0;
  for (int i = 0; i < 3; ++i) {
    if (g->dims[i] <= 0 || g->window[i] <= 0 || g->shift[i] < 0) return SSW_E_INVALID;
    g->ws[i] = g->window[i];
    g->ss[i] = g->shift[i];
    if (g->dims[i] <= g->window[i]) {  // clamp rule of get_window_size
      g->ws[i] = g->dims[i];
      g->ss[i] = 0;
    }
    if (g->ss[i] >= g->ws[i]) return SSW_E_INVALID;
    g->dims_p[i] = g->dims[i] + (g->ws[i] - g->dims[i] % g->ws[i]) % g->ws[i];
    g->nwin[i] = g->dims_p[i] / g->ws[i];
    nw *= g->nwin[i];
    n *= g->ws[i];
    if (g->ss[i] > 0) g->shifted = 1;
  }
  if (n > kMaxPerWindow) return SSW_E_UNSUPPORTED;
  if (nw * n >= (int64_t(1) << 31)) return SSW_E_RANGE;
  g->n_per_window = (int32_t)n;
  g->n_windows = (int32_t)nw;
  return SSW_OK;
}

extern "C" int ssw_window_keys(const int32_t* coords, int64_t n_vox, const ssw_geometry* g, int32_t* indices,
                               int8_t* region, int32_t* dev_error, void* stream) {
  if (!g || n_vox < 0 || (n_vox > 0 && (!coords || !indices))) return SSW_E_INVALID;
  if (n_vox >= (int64_t(1) << 31)) return SSW_E_RANGE;
  if (n_vox == 0) return SSW_OK;
  KeySrc s;
  fill_keysrc(s, coords, g, nullptr, nullptr, 0, nullptr, g->n_windows, g->n_per_window);
  k_window_keys<<<(unsigned)ceil_div64(n_vox, 256), 256, 0, (cudaStream_t)stream>>>(s, n_vox, indices, region,
                                                                                     dev_error);
  SSW_LAUNCH_CHECK("k_window_keys");
  return SSW_OK;
}

extern "C" int ssw_plan_layout_init(ssw_plan_layout* L, int64_t n_vox, int32_t n_windows, int32_t n_per_window,
                                    int32_t tile_rows, int32_t padded) {
  if (!L || n_vox < 0 || n_windows <= 0 || n_per_window <= 0) return SSW_E_INVALID;
  if (n_per_window > kMaxPerWindow) return SSW_E_UNSUPPORTED;
  if (n_vox >= (int64_t(1) << 31) - 4096) return SSW_E_RANGE;
  if (tile_rows <= 0) tile_rows = 64;
  if (tile_rows > 64) return SSW_E_INVALID;
  if (padded && (tile_rows & 15)) return SSW_E_INVALID;
  L->n_vox = n_vox;
  L->n_windows = n_windows;
  L->n_per_window = n_per_window;
  L->tile_rows = tile_rows;
  L->padded = padded ? 1 : 0;
  L->w_cap = (int32_t)(n_vox < n_windows ? n_vox : n_windows);
  if (L->w_cap < 1) L->w_cap = 1;
  // Work items: a bin of cnt windows with occupancy c gives ceil(cnt / floor(tile / slots(c))) packs
  // (c <= tile) or cnt * ceil(c / tile) query tiles.  With floor(x) >= x / 2 for x >= 1 and
  // slots(c) = c (contiguous) or < 2c (padded) the sum over bins stays below
  // (2 or 4) * N / tile + one item of rounding per occupancy.
  int64_t pack_cap = (padded ? 4 : 2) * ceil_div64(n_vox, tile_rows) + n_per_window + 2;
  if (pack_cap >= (int64_t(1) << 31)) return SSW_E_RANGE;
  L->pack_cap = (int32_t)pack_cap;
  L->bitmap_words = (n_per_window + 31) / 32;
  int64_t o = 0;
  L->off_header = o; o += SSW_HEADER_INTS;
  L->off_bins = o; o = align4(o + 5ll * (n_per_window + 2));
  L->off_perm = o; o = align4(o + n_vox);
  L->off_inv_perm = o; o = align4(o + n_vox);
  L->off_win_id = o; o = align4(o + L->w_cap);
  L->off_win_start = o; o = align4(o + L->w_cap + 1);
  L->off_coo_start = o; o = align4(o + L->w_cap + 1);
  L->off_win_pstart = o; o = align4(o + L->w_cap);
  L->off_pack_win = o; o = align4(o + L->w_cap);
  L->off_pack_perm = o; o = align4(o + n_vox);
  L->off_pack_meta = o; o = align4(o + n_vox);
  L->off_pack_desc = o; o = align4(o + 4ll * L->pack_cap);
  L->plan_ints = o;
  int64_t blocks = ceil_div64(n_windows, kScanBlock);
  int64_t s = 0;
  L->off_count = s; s = align4(s + n_windows);
  L->off_bitmap = s; s = align4(s + (int64_t)n_windows * L->bitmap_words);
  L->off_partials = s; s = align4(s + 4 * blocks);
  L->scratch_ints = s;
  return SSW_OK;
}

extern "C" int ssw_bucket_windows(const int32_t* coords, const ssw_geometry* geom, const int32_t* indices,
                                  const int8_t* mask, int32_t mask_windows, const int32_t rpb_window[3],
                                  const ssw_plan_layout* L, int32_t* plan, int32_t* scratch, void* stream_) {
  return ssw_bucket_windows_range(coords, geom, indices, mask, mask_windows, rpb_window, L, plan, scratch, 0, 0x7fffffff,
                                  stream_);
}

extern "C" int ssw_bucket_windows_range(const int32_t* coords, const ssw_geometry* geom, const int32_t* indices,
                                        const int8_t* mask, int32_t mask_windows, const int32_t rpb_window[3],
                                        const ssw_plan_layout* L, int32_t* plan, int32_t* scratch, int32_t win_lo,
                                        int32_t win_hi, void* stream_) {
  if (!L || !plan || !scratch || !rpb_window) return SSW_E_INVALID;
  if (win_lo < 0 || win_hi < win_lo) return SSW_E_INVALID;
  if ((coords != nullptr) == (indices != nullptr) && L->n_vox > 0) return SSW_E_INVALID;
  if (coords && !geom) return SSW_E_INVALID;
  if (coords && (geom->n_windows != L->n_windows || geom->n_per_window != L->n_per_window)) return SSW_E_INVALID;
  if (mask && mask_windows <= 0) return SSW_E_INVALID;
  for (int i = 0; i < 3; ++i)
    if (rpb_window[i] <= 0) return SSW_E_INVALID;
  // relative-position code must fit 15 bits
  {
    int64_t top = ((int64_t)(rpb_window[0]) * (2 * rpb_window[1] - 1) + rpb_window[1]) * (2 * rpb_window[2] - 1) +
                  rpb_window[2];
    int64_t need = (int64_t)L->n_per_window / (rpb_window[1] * rpb_window[2]) + 1;
    int64_t worst = (need * (2 * rpb_window[1] - 1) + rpb_window[1]) * (2 * rpb_window[2] - 1) + rpb_window[2];
    if (top >= 32768 || worst >= 32768) return SSW_E_UNSUPPORTED;
  }
  cudaStream_t stream = (cudaStream_t)stream_;
  const int64_t N = L->n_vox;
  const int n = L->n_per_window;
  int32_t* header = plan + L->off_header;
  // header and the bin tables are adjacent: one clear covers both
  SSW_CUDA_TRY(cudaMemsetAsync(plan, 0, sizeof(int32_t) * (size_t)(L->off_perm), stream));
  if (N == 0) return SSW_OK;
  SSW_CUDA_TRY(cudaMemsetAsync(scratch, 0, sizeof(int32_t) * (size_t)L->off_partials, stream));
  KeySrc s;
  fill_keysrc(s, coords, geom, indices, mask, mask_windows, rpb_window, L->n_windows, n);
  s.win_lo = win_lo;
  s.win_hi = win_hi;
  int32_t* count = scratch + L->off_count;
  uint32_t* bitmap = reinterpret_cast<uint32_t*>(scratch + L->off_bitmap);
  int32_t* partials = scratch + L->off_partials;
  const unsigned vox_blocks = (unsigned)ceil_div64(N, 256);
  // first of the chain: ordinary launch, fully ordered behind the clears and the caller's earlier work
  k_count<<<vox_blocks, 256, 0, stream>>>(s, N, L->bitmap_words, count, bitmap, header);
  SSW_LAUNCH_CHECK("k_count");
  const int blocks = (int)ceil_div64(L->n_windows, kScanBlock);
  SSW_CUDA_TRY(launch_chained(k_reduce, dim3(blocks), dim3(kScanThreads), 0, stream, (const int32_t*)count,
                              (int)L->n_windows, partials, header, blocks));
  SSW_CUDA_TRY(launch_chained(k_compact, dim3(blocks), dim3(kScanThreads), sizeof(int32_t) * (n + 2), stream, count,
                              (int)L->n_windows, (const int32_t*)partials, header, plan + L->off_win_id,
                              plan + L->off_win_start, plan + L->off_coo_start, plan + L->off_bins, n,
                              (int)L->tile_rows, (int)L->padded, blocks, (int)L->pack_cap));
  const int w_blocks = (int)ceil_div64(L->w_cap, 256);
  const int p_blocks = (int)ceil_div64(L->pack_cap, 256);
  SSW_CUDA_TRY(launch_chained(k_order, dim3(w_blocks + p_blocks), dim3(256), 0, stream, (const int32_t*)header,
                              (const int32_t*)(plan + L->off_win_start), plan + L->off_win_pstart,
                              plan + L->off_pack_win, plan + L->off_pack_desc, plan + L->off_bins, n,
                              (int)L->tile_rows, (int)L->padded, w_blocks, (int)L->pack_cap));
  SSW_CUDA_TRY(launch_chained(k_scatter, dim3(vox_blocks), dim3(256), 0, stream, s, N, (int)L->bitmap_words,
                              (const int32_t*)count, (const uint32_t*)bitmap, (const int32_t*)(plan + L->off_win_start),
                              (const int32_t*)(plan + L->off_win_pstart), plan + L->off_perm, plan + L->off_inv_perm,
                              plan + L->off_pack_perm, plan + L->off_pack_meta));
  return SSW_OK;
}

// ---------------------------------------------------------------------------------------------
// Bucketing without a caller-provided scratch buffer
// ---------------------------------------------------------------------------------------------
// Some hosts of this library cannot give it scratch memory: a plugin that runs inside another
// framework's memory plan, or under a runtime that forbids device allocation after start-up, has
// nowhere to get the per-window counters and occupancy bitmaps from (cudaMalloc is off limits and
// no allocator handle crosses the C ABI).  For them the scratch lives here, in a fixed array that
// is part of the loaded module: 4 Mi int32 = 16 MiB, held by every device that loads the library
// until the process exits.
constexpr int64_t kStaticScratchInts = int64_t(4) << 20;
static __device__ __align__(256) int32_t g_static_scratch[kStaticScratchInts];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the
// address a kernel can use has to be asked for, once per device, with that device current.  The
// answer is cached per device for the life of the process: a caller that destroys the device's
// context (cudaDeviceReset) invalidates it and must not use this entry point afterwards.
static int32_t* g_static_scratch_ptr[64] = {nullptr};

extern "C" int64_t ssw_bucket_windows_static_capacity(void) { return kStaticScratchInts; }

extern "C" int ssw_bucket_windows_static(const int32_t* coords, const ssw_geometry* geom, const int32_t* indices,
                                         const int8_t* mask, int32_t mask_windows, const int32_t rpb_window[3],
                                         const ssw_plan_layout* L, int32_t* plan, void* stream) {
  if (!L) return SSW_E_INVALID;
  if (L->scratch_ints > kStaticScratchInts) {
    char msg[160];
    snprintf(msg, sizeof(msg), "ssw_bucket_windows_static: needs %lld scratch ints, the built-in array holds %lld",
             (long long)L->scratch_ints, (long long)kStaticScratchInts);
    ssw::set_error_text(msg);
    return SSW_E_WORKSPACE;
  }
  int dev = 0;
  SSW_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return SSW_E_UNSUPPORTED;
  if (!g_static_scratch_ptr[dev]) {  // set-up: first call on this device
    void* p = nullptr;
    SSW_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
    g_static_scratch_ptr[dev] = static_cast<int32_t*>(p);
  }
  return ssw_bucket_windows(coords, geom, indices, mask, mask_windows, rpb_window, L, plan, g_static_scratch_ptr[dev],
                            stream);
}
