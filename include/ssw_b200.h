/*
 * ssw_b200.h — C ABI of the B200 (sm_100a) sparse window-attention library.
 *
 * Every entry point takes raw device pointers, plain integer sizes and a CUDA stream
 * (passed as void*, NULL = the legacy default stream) and returns an int status
 * (SSW_OK or a negative SSW_E_* code).  Nothing here allocates device memory unless
 * its comment says so; the caller owns every buffer.  No exception crosses this
 * boundary and no PyTorch type appears in it.
 *
 * Each declaration cites the upstream SparseSwin3D interface it replaces, as
 * file:line inside that project.
 */
#ifndef SSW_B200_H
#define SSW_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ---------------------------------------------------------------- */
#define SSW_OK 0
#define SSW_E_INVALID (-1)     /* bad argument (null pointer, size, alignment, dtype)  */
#define SSW_E_RANGE (-2)       /* a size leaves the int32 domain the layout can hold   */
#define SSW_E_UNSUPPORTED (-3) /* head_dim / window size outside the compiled variants */
#define SSW_E_CUDA (-4)        /* a CUDA runtime call failed; see ssw_last_cuda_error  */
#define SSW_E_WORKSPACE (-5)   /* caller-provided buffer smaller than the layout needs */

/* Bits of the device-side error word (plan header slot SSW_H_ERROR). */
#define SSW_DEV_BAD_COORD 1u   /* a voxel falls outside the grid / window table         */
#define SSW_DEV_DUPLICATE 2u   /* two voxels share (window, pos); upstream forbids it   */
#define SSW_DEV_COO_RANGE 4u   /* sum c^2 * H would not fit int32 (COO path unusable)   */
#define SSW_DEV_TIMEOUT 8u     /* a bounded wait on an async copy gave up               */
#define SSW_DEV_BAD_PLAN 16u   /* the plan handed to an attention kernel is inconsistent */

/* ---- element types --------------------------------------------------------------- */
#define SSW_F32 0
#define SSW_BF16 1
#define SSW_F16 2

const char* ssw_status_string(int status);
const char* ssw_last_cuda_error(void);
int ssw_version(void);

/* ---- window geometry --------------------------------------------------------------
 * Replaces get_window_size (swin3d_base.py:276-300), the pad amounts of
 * SwinTransformerBlock.forward_part1 (swin3d_base.py:743-751), pad_sparse_tensor
 * (:501-526), roll_sparse_tensor (:529-554), window_partition_sparse (:336-372) and
 * the region ids of compute_mask (:436-452) with one closed-form description. */
typedef struct ssw_geometry {
  int32_t batch;        /* number of scenes in the batch                               */
  int32_t dims[3];      /* dense grid (D,H,W) before padding                           */
  int32_t window[3];    /* requested window size                                       */
  int32_t shift[3];     /* requested cyclic shift (0,0,0 for W-MSA)                    */
  /* filled by ssw_geometry_resolve: */
  int32_t ws[3];        /* window after clamping to the grid                           */
  int32_t ss[3];        /* shift after clamping                                        */
  int32_t dims_p[3];    /* dims padded up to a multiple of ws                          */
  int32_t nwin[3];      /* windows per axis                                            */
  int32_t n_per_window; /* ws[0]*ws[1]*ws[2]                                           */
  int32_t n_windows;    /* batch * nwin[0]*nwin[1]*nwin[2], empty windows included     */
  int32_t shifted;      /* 1 if any ss > 0                                             */
} ssw_geometry;

/* Host only.  SSW_E_RANGE when n_windows * n_per_window does not fit int32. */
int ssw_geometry_resolve(ssw_geometry* g);

/* coords[N,4] int32 (b,z,y,x) -> indices[N,2] int32 (window,pos); region[N] int8 (may be
 * NULL) receives the compute_mask region id of every voxel in the shifted frame.
 * dev_error (int32*, may be NULL) gets SSW_DEV_BAD_COORD or-ed in for out-of-grid rows. */
int ssw_window_keys(const int32_t* coords, int64_t n_vox, const ssw_geometry* g,
                    int32_t* indices, int8_t* region, int32_t* dev_error, void* stream);

/* ---- window bucketing -------------------------------------------------------------
 * One device-side counting sort of the N voxels by (window, pos) with int32 keys only.
 * Replaces the three radix sorts over N*C keys that qkv_sparse_indices / permute do
 * (ops.cu:276-335, swin3d_base.py:47-59, :673), the bincount/unique/cumsum chain that
 * derives `_c` and the block offsets (ops.cu:775-784, 813-841) and return_inverse
 * (ops.cu:718-730, used at swin3d_base.py:674).
 *
 * All results live in ONE int32 array `plan` whose sub-array offsets are given by
 * ssw_plan_layout (so the caller can allocate once and slice).  `scratch` is a second
 * int32 array that the call zeroes and uses; its contents are meaningless afterwards. */
#define SSW_HEADER_INTS 64
enum {
  SSW_H_N = 0,        /* voxels                                                        */
  SSW_H_W = 1,        /* non-empty windows                                             */
  SSW_H_PACKS = 2,    /* work items of the fused kernel                                */
  SSW_H_ERROR = 3,    /* SSW_DEV_* bits                                                */
  SSW_H_CMAX = 4,     /* largest window occupancy                                      */
  SSW_H_SUMC2_LO = 5, /* sum over windows of c^2, low / high 32 bits                   */
  SSW_H_SUMC2_HI = 6,
  SSW_H_TILE = 7,     /* tile_rows the plan was built for                              */
  SSW_H_TICKET_A = 8, /* internal                                                      */
  SSW_H_TICKET_B = 9, /* internal                                                      */
  SSW_H_PACKS_SMALL = 10, /* leading work items that are packs of windows with c <= tile */
  SSW_H_PADDED = 11   /* 1: packs give every window a padded run of row slots (tensor-core kernel) */
};

typedef struct ssw_plan_layout {
  int64_t n_vox;
  int32_t n_windows;    /* dense window count (geometry.n_windows)                      */
  int32_t n_per_window; /* positions per window                                         */
  int32_t tile_rows;    /* query/key rows one work item of the fused kernel holds       */
  int32_t w_cap;        /* capacity for non-empty windows = min(n_vox, n_windows)       */
  int32_t pack_cap;     /* upper bound of fused-kernel work items                       */
  int32_t bitmap_words; /* ceil(n_per_window / 32)                                      */
  int32_t padded;       /* packs pad windows to 1,2,4,8,16,32,.. row slots (16-bit inputs)   */
  int32_t reserved_;    /* keeps the 64-bit members aligned                             */
  /* offsets into `plan`, in int32 units */
  int64_t off_header;   /* [SSW_HEADER_INTS]                                            */
  int64_t off_perm;     /* [N]   sorted row (window,pos order) -> voxel                 */
  int64_t off_inv_perm; /* [N]   voxel -> sorted row  (upstream's arg_sort)             */
  int64_t off_win_id;   /* [w_cap]   k-th non-empty window -> dense window id           */
  int64_t off_win_start;/* [w_cap+1] k -> first sorted row; diff = occupancy c_k (`_c`) */
  int64_t off_coo_start;/* [w_cap+1] k -> exclusive sum of c^2 (valid if no COO_RANGE)  */
  int64_t off_win_pstart;/*[w_cap]   k -> first row in occupancy-class ("pack") order   */
  int64_t off_pack_win; /* [w_cap]   window slot in pack order -> k                     */
  int64_t off_pack_perm;/* [N]   pack-order row -> voxel                                */
  int64_t off_pack_meta;/* [N]   pack-order row -> pos | region<<10 | relcode<<16       */
  int64_t off_pack_desc;/* [pack_cap*4] work items {first row, c, nwin | -(qtile+1), slot} */
  int64_t off_bins;     /* [5*(n_per_window+2)] per-occupancy tables                    */
  int64_t plan_ints;    /* total size of `plan`                                         */
  /* offsets into `scratch`, in int32 units */
  int64_t off_count;    /* [n_windows]                                                  */
  int64_t off_bitmap;   /* [n_windows*bitmap_words]                                     */
  int64_t off_partials; /* [4*blocks]                                                   */
  int64_t scratch_ints;
} ssw_plan_layout;

/* Host only.  tile_rows in 1..64 (0 means 64).  padded != 0 builds the work list for the
 * tensor-core kernel that serves 16-bit inputs (tile_rows then a multiple of 16); take both values
 * from ssw_default_tile_rows / ssw_default_padded for the configuration. */
int ssw_plan_layout_init(ssw_plan_layout* L, int64_t n_vox, int32_t n_windows, int32_t n_per_window,
                         int32_t tile_rows, int32_t padded);
/* The default tile_rows for a configuration (host only): the largest tile that leaves three
 * (fp32, CUDA-core kernel) or four (16-bit, tensor-core kernel) pipeline stages in one SM's shared
 * memory next to the bias table, when that is small enough to be staged there. */
int32_t ssw_default_tile_rows(int32_t heads, int32_t head_dim, int dtype, const int32_t rpb_window[3]);
/* 1 when ssw_attn_fused serves this dtype with the tensor-core kernel (bf16, fp16), else 0. */
int32_t ssw_default_padded(int dtype);

/* Key source of ssw_bucket_windows: exactly one of `coords` (with `geom`) or `indices` is
 * non-NULL.  With `indices` ([N,2] int32, the layout window_partition_sparse leaves in
 * x.indices, swin3d_base.py:351-371) the optional `mask` [mask_windows, n_per_window] int8
 * is the tensor compute_mask returns (swin3d_base.py:436-452) and region ids are gathered
 * from it as sp_add_mask does (:574-576); with `coords` they are computed in closed form
 * when geom->shifted.  rpb_window is the window size the module's bias table was built
 * for (swin3d_base.py:624-647); it only affects the relative-position code in pack_meta. */
int ssw_bucket_windows(const int32_t* coords, const ssw_geometry* geom,
                       const int32_t* indices, const int8_t* mask, int32_t mask_windows,
                       const int32_t rpb_window[3],
                       const ssw_plan_layout* L, int32_t* plan, int32_t* scratch, void* stream);

/* ssw_bucket_windows restricted to the voxels whose window id (as ssw_window_keys gives it) lies
 * in [win_lo, win_hi): the others are skipped without error, their inv_perm entries stay
 * unwritten, and header[SSW_H_N] counts the voxels taken.  Voxel ids in the plan still refer to the
 * caller's full arrays.  This is the shard of one scene a GPU works on when the scene is split by
 * contiguous window ranges (windows never interact: ops.cu:359-377 computes block by block). */
int ssw_bucket_windows_range(const int32_t* coords, const ssw_geometry* geom,
                             const int32_t* indices, const int8_t* mask, int32_t mask_windows,
                             const int32_t rpb_window[3],
                             const ssw_plan_layout* L, int32_t* plan, int32_t* scratch,
                             int32_t win_lo, int32_t win_hi, void* stream);

/* No counterpart in upstream.  ssw_bucket_windows for callers that cannot hand over scratch memory:
 * hosts that embed this library inside another framework's memory plan, or run under a runtime
 * that forbids device allocation once it has started, have no buffer to pass as `scratch`.  The
 * scratch is a fixed 16 MiB (4 Mi int32) array inside the library image instead, resident on every
 * device that loads the library until the process exits.  Same arguments and results as
 * ssw_bucket_windows minus `scratch`; the caller still provides `plan`.  Returns SSW_E_WORKSPACE
 * (details in ssw_last_cuda_error) when L->scratch_ints exceeds
 * ssw_bucket_windows_static_capacity().  The function allocates nothing, neither through CUDA nor
 * through any library.  The first call on a device looks up the array's device address; make that
 * first call outside any stream capture.  The address is remembered per device for the life of
 * the process, so do not call this after destroying the device's context (cudaDeviceReset).  All
 * calls on a device share the one array and each call
 * clears the part it uses, so two calls whose kernels overlap on the GPU (different streams)
 * corrupt each other: serialise them. */
int64_t ssw_bucket_windows_static_capacity(void);
int ssw_bucket_windows_static(const int32_t* coords, const ssw_geometry* geom,
                              const int32_t* indices, const int8_t* mask, int32_t mask_windows,
                              const int32_t rpb_window[3],
                              const ssw_plan_layout* L, int32_t* plan, void* stream);

/* ---- fused W-MSA / SW-MSA core ----------------------------------------------------
 * Replaces, in one kernel per call, everything WindowAttentionSparse.forward does
 * between its two Linear layers (swin3d_base.py:659-675): qkv_sparse_cuda (:483-498),
 * q*scale (:660), spspmm_block_naive 'q_k' (ops.cu:344-378, 788-867), sp_add_rpb
 * (:557-566), sp_add_mask (:569-581), softmax_last_dim (ops.cu:128-167, including its
 * max(0,.) and +1e-8), spspmm_block_naive 'qk_v' (ops.cu:381-418, 868-903), the head
 * permute (:673) and the un-sort to voxel order (:674-675).
 *
 *   qkv   [N, 3, heads, head_dim] of `dtype`, contiguous (the reshaped qkv Linear output)
 *   table [(2Wz-1)(2Wy-1)(2Wx-1), heads] fp32, the relative_position_bias_table
 *   out   [N, heads*head_dim] of `dtype`, rows in the caller's voxel order
 *   attn_vals (may be NULL) receives the post-softmax COO values in upstream order
 *         (window, head, pos_i, pos_j), sum c^2 * heads elements of `dtype`.
 * use_mask != 0 applies the -100 shift mask from the region ids stored in the plan.
 * A contiguous plan runs the CUDA-core kernel (any dtype); a padded plan runs the tensor-core
 * kernel (bf16 / fp16 only, attn_vals must be NULL, SSW_E_INVALID otherwise). */
int ssw_attn_fused(const void* qkv, int dtype, int32_t heads, int32_t head_dim,
                   const ssw_plan_layout* L, const int32_t* plan,
                   const float* table, const int32_t rpb_window[3], float scale, int use_mask,
                   void* out, void* attn_vals, void* stream);

/* ssw_attn_fused with several destination buffers: every finished output row is stored to
 * outs[0..n_outs-1] (1 <= n_outs <= 8), each an [N, heads*head_dim] buffer of `dtype`.  outs[0] is
 * the caller's own; the others are the same buffer on peer GPUs of the node, mapped into the
 * context of the launching device (ssw_peer_buffer_open for another process's buffer,
 * ssw_enable_peer_access for another device of this process): this is how one scene split over several GPUs by
 * window ranges ends with the complete output on every GPU and no gather step - plain stores over
 * NVLink from the kernel's epilogue.  Upstream has no multi-GPU path (it relies on its trainer's
 * data parallelism); the single-destination semantics are those of ssw_attn_fused. */
int ssw_attn_fused_multi(const void* qkv, int dtype, int32_t heads, int32_t head_dim,
                         const ssw_plan_layout* L, const int32_t* plan,
                         const float* table, const int32_t rpb_window[3], float scale, int use_mask,
                         void* const* outs, int32_t n_outs, void* attn_vals, void* stream);
/* Host only: lets kernels on the current device store to memory of `peer_device` (cudaDeviceEnablePeerAccess;
 * "already enabled" is not an error).  SSW_E_UNSUPPORTED when the two devices cannot reach each other. */
int ssw_enable_peer_access(int32_t peer_device);
/* Host only: an output buffer that kernels of OTHER PROCESSES on the node can store to.
 * _create allocates `bytes` of zeroed device memory on the current device (cudaMalloc: this call
 * allocates, it belongs to set-up, not to a pass) and writes its CUDA IPC handle (SSW_IPC_HANDLE_BYTES
 * bytes, to be sent to the peers by any host channel).  _open maps a peer's buffer into the context of
 * the CURRENT device - the device whose kernels will store to it; a mapping made under another device
 * of this process is not reachable from the launching device and faults - and enables peer access as
 * needed.  _close unmaps an opened buffer; every peer must have closed before the owner calls _destroy. */
#define SSW_IPC_HANDLE_BYTES 64
int ssw_peer_buffer_create(int64_t bytes, void** ptr, unsigned char* handle);
int ssw_peer_buffer_open(const unsigned char* handle, void** ptr);
int ssw_peer_buffer_close(void* ptr);
int ssw_peer_buffer_destroy(void* ptr);

/* The element-wise shell of a Swin block between its GEMMs (swin3d_base.py:741-782: norm1, the
 * residual add after attention, norm2, the residual add after the MLP) in one pass over the voxel
 * rows: sum = a + b (b may be NULL: sum = a), norm = LayerNorm(sum) * gamma + beta over the
 * `channels` of each row (biased variance, eps inside the square root, as torch.nn.LayerNorm).
 * a, b, sum_out, norm_out: [n_rows, channels] of `dtype`, 16-byte aligned, channels * element size a
 * multiple of 16 and at most 2048 bytes; sum_out may be a (in place) or NULL, norm_out may be NULL;
 * gamma, beta: fp32 [channels].  With 16-bit rows the normalised value is the rounded sum, i.e. what
 * a separate add followed by LayerNorm computes.  Statistics in fp32. */
int ssw_add_layernorm(const void* a, const void* b, const float* gamma, const float* beta, float eps,
                      int dtype, int64_t n_rows, int32_t channels, void* sum_out, void* norm_out,
                      void* stream);

/* Sparse 3-D convolutions of the layers around the attention stages (upstream takes them from the
 * spconv library: SubMConv3d swin3d_base.py:915-923, 1039-1059; SparseConv3d :932-935, 965-970;
 * SparseInverseConv3d :989-994).  A convolution here is a rulebook (integer kernels), a gathered
 * operand cols[m, tap * Cin + c] = x[nbr[m, tap], c] and one dense GEMM by the host side.
 *
 * ssw_voxel_grid_build: grid[((b * D + z) * H + y) * W + x] = id of the voxel in that cell, -1 for an
 *   empty cell (batch * D * H * W int32, must stay below 2^31 cells).  `err` (may be NULL): device
 *   word that gets SSW_DEV_BAD_COORD / SSW_DEV_DUPLICATE or-ed in.
 * ssw_subm_neighbors: nbr[i, t] for the k^3 taps of a submanifold convolution (k odd, offsets
 *   -k/2..k/2 in z, y, x order, t = (dz * k + dy) * k + dx as a dense cross-correlation with
 *   padding k/2 numbers them); -1 where the neighbour cell is empty or outside the grid.
 * ssw_gather_cols: cols[m, t * cin + c] = x[nbr[m, t], c], zero where nbr < 0 (or >= n_src).
 * ssw_gather_slices: out[i, :] = z[parent[i], tap[i] * cout : (tap[i] + 1) * cout] (z has taps * cout
 *   columns), zero where parent[i] < 0: the scatter side of an inverse convolution whose GEMM
 *   produced all taps of every coarse voxel at once.
 * ssw_gather_reduce: out[i, :] = base[i, :] + sum of y[slots[p], :] over p in [row_start[i], row_start[i+1])
 *   (base may be NULL; row_start has n + 1 entries), summed in fp32 in list order: the output side of
 *   a convolution whose products were formed only for the (input, output) pairs that exist,
 *   grouped by tap.  c * element size a multiple of 16. */
int ssw_voxel_grid_build(const int32_t* coords, int64_t n, int32_t batch, const int32_t dims[3],
                         int32_t* grid, int32_t* err, void* stream);
int ssw_subm_neighbors(const int32_t* coords, int64_t n, int32_t batch, const int32_t dims[3],
                       const int32_t* grid, int32_t ksize, int32_t* nbr, void* stream);
int ssw_gather_cols(const void* x, int dtype, int64_t n_src, int64_t m_rows, int32_t taps, int32_t cin,
                    const int32_t* nbr, void* cols, void* stream);
int ssw_gather_slices(const void* z, int dtype, int64_t n_src, int32_t taps, int32_t cout, int64_t n,
                      const int32_t* parent, const int32_t* tap, void* out, void* stream);
int ssw_gather_reduce(const void* base, const void* y, int dtype, int64_t n_y, const int32_t* row_start,
                      const int32_t* slots, int64_t n_slots, int64_t n, int32_t c, void* out, void* stream);

/* Backward of ssw_attn_fused: gradients of qkv and of the bias table from the gradient of `out`,
 * with the probabilities recomputed instead of stored.  It replaces what upstream's autograd runs
 * for the same span: softmax_last_dim_backward (ops.cu:169-194, swin3d_base.py:177-188) and the
 * blocked gradient products rc_cr / rr_rc / cr_rr with their transposes (ops.cu:422-557, 663-715,
 * 945-1031; swin3d_base.py:106-138), the index_select gradients of sp_add_rpb (:557-566) and the
 * un-sort (:674-675).
 *   grad_out [N, heads*head_dim] and dqkv [N, 3, heads, head_dim] of `dtype`, voxel order
 *   dtable   [(2Wz-1)(2Wy-1)(2Wx-1), heads] fp32: the gradient is ADDED to it (zero it first)
 *   workspace: ssw_attn_fused_bwd_workspace_floats(N, heads) floats, 16-byte aligned
 * Works on contiguous and padded plans alike. */
int64_t ssw_attn_fused_bwd_workspace_floats(int64_t n_vox, int32_t heads);
int ssw_attn_fused_bwd(const void* qkv, const void* grad_out, int dtype, int32_t heads, int32_t head_dim,
                       const ssw_plan_layout* L, const int32_t* plan,
                       const float* table, const int32_t rpb_window[3], float scale, int use_mask,
                       void* dqkv, float* dtable, float* workspace, void* stream);

/* ---- COO operator surface ----------------------------------------------------------
 * The unfused operators upstream exports from sparse_swin/ops.cpp:7-18, with upstream's layouts.
 * Functions whose output size depends on the data come in two steps: a *_plan call that leaves
 * the counts in a small device array (the caller reads them back, as upstream does with .item())
 * and a run call that fills caller-allocated outputs. */

/* flatten_indices (ops.cpp:11, ops.cu:232-273).  indices [D, nnz] int32, sizes: D host ints; the
 * hash is accumulated in int32 and wraps exactly like upstream's. */
int ssw_flatten_indices(const int32_t* indices, int32_t D, int64_t nnz, const int32_t* sizes, int32_t* out,
                        void* stream);

/* sort_indices (ops.cpp:12, ops.cu:276-289): stable argsort of int32 keys, signed order. */
int64_t ssw_argsort_workspace_bytes(int64_t n);
int ssw_argsort_i32(const int32_t* keys, int64_t n, int32_t* perm_out, void* workspace, int64_t workspace_bytes,
                    void* stream);

/* return_inverse (ops.cpp:13, ops.cu:718-730): rank of every x[i] among the distinct values present
 * (all in [0, maxnum)); count_out[0] (device) = number of distinct values; err (device int32) gets
 * SSW_DEV_BAD_COORD or-ed in when a value lies outside [0, maxnum). */
int64_t ssw_return_inverse_workspace_bytes(int64_t maxnum);
int ssw_return_inverse(const int32_t* x, int64_t n, int64_t maxnum, int32_t* rank_out, int32_t* count_out,
                       int32_t* err, void* workspace, int64_t workspace_bytes, void* stream);

/* unique_consecutive_indices (ops.cpp:14, ops.cu:32-103): inverse of unique_consecutive. */
int64_t ssw_scan_workspace_bytes(int64_t n);
int ssw_unique_consecutive_inverse(const int32_t* x, int64_t n, int32_t* out, void* workspace, int64_t workspace_bytes,
                                   void* stream);

/* qkv_sparse_indices (ops.cpp:10, ops.cu:293-335).  indices [N,2] int32; `plan` is the result of
 * ssw_bucket_windows on the same indices.  idx_qv / idx_k [4, N*heads*c] are the UNSORTED index
 * blocks in (voxel, head, channel) order with rows (window, head, pos, ch) / (window, head, ch,
 * pos); perm_qv / perm_k are the argsorts of their row-major keys, produced from the bucketing
 * instead of two radix sorts over N*heads*c keys (so they stay lexicographic even where upstream's
 * int32 hash would wrap). */
int ssw_qkv_sparse_indices(const int32_t* indices, int64_t n_vox, int32_t heads, int32_t c, const ssw_plan_layout* L,
                           const int32_t* plan, int32_t* idx_qv, int32_t* perm_qv, int32_t* idx_k, int32_t* perm_k,
                           void* stream);

/* matmul_cuda_naive (ops.cpp:8, ops.cu:1034-1088 -> 788-943), in two steps.
 * ssw_coo_block_plan reads the index rows of the operand that defines the blocks (the LHS for
 * "q_k", the RHS for "qk_v"; rows of `row_len` = head_dim elements) and writes
 *   blk_start [rows+1]: first row of every (window, head) block, then the row count
 *   sq_start  [rows+1]: exclusive sums of c_b^2
 *   counts (device int64[2]): number of blocks, sum of c_b^2.
 * ssw_coo_matmul (mul_type 0 = "q_k", 1 = "qk_v") then fills out_v [total], out_idx [4,total] and
 * c_out [n_blocks] (upstream's `_c`), total = sum c^2 for q_k and the RHS nnz for qk_v.  The
 * products are sequential FMA chains in upstream's order (ops.cu:371-375, 411-415). */
int64_t ssw_coo_plan_workspace_bytes(int64_t n_rows);
int ssw_coo_block_plan(const int32_t* idx, int64_t nnz, int32_t row_len, int32_t* blk_start, int32_t* sq_start,
                       int64_t* counts, void* workspace, int64_t workspace_bytes, void* stream);
int ssw_coo_matmul(int mul_type, int dtype, const void* m1_v, const int32_t* m1_idx, int64_t nnz1, const void* m2_v,
                   int32_t C, const int32_t* blk_start, const int32_t* sq_start, int64_t n_blocks, int64_t total,
                   void* out_v, int32_t* out_idx, int32_t* c_out, const int64_t* counts, void* stream);

/* Offsets for the `_c`-keyed backward operators: exclusive sums of c and of c^2, [nb+1] each. */
int ssw_coo_offsets_from_counts(const int32_t* c, int64_t nb, int32_t* cstart, int32_t* sqstart, void* workspace,
                                int64_t workspace_bytes, void* stream);
/* matmul_grad_cuda_naive (ops.cpp:9, ops.cu:945-1031): mode 0 "rc_cr", 1 "rr_rc", 2 "cr_rr". */
int ssw_coo_matmul_grad(int mode, int dtype, const void* m1_v, const void* m2_v, const int32_t* cstart,
                        const int32_t* sqstart, int64_t nb, int32_t C, void* out_v, void* stream);
/* qkv_transpose (ops.cpp:17, ops.cu:663-715): rr = 0 "rc", rr = 1 "rr". */
int ssw_coo_block_transpose(int rr, int dtype, const void* m1_v, const int32_t* cstart, const int32_t* sqstart,
                            int64_t nb, int32_t C, void* out_v, void* stream);

/* softmax_last_dim_forward / _backward (ops.cpp:15-16, ops.cu:128-194), fp32.  row_ids: sorted,
 * consecutive from 0; n_rows = row_ids[nnz-1] + 1 (host value, as upstream's .item()); row_start:
 * caller scratch [n_rows + 1].  Forward keeps upstream's max(0, .) and +1e-8. */
int ssw_softmax_rows_fwd(const int32_t* row_ids, int64_t nnz, int32_t n_rows, const float* vals, float* out,
                         int32_t* row_start, void* stream);
int ssw_softmax_rows_bwd(const int32_t* row_ids, int64_t nnz, int32_t n_rows, const float* y, const float* g,
                         float* out, int32_t* row_start, void* stream);

/* sp_add_rpb + sp_add_mask (swin3d_base.py:557-581) in one pass: vals + dense[h, pos_i, pos_j]
 * (dense [H, n, n] of the value dtype, may be NULL) and -100 where mask[w % mask_windows, pos_i] !=
 * mask[..., pos_j] (mask [mask_windows, mask_n] int8, may be NULL). */
int ssw_coo_add_bias_mask(int dtype, const void* vals, const int32_t* idx, int64_t nnz, const void* dense, int32_t n,
                          const int8_t* mask, int32_t mask_windows, int32_t mask_n, void* out, void* stream);

/* ---- debugging aid (host only) -------------------------------------------------------
 * No counterpart in upstream (it launches on the legacy default stream and captures nothing).
 * Writes the dependency edges of a captured CUDA graph (a cudaGraph_t) as text, one per line:
 *   <from> -> <to> <full|programmatic> from_port=<p> to_port=<p>
 * nodes as <index>:<name>, kernel nodes by function name, other nodes as node_type_<n>.  The launches of one call of this
 * library are chained with programmatic dependent launch; this shows how a capture wired them and
 * that joins between streams stayed full dependencies.  SSW_E_WORKSPACE if `text` is too small. */
int ssw_debug_graph_edges(void* graph, char* text, int64_t text_bytes, int64_t* n_nodes, int64_t* n_edges,
                          int64_t* n_programmatic);

#ifdef __cplusplus
}
#endif
#endif /* SSW_B200_H */
