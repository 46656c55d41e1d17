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
  SSW_H_PACKS_SMALL = 10 /* leading work items that are packs of windows with c <= tile */
};

typedef struct ssw_plan_layout {
  int64_t n_vox;
  int32_t n_windows;    /* dense window count (geometry.n_windows)                      */
  int32_t n_per_window; /* positions per window                                         */
  int32_t tile_rows;    /* query/key rows one work item of the fused kernel holds       */
  int32_t w_cap;        /* capacity for non-empty windows = min(n_vox, n_windows)       */
  int32_t pack_cap;     /* upper bound of fused-kernel work items                       */
  int32_t bitmap_words; /* ceil(n_per_window / 32)                                      */
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

/* Host only.  tile_rows in 1..64; 0 means 64. */
int ssw_plan_layout_init(ssw_plan_layout* L, int64_t n_vox, int32_t n_windows, int32_t n_per_window,
                         int32_t tile_rows);
/* The default tile_rows for a configuration (host only): the largest tile whose two pipeline
 * stages, plus the bias table when it is small enough to stage, let two CTAs share an SM. */
int32_t ssw_default_tile_rows(int32_t heads, int32_t head_dim, int dtype, const int32_t rpb_window[3]);

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
 * use_mask != 0 applies the -100 shift mask from the region ids stored in the plan. */
int ssw_attn_fused(const void* qkv, int dtype, int32_t heads, int32_t head_dim,
                   const ssw_plan_layout* L, const int32_t* plan,
                   const float* table, const int32_t rpb_window[3], float scale, int use_mask,
                   void* out, void* attn_vals, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SSW_B200_H */
