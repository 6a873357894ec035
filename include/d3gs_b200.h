/*
 * d3gs_b200 -- C ABI of the B200 (sm_100a) 3D-Gaussian-splatting training-step library.
 *
 * Every entry point replaces one device launch site of the reference operator
 * (d3sim/algos/d3gs/render.py, d3sim/ops/image/fused_ssim.py, d3sim/ops/optim/adam.py,
 * d3sim/algos/d3gs/origin/strategy.py) or the reference's one native module
 * (d3sim/csrc/devsort.py).  The reference launches its kernels through cumm's
 * `inliner.kernel_raw/kernel_1d` on torch's current stream with torch-allocated tensors
 * (render.py:676-681, 839-840, 883); the same contract holds here:
 *
 *   - all buffers are caller-owned device memory (plain pointers + element counts);
 *     the library never allocates or frees, workspaces are sized by *_workspace_bytes();
 *   - every call is asynchronous on the CUDA stream passed as `stream` (a cudaStream_t);
 *   - return value 0 = success, negative = error; d3gs_last_error() returns the message of the
 *     calling thread's last failure.  Device-side problems (a bounded wait that gave up) are
 *     reported through the `status` word the caller passes, never by trapping.
 *
 * Flat indexing over a view batch follows render.py:317-318, 757: i = view * num + gaussian.
 */
#ifndef D3GS_B200_H_
#define D3GS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define D3GS_MAX_VIEWS 8          /* views per launch (CameraBundle batch, render.py:129-150) */
#define D3GS_SPLAT_RECORD_FLOATS 12   /* staged splat record: [u v hx hy][ha nb hc opacity][r g b thr] */
#define D3GS_SPLAT_GRAD_FLOATS 12     /* packed per-splat raster gradient, see d3gs_raster_backward */

/* error codes */
#define D3GS_OK 0
#define D3GS_ERR_INVALID_ARGUMENT (-1)
#define D3GS_ERR_CUDA (-2)
#define D3GS_ERR_UNSUPPORTED (-3)

/* device status word bits (written by kernels whose bounded waits ran out) */
#define D3GS_STATUS_SCAN_TIMEOUT 1u
#define D3GS_STATUS_SORT_TIMEOUT 2u
#define D3GS_STATUS_COPY_TIMEOUT 4u
#define D3GS_STATUS_PEER_TIMEOUT 8u   /* another rank's flag (gradients ready / update done) did not arrive */

/* One pinhole camera: cam2world[:3].T flattened ([4,3]: rows 0..2 are the columns of the
 * camera-to-world rotation, row 3 the camera centre; render.py:136, 205-206) and intrinsics. */
typedef struct D3gsCamera {
    float cam2world_T[12];
    float fx, fy, cx, cy;
} D3gsCamera;

/* Scalar options of the operator; names and defaults follow GaussianSplatConfig
 * (d3sim/algos/d3gs/config_def.py:77-161). */
typedef struct D3gsOpConfig {
    int32_t width, height;
    int32_t tile_x, tile_y;                 /* 16 x 16 only */
    float near_plane, far_plane;            /* near / far */
    float eps;                              /* 1e-6, conic determinant guard */
    float cov2d_radii_eigen_eps;            /* 0.1 */
    float projected_clamp_factor;           /* 1.3 */
    float gaussian_std_sigma;               /* 3.0 */
    float gaussian_lowpass_filter;          /* 0.3 */
    float alpha_eps;                        /* 1/255 */
    float transmittance_eps;                /* 1e-4 */
    float scale_global;                     /* inference only */
    int32_t early_filter_algo;              /* EarlyFilterAlgo: 0 NONE, 1 AABB, 2 ELLIPSE, 3 OBB, 4 OBB_DFVT */
    int32_t sh_degree;                      /* active degree 0..3 (model.cur_sh_degree) */
    int32_t training;
    int32_t clamp_mask_reference_order;     /* 1: gate dcolor like render.py:3344-3350 */
    int32_t fused_activations;              /* 1: normalize/exp/sigmoid applied in-kernel (GaussianModelOriginFused,
                                               origin/model.py:453-462); 0: tensors are already activated */
    float bg_color[3];
    int32_t key_shift_bits;                 /* 0 or 32: key = tile << 32 | depth bits (64-bit sort keys);
                                               18: enable_32bit_sort (render.py:737, 767-770): key = tile << 18 |
                                               (uint32(depth / depth_32bit_prec) & 0x3FFFF), sorted on 32 bits */
    float depth_32bit_prec;                 /* 0.001, used with key_shift_bits == 18 */
    int32_t anti_aliasing;                  /* enable_anti_aliasing (render.py:391-406, 449-462; gs3d.py:592-619):
                                               conic = inverse of the low-passed covariance without the eps guard,
                                               opacity *= sqrt(max(2.5e-5, det(cov) / det(cov + lowpass I))) */
    int32_t inv_depth;                      /* render_inv_depth (render.py:582): ctx.depths holds 1/z, which, as in the
                                               reference, is also the value the sort keys are built from */
    int32_t num_views;                      /* B */
    D3gsCamera cameras[D3GS_MAX_VIEWS];
    /* Instance rendering (render.py:207-220, 346-354, 3031-3039), read by d3gs_preprocess_forward and
     * d3gs_preprocess_backward only.  instance_id NULL = off.  A Gaussian g with instance_id[g] >= 0 lives in the
     * frame of object instance_id[g]; for it view b's camera is taken into that frame, cam2instance =
     * inverse(instance2world[frame_ids[b]][instance_id[g]]) @ cam2world, and the rest is unchanged (gradients are
     * those of the Gaussian's parameters in its own frame; the transforms receive none, as in the reference).
     * instance2world_T: device [num_frame, num_instance, 4, 3] floats, every [4,3] laid out like cam2world_T
     * (rows 0-2 the transposed rotation, row 3 the translation); rigid transforms (the inverse rotation is the
     * transpose). */
    const int32_t* instance_id;             /* device [N] */
    const float* instance2world_T;
    int32_t num_instance;
    int32_t frame_ids[D3GS_MAX_VIEWS];      /* frame of every view (BasicPinholeCamera.frame_local_id /
                                               CameraBundle.frame_ids) */
    int32_t reserved_;
} D3gsOpConfig;

/* Gaussian parameters in the reference model layout (origin/model.py:36-44).  `sh_base` /
 * `sh_rest` with strides (in floats per Gaussian) cover both the split layout
 * (color_sh_base[N,3] + color_sh[N,15,3]) and the un-split one (color_sh[N,16,3]). */
typedef struct D3gsModel {
    int64_t num;
    const float* xyz;               /* [N,3] */
    const float* quaternion_xyzw;   /* [N,4] raw; normalised in-kernel */
    const float* scale;             /* [N,3] log-scale */
    const float* opacity;           /* [N]   logit */
    const float* sh_base;           /* l=0 coefficients */
    const float* sh_rest;           /* l>=1 coefficients, coefficient-major [.,3] */
    int32_t sh_base_stride;
    int32_t sh_rest_stride;
} D3gsModel;

typedef struct D3gsModelGrad {
    float* xyz;
    float* quaternion_xyzw;
    float* scale;
    float* opacity;
    float* sh_base;
    float* sh_rest;
    int32_t sh_base_stride;
    int32_t sh_rest_stride;
    int32_t sh_rest_floats;         /* floats of l>=1 coefficients stored per Gaussian (45 for degree 3);
                                       those above the active degree are written as zero */
    int32_t reserved;
} D3gsModelGrad;

/* Per-(view,Gaussian) context written by the preprocess and consumed downstream
 * (GaussianSplatOpContext, render.py:57-72; allocation render.py:641-665). */
typedef struct D3gsSplatContext {
    int32_t* tiles_touched;   /* [B*N] */
    int32_t* radii;           /* [B*N] */
    float* depths;            /* [B*N] */
    float* uvs;               /* [B*N,2] */
    float* conic_opacity;     /* [B*N,4] */
    float* rgb_gaussian;      /* [B*N,3] */
    float* cov2d_vecs;        /* [B*N,3] training only, may be NULL */
    uint8_t* sh_to_rgb_ne_0;  /* [B*N]   training only, may be NULL */
    uint64_t* tile_mask;      /* [B*N]   optional (may be NULL; not in the reference): the tiles the early filter
                                 accepted, as a row-major bit mask over the 3-sigma tile rect when that rect has at
                                 most 64 tiles.  Written by the preprocess, read by the key duplication, which then
                                 does not repeat the overlap tests. */
    float* records;           /* [B*N,12] optional (may be NULL; not in the reference), 16-byte aligned: the 48-byte
                                 raster record of every visible Gaussian, [u v hx hy][ha nb hc o][r g b thr].  Written
                                 by the preprocess; with it the raster kernels gather their records by sorted id and
                                 the per-pair packing pass (d3gs_pack_splats) is not needed. */
    int32_t* tile_counts;     /* [B*tiles] optional (may be NULL; not in the reference): zero-filled by the preprocess,
                                 which then adds 1 to the entry of every (view, tile) an accepted Gaussian touches:
                                 the per-tile list lengths, known before any key exists (tile-bucket binning below) */
} D3gsSplatContext;

/* ---- helpers -------------------------------------------------------------------------- */
const char* d3gs_version(void);
/* copies the calling thread's last error message; returns its length */
size_t d3gs_last_error(char* buf, size_t cap);
/* DeviceSort.get_higher_msb (csrc/devsort.py:129-149): number of bits needed for n */
int32_t d3gs_bit_length(uint32_t n);
/* Number of kernels this library has launched in the calling process since it was loaded (every entry point
 * counts its own launches; memsets and copies are not counted).  For accounting, e.g. launches per step. */
uint64_t d3gs_kernel_launch_count(void);
/* For tests of the error paths (no counterpart in the reference): every bounded wait of the kernels launched by this
 * process afterwards gives up after poll_limit polls (0 = the built-in limits), and the CTA / tile number `hold` (-1 =
 * none) withholds what a wait depends on -- its look-back flag in the scan and the sort, the bulk copy its own barrier
 * expects elsewhere.  The waiting code then sets its D3GS_STATUS_* bit and returns; nothing faults and nothing waits
 * for ever.  d3gs_test_hooks(0, -1) restores normal operation. */
void d3gs_test_hooks(uint32_t poll_limit, int32_t hold);
/* sizeof() of the ABI structs, so a binding can verify its mirror: 0 D3gsCamera, 1 D3gsOpConfig,
 * 2 D3gsModel, 3 D3gsModelGrad, 4 D3gsSplatContext, 5 D3gsAdamSegment, 6 D3gsDensifyStats, 7 D3gsPeerSet,
 * 8 D3gsRefineConfig, 9 D3gsRefineMoments, 10 D3gsPeerViews */
size_t d3gs_struct_size(int32_t which);

/* ---- K1 preprocess forward (render.py:250-681) ------------------------------------------- */
/* mask: optional [B*N] bytes, non-zero = skip (render.py:306-309).  status: optional device word;
 * D3GS_STATUS_COPY_TIMEOUT is OR-ed in when the staging copy of a CTA's SH rows did not arrive (the launch's results
 * are then invalid). */
int32_t d3gs_preprocess_forward(const D3gsOpConfig* cfg, const D3gsModel* model, const uint8_t* mask,
                                const D3gsSplatContext* ctx, uint32_t* status, void* stream);

/* ---- K2 inclusive scan of tile counts (tiles_touched.cumsum_(0), render.py:694-695) ------ */
size_t d3gs_scan_workspace_bytes(int64_t n);
/* out may alias in.  total[0] (device int64) receives the last element = num_rendered. */
int32_t d3gs_scan_tiles(const int32_t* in, int32_t* out, int64_t n, int64_t* total, void* workspace,
                        size_t workspace_bytes, uint32_t* status, void* stream);

/* ---- allocation-free scan (no counterpart in the reference) ------------------------------
 * The same scan for callers that cannot obtain device memory when they call: a host whose whole memory
 * budget belongs to another engine's pool, a frame loop that must not run into cudaMalloc's device-wide
 * synchronisation, or a thin C caller without an allocator.  The tile-status scratch is a fixed
 * 32,784-byte array inside the module (every GPU that loads the library holds it until exit), so the call
 * takes no workspace and performs no cudaMalloc/cudaFree.  Limit: n <= d3gs_scan_tiles_static_max_items()
 * = 16,777,216; larger n is rejected with an error (use d3gs_scan_tiles).  The first call on each device
 * looks up the array's device address (cudaGetSymbolAddress, with that device current): make that first
 * call before any stream capture.  All calls share the one array: calls that may overlap on the GPU
 * (different streams) race on it and must be serialised by the caller. */
int64_t d3gs_scan_tiles_static_max_items(void);
int32_t d3gs_scan_tiles_static(const int32_t* in, int32_t* out, int64_t n, int64_t* total, uint32_t* status,
                               void* stream);

/* ---- K3 key duplication (render.py:739-840) ---------------------------------------------- */
/* key = (view*tiles + y*tiles_x + x) << 32 | float_bits(depth); value = flat index i */
int32_t d3gs_duplicate_keys(const D3gsOpConfig* cfg, int64_t num, const int32_t* scan, const D3gsSplatContext* ctx,
                            uint64_t* keys, int32_t* values, void* stream);

/* ---- K4 radix sort (DeviceSort, csrc/devsort.py:26-127) ---------------------------------- */
size_t d3gs_sort_workspace_bytes(int64_t n, int32_t begin_bit, int32_t end_bit);
/* Stable LSD radix sort of (uint64 key, int32 value) pairs on bits [begin_bit,end_bit), ping-ponging
 * between the two buffer pairs like cub::DoubleBuffer.  *result_in_alt = 1 when the sorted data
 * ended in keys_alt/values_alt (the reference's key_swap/value_swap, render.py:884-887). */
int32_t d3gs_sort_pairs(uint64_t* keys, uint64_t* keys_alt, int32_t* values, int32_t* values_alt, int64_t n,
                        int32_t begin_bit, int32_t end_bit, void* workspace, size_t workspace_bytes,
                        int32_t* result_in_alt, uint32_t* status, void* stream);

/* ---- K5 tile ranges (render.py:896-939) --------------------------------------------------- */
/* ranges [num_tiles,2] int32 is zero-filled by this call, then [start,end) written per tile */
int32_t d3gs_tile_ranges(const uint64_t* sorted_keys, int64_t n, int32_t* ranges, int64_t num_tiles,
                         int32_t key_shift_bits, void* stream);

/* ---- tile-bucket binning (no counterpart in the reference; produces what render.py:739-939 produces) -----------
 * The same sorted per-tile lists and tile ranges as d3gs_duplicate_keys + d3gs_sort_pairs + d3gs_tile_ranges,
 * without a global sort: the upper key bits only name the tile, and the preprocess has already counted the pairs
 * of every tile (D3gsSplatContext.tile_counts).  Call order:
 *   d3gs_scan_tiles(tile_counts -> tile_scan, total = number of pairs)
 *   d3gs_bucket_prepare: ranges [num_tiles,2] ({0,0} for empty tiles, like d3gs_tile_ranges), cursor [num_tiles] =
 *       every tile's start, *max_count (device int64) = the longest list;
 *   (the caller reads total and max_count, allocates entries [total] uint64 and sorted_values [total] int32)
 *   d3gs_bucket_emit: one entry per pair, depth bits << 32 | flat index, at a position drawn from its tile's cursor;
 *   d3gs_bucket_sort: every tile's entries sorted in shared memory; sorted_values receives the flat indices,
 *       sorted_keys (optional, may be NULL) the reference's keys tile << 32 | depth bits.
 * Entries are unique, so their order is the reference's: by depth, ties by ascending flat index (a stable sort of
 * pairs emitted in index order).  d3gs_bucket_sort returns D3GS_ERR_UNSUPPORTED when max_count exceeds
 * d3gs_bucket_sort_capacity() (16384): take the radix-sort path for that launch.  64-bit sort keys only. */
int64_t d3gs_bucket_sort_capacity(void);
/* Launching without waiting for the counts: a caller that sizes entries / sorted_values from the PREVIOUS launch
 * passes that size as pair_capacity (> 0) to prepare and emit, and total_pairs = the device word d3gs_scan_tiles
 * wrote.  If the pairs do not fit, prepare leaves every range {0,0} and emit writes nothing, so the sort and the
 * raster kernels queued behind them touch no pair; the caller reads total and max_count when it likes and repeats
 * the chain with larger buffers.  A list longer than the classes d3gs_bucket_sort launched for its max_count
 * argument has its indices passed through in emission order (valid, unsorted): the caller compares the true
 * max_count with the one it passed and repeats.
 * pair_capacity 0 (and total_pairs NULL) = sizes are exact, no check. */
int32_t d3gs_bucket_prepare(const int32_t* tile_counts, const int32_t* tile_scan, int64_t num_tiles, int32_t* ranges,
                            int32_t* cursor, int64_t* max_count, int64_t pair_capacity, void* stream);
int32_t d3gs_bucket_emit(const D3gsOpConfig* cfg, int64_t num, const D3gsSplatContext* ctx, int32_t* cursor,
                         uint64_t* entries, const int64_t* total_pairs, int64_t pair_capacity, void* stream);
int32_t d3gs_bucket_sort(const uint64_t* entries, const int32_t* ranges, int64_t num_tiles, int64_t max_count,
                         int32_t* sorted_values, uint64_t* sorted_keys, void* stream);

/* ---- staging for the rasteriser: gather splats into sorted, contiguous 48-byte records ------
 * (replaces the per-batch gathers of render.py:1702-1716; lets the raster kernels stream their
 * tile's list with bulk async copies).  records: [n, 12] floats, 16-byte aligned. */
int32_t d3gs_pack_splats(const int32_t* sorted_values, int64_t n, const D3gsSplatContext* ctx, float alpha_eps,
                         float* records, void* stream);

/* Optional schedule for the two raster launches (no counterpart in the reference, whose grid walks the tiles
 * in index order, render.py:1380-1386): order[k] = the tile CTA k handles, tiles with the longest lists first.
 * Raster results do not depend on it. */
int32_t d3gs_tile_order(const int32_t* ranges, int64_t num_tiles, int32_t* order, void* stream);

/* ---- K6 raster forward (render.py:1329-2316, is_bwd=False) ------------------------------- */
/* color [B,H,W,3] (NHWC), final_T [B,H,W], n_contrib [B,H,W]; tile_order [B*tiles] from d3gs_tile_order or NULL.
 * records: with sorted_values == NULL the per-pair records of d3gs_pack_splats, in list order; with
 * sorted_values (the sorted value list of the sort) the per-Gaussian table D3gsSplatContext.records, from
 * which the kernel gathers by id, like the reference's per-batch gathers (render.py:1702-1716). */
int32_t d3gs_raster_forward(const D3gsOpConfig* cfg, const int32_t* ranges, const int32_t* tile_order,
                            const float* records, const int32_t* sorted_values, float* color, float* final_T,
                            int32_t* n_contrib, uint32_t* status, void* stream);

/* ---- K7 raster backward (render.py:1589-1676, 1774-2210) -------------------------------- */
/* drgb [B,H,W,3], dT [B,H,W] or NULL.  The reference's four per-splat gradient tensors (duv, dconic,
 * dopacity, dcolor, render.py:1388-1401) are one packed array here so that the kernel can use 16-byte
 * vector atomics: splat_grads [B*N, 12] = {dconic a,b,c, dopacity | dcolor r,g,b, dz | duv x,y, 0, 0},
 * 16-byte aligned, zero-filled by this call.  sorted_values: the sorted value list of the sort.
 * mode: bit flags.  D3GS_RASTER_RECORDS_BY_ID: records is the per-Gaussian table (see d3gs_raster_forward), else
 * the per-pair records.  D3GS_RASTER_DIRECT_ATOMICS: every group of four lanes adds its sums for a splat to
 * splat_grads directly instead of accumulating them per tile in shared memory first; faster while a splat
 * overlaps few 4x2 pixel blocks of a tile (about three sort pairs per Gaussian or fewer), slower for scenes of
 * large splats.  Same gradients up to the order of the float additions.
 * atomic_counts: NULL, or two device uint64 that the call ADDS to (the caller zeroes them) -- the reference's
 * measure_atomic_add_count (config_def.py:134; render.py:1451-1453, 2145-2148): [0] groups of global atomic adds
 * issued, one per Gaussian that a reducing lane set (4 lanes = 4x2 pixels with DIRECT_ATOMICS, else a whole tile's
 * flush) adds to; [1] warp passes that had a valid pixel (in a pass each of the warp's eight lane groups handles
 * the next splat of its own survivor list).  Non-NULL selects an instrumented instance of the kernel: same
 * gradients, slower. */
#define D3GS_RASTER_RECORDS_BY_ID 1
#define D3GS_RASTER_DIRECT_ATOMICS 2
int32_t d3gs_raster_backward(const D3gsOpConfig* cfg, int64_t num, const int32_t* ranges, const int32_t* tile_order,
                             const float* records, int32_t mode, const int32_t* sorted_values, const float* color,
                             const float* final_T, const int32_t* n_contrib, const float* drgb, const float* dT,
                             float* splat_grads, uint64_t* atomic_counts, uint32_t* status, void* stream);

/* ---- K8 preprocess backward (render.py:2779-3374) ---------------------------------------- */
/* every gradient element is written (zeros for culled Gaussians); sums over the view batch.  Slot 7 of a
 * splat_grads row (zero after d3gs_raster_backward) is dz, the gradient of the splat's depth value when a
 * depth image was rendered (render.py:3053-3057): it joins the camera-space z gradient. */
/* status: optional device word; D3GS_STATUS_COPY_TIMEOUT is OR-ed in when the staging copy of a CTA's SH rows did not
 * arrive (that CTA then writes no gradient). */
int32_t d3gs_preprocess_backward(const D3gsOpConfig* cfg, const D3gsModel* model, const D3gsSplatContext* ctx,
                                 const float* splat_grads, const D3gsModelGrad* grad, uint32_t* status, void* stream);

/* ---- K9/K10 SSIM map and fused L1 + D-SSIM (fused_ssim.py:93-416, losses.py:19-20) ---------- */
/* ssim map forward: x NHWC or NCHW [B,3,H,W]/[B,H,W,3], y NCHW; outputs NCHW; dmu* may be NULL */
int32_t d3gs_ssim_forward(const float* x, const float* y, int32_t batch, int32_t height, int32_t width,
                          int32_t x_is_nhwc, float* ssim_map, float* dmu1, float* dmu11, float* dmu12,
                          void* stream);
int32_t d3gs_ssim_backward(const float* dssim_map, const float* dmu1, const float* dmu11, const float* dmu12,
                           const float* x, const float* y, int32_t batch, int32_t height, int32_t width,
                           int32_t x_is_nhwc, float* dx, void* stream);
/* loss = (1-lambda)*mean|x-y| + lambda*(1-mean(SSIM)) for x NHWC (the op's colour) and y NCHW;
 * sums[0..1] (device doubles: sum|x-y|, sum SSIM) are zeroed and accumulated; dx NHWC receives
 * grad_scale * dloss/dx.  scratch: 3*B*3*H*W floats. */
size_t d3gs_l1_dssim_scratch_bytes(int32_t batch, int32_t height, int32_t width);
int32_t d3gs_l1_dssim_forward_backward(const float* x, const float* y, int32_t batch, int32_t height,
                                       int32_t width, float lambda_dssim, float grad_scale, double* sums,
                                       float* dx, void* scratch, size_t scratch_bytes, void* stream);

/* ---- K11 + K12 fused Adam and densification statistics ------------------------------------
 * (adam.py:32-148, 382-418; csrc/optim.py:22-49; origin/strategy.py:93-122) */
typedef struct D3gsAdamSegment {
    float* param;
    const float* grad;
    float* exp_avg;
    float* exp_avg_sq;
    int64_t count;
    float lr, beta1, beta2, eps;
    float bias_correction1, bias_correction2_sqrt;   /* host doubles rounded to float, adam.py:55-57 */
    float grad_scale, weight_decay;
} D3gsAdamSegment;

typedef struct D3gsDensifyStats {
    const float* duv;          /* (view, Gaussian) pair k at duv + k*duv_stride: 2 floats */
    const int32_t* radii;      /* [B*N] */
    float* duv_ndc_length;     /* [N] */
    float* count;              /* [N] */
    float* max_radii;          /* [N] */
    int64_t num;
    int32_t batch, width, height, need_max_radii;
    int32_t loss_batch;        /* views the loss was averaged over (duv is scaled back by it,
                                  origin/strategy.py:105-106); 0 = same as batch.  Larger than batch when the
                                  view batch is spread over several GPUs. */
    int32_t duv_stride;        /* floats between consecutive pairs: 2 for a dense [B,N,2] tensor, 12 when duv is
                                  read in place from splat_grads + 8; 0 = 2 */
} D3gsDensifyStats;

/* one launch over up to 8 parameter tensors; stats may be NULL */
int32_t d3gs_adam_stats_step(const D3gsAdamSegment* segments, int32_t num_segments, const D3gsDensifyStats* stats,
                             void* stream);
int32_t d3gs_densify_stats(const D3gsDensifyStats* stats, void* stream);

/* K8 + K11 in one launch for single-GPU, single-view training: the preprocess backward applies Adam to the
 * 59 floats of every Gaussian as it produces their gradient, so the gradient tensors of
 * d3gs_preprocess_backward are never written or read (render.py:3176-3360 followed by adam.py:382-418).
 * segments[0..5] = xyz, quaternion_xyzw, scale, opacity, sh_base, sh_rest in this order; segment.param must be
 * the model's tensor (updated in place), segment.count its element count, segment.grad is ignored.  Needs the
 * split degree-3 layout (sh_base_stride 3, sh_rest_stride 45) and cfg->num_views == 1.  stats (may be NULL):
 * the densification statistics of the same iteration, accumulated by the same launch.
 * status: as for d3gs_preprocess_backward; a CTA whose copy did not arrive takes no optimizer step. */
int32_t d3gs_preprocess_backward_adam(const D3gsOpConfig* cfg, const D3gsModel* model, const D3gsSplatContext* ctx,
                                      const float* splat_grads, const D3gsAdamSegment* segments,
                                      const D3gsDensifyStats* stats, uint32_t* status, void* stream);

/* ---- data-parallel update over peer memory (no counterpart in the reference, which trains on one GPU;
 * the batch semantics it implements are those of train.py:170-172 and tools.py:146-163) ------------
 * Every rank (one process per GPU) renders its own view and holds the full model.  The flat gradient
 * and parameter buffers of all ranks live in buffers that each process has mapped (CUDA IPC, NVLink
 * peer access).  A rank owns one slice of the parameters with its Adam moments; one launch
 *   - reads that slice of EVERY rank's gradient buffer (bulk async copies into shared memory, so that
 *     enough bytes are in flight to cover the latency of the links) and adds them in rank order,
 *   - applies Adam to the slice,
 *   - writes the new parameters into EVERY rank's parameter buffer (peer stores),
 * so gradients and parameters cross NVLink in opposite directions at the same time and never make a
 * second trip through HBM.  The kernel does not wait for other ranks: the caller orders the launches with
 * a collective barrier before (all gradients written) and after (all parameters written).
 * Segments: param points into param[rank], grad into grad[rank]; their element offsets are applied to
 * every peer's buffer. */
#define D3GS_MAX_PEERS 8
typedef struct D3gsPeerSet {
    int32_t world, rank;
    const float* grad[D3GS_MAX_PEERS];   /* each rank's flat gradient buffer as mapped in this process */
    float* param[D3GS_MAX_PEERS];        /* each rank's flat parameter buffer as mapped in this process */
    uint32_t* status;                    /* optional device word: D3GS_STATUS_COPY_TIMEOUT is OR-ed in when a
                                            staged copy did not arrive in time (that chunk is left unchanged) */
    /* Optional: multicast addresses of the SAME buffers (a switch multicast mapping over all ranks' copies, e.g.
     * torch symmetric memory's multicast_ptr).  With them the launch takes the path through the NVLink switch: one
     * multimem.ld_reduce per gradient element (the switch adds the ranks' copies) and one multimem.st per new
     * parameter, so that S/world + S bytes enter and leave every GPU instead of 2 (world-1)/world S. */
    const float* grad_mc;
    float* param_mc;
    /* Optional: ordering inside the launch instead of by the caller's collectives.  flags[q] = rank q's block of
     * D3GS_PEER_FLAG_WORDS uint32 words as mapped in this process (zero-filled once, before the first launch);
     * epoch = number of this launch: 1, 2, 3, ... the same on every rank.  A launch then (1) announces "my
     * gradients are complete" to all ranks and waits for everybody's announcement before it reads, (2) after its
     * last store announces "done" with its status bits and waits for everybody's, so that when the kernel ends the
     * whole parameter buffer of this rank is up to date.  Every rank must launch epoch e before any rank can
     * finish it; a wait gives up after wait_limit polls (0 = a default of seconds) and sets
     * D3GS_STATUS_PEER_TIMEOUT, and a status bit set on any rank is OR-ed into every rank's status word.
     * With flags[0] == NULL the caller orders the launches as described above. */
    uint32_t* flags[D3GS_MAX_PEERS];
    uint32_t epoch;
    uint32_t wait_limit;
    /* d3gs_preprocess_backward_adam_peers only: lanes that share one Gaussian, each taking every
     * lanes_per_gaussian-th view, so that the loads from several ranks are in flight together: 1, 2 or 4;
     * 0 = chosen by the library (4 from eight ranks on, 2 from four, else 1) */
    int32_t lanes_per_gaussian;
    int32_t reserved_;
} D3gsPeerSet;
#define D3GS_PEER_FLAG_WORDS 32
int32_t d3gs_adam_stats_step_peers(const D3gsAdamSegment* segments, int32_t num_segments,
                                   const D3gsDensifyStats* stats, const D3gsPeerSet* peers, void* stream);

/* K8 + gradient sum over the ranks + K11 + parameter broadcast in ONE launch (no counterpart in the reference; batch
 * semantics of train.py:170-172, render.py:3182-3199).  One view per rank.  Rank r owns the Gaussians
 * [g_begin, g_begin + g_count) and their Adam moments.  Its launch reads, for those Gaussians, EVERY rank's per-splat
 * raster gradients and context (views->...[b] = rank b's buffers of ITS view, each indexed by the Gaussian, as mapped
 * in this process), runs the backward through projection and SH for all views (cfg->cameras[b] = rank b's camera,
 * cfg->num_views = world), sums over the views in registers, applies Adam and stores the new parameters into every
 * rank's flat parameter buffer (peers->param[q]; model's tensors lie inside peers->param[rank]).  The parameter
 * gradient (236 bytes per Gaussian) is never formed: per Gaussian and peer 65 bytes come in over NVLink instead of
 * 236, and the backward arithmetic overlaps the transfers.  segments[0..5]: xyz, quaternion_xyzw, scale, opacity,
 * sh_base, sh_rest; param = the model's tensor + g_begin * floats-per-Gaussian, count = floats-per-Gaussian * g_count,
 * exp_avg / exp_avg_sq = this rank's moments for its share.  peers->flags / epoch / wait_limit order the ranks'
 * launches as for d3gs_adam_stats_step_peers (with flags[0] == NULL the caller does); peers->grad is not used.
 * stats (may be NULL): the densification statistics of the rank's Gaussians over ALL views are accumulated in the
 * same launch (duv_ndc_length, count, max_radii indexed by the Gaussian; width, height, loss_batch, need_max_radii as
 * usual; duv and radii are not read -- the views carry them), i.e. already summed over the ranks, for the rank's own
 * range only.  g_begin must be a multiple of 4.  Every rank must launch, also with g_count == 0. */
typedef struct D3gsPeerViews {
    const float* splat_grads[D3GS_MAX_PEERS];        /* [N,12] packed raster gradients of rank b's view */
    const int32_t* radii[D3GS_MAX_PEERS];            /* [N] */
    const float* cov2d_vecs[D3GS_MAX_PEERS];         /* [N,3] */
    const uint8_t* sh_to_rgb_ne_0[D3GS_MAX_PEERS];   /* [N] */
} D3gsPeerViews;
int32_t d3gs_preprocess_backward_adam_peers(const D3gsOpConfig* cfg, const D3gsModel* model, const D3gsPeerViews* views,
                                            int64_t g_begin, int64_t g_count, const D3gsAdamSegment* segments,
                                            const D3gsDensifyStats* stats, const D3gsPeerSet* peers, void* stream);

/* Buffers another process on the same node can map.  create: cudaMalloc on the current device, zero-filled,
 * plus a 64-byte handle to send to the peers; open: map a peer's buffer into this process (enables peer
 * access to its device); close / destroy release a mapping / the allocation.  Not for the per-step path:
 * all four synchronise the device. */
#define D3GS_PEER_HANDLE_BYTES 64
int32_t d3gs_peer_buffer_create(int64_t bytes, void** ptr, void* handle);
int32_t d3gs_peer_buffer_open(const void* handle, void** ptr);
int32_t d3gs_peer_buffer_close(void* ptr);
int32_t d3gs_peer_buffer_destroy(void* ptr);

/* ---- densification, pruning, opacity reset (origin/strategy.py:159-363, strategy.py:131-202,
 * origin/trainer.py:388-417): the step that follows every refine_every-th training iteration ----------
 * d3gs_refine_classify applies the reference's tests to every Gaussian and writes
 *   columns [4][N] int32: keep (not pruned), duplicate that is kept, split whose two children are kept, split;
 *   flags   [N] uint8: bit0 duplicate, bit1 split, bit2 pruned, bit3 split children pruned.
 * The caller scans each column (d3gs_scan_tiles), reads the four totals {keep, dup, split_kept, split},
 * allocates the new model of keep + dup + 2*split_kept Gaussians and 2*split unit normals (the reference draws
 * them with torch.randn, strategy.py:286), and calls d3gs_refine_apply, which writes the output rows in the
 * reference's order [survivors | duplicates | first split copies | second split copies]: parameters copied,
 * split children moved to R(q)(normal*scale) + xyz with scale/1.6, Adam moments gathered for survivors and
 * zero for new Gaussians, src_index (optional) = source Gaussian of every output row. */
typedef struct D3gsRefineConfig {
    float prune_opacity_thresh, grow_grad2d, grow_scale3d, grow_scale2d, prune_scale3d, prune_scale2d;
    float scene_scale;
    int32_t prune_too_big;      /* step > reset_opacity_every (strategy.py:178) */
    int32_t refine_by_radii;    /* step < refine_scale2d_stop_iter (strategy.py:177) */
    int32_t fused_activations;  /* the model stores raw scale / opacity / quaternion (GaussianModelOriginFused) */
} D3gsRefineConfig;

typedef struct D3gsRefineMoments {  /* per field xyz, quaternion, scale, opacity, sh_base, sh_rest; NULL = skip */
    const float* exp_avg_src[6];
    const float* exp_avg_sq_src[6];
    float* exp_avg_dst[6];
    float* exp_avg_sq_dst[6];
} D3gsRefineMoments;

int32_t d3gs_refine_classify(const D3gsModel* model, const D3gsRefineConfig* rc, const float* duv_ndc_length,
                             const float* count, const float* max_radii, int32_t* columns, uint8_t* flags,
                             void* stream);
/* dst's tensors are written (the struct's const qualifiers describe the other entry points); scans = the
 * inclusive scans of columns; totals = host array of the four totals; moments may be NULL */
int32_t d3gs_refine_apply(const D3gsModel* src, const D3gsModel* dst, const D3gsRefineConfig* rc,
                          const D3gsRefineMoments* moments, const int32_t* scans, const uint8_t* flags,
                          const float* normals, const int64_t* totals, int32_t* src_index, void* stream);
/* opacity = logit(min(activated opacity, thresh)) in place; the given Adam moments of opacity are zeroed */
int32_t d3gs_reset_opacity(float* opacity, int64_t num, float thresh, int32_t fused_activations, float* exp_avg,
                           float* exp_avg_sq, void* stream);

/* ---- sparse_mode (config_def.py:119; render.py:235-238, 478-499, 622-637, 2860-2903) ---------------------------------
 * The tensors kept between forward and backward hold the visible (view, Gaussian) items only, in flat-index order
 * (the reference: in the arrival order of an atomic counter), with gaussian_ids / batch_ids naming every kept item
 * (GaussianSplatOutput.sparse_gaussian_ids / sparse_batch_ids).  Forward, after the dense pipeline:
 *   d3gs_sparse_flags(radii, N, B, 0, flags)            flags[i] = radii[i] != 0 over the B*N items
 *   d3gs_scan_tiles(flags -> scan, total = kept)        (one read of `kept`, like render.py:635)
 *   d3gs_sparse_compact(dense ctx, N, B, scan, compact ctx, gaussian_ids, batch_ids)   radii, depths, uvs,
 *       conic_opacity, rgb_gaussian and, where both contexts hold them, cov2d_vecs, sh_to_rgb_ne_0, records
 *   d3gs_sparse_remap(sorted_values, K, scan)           sorted indices -> rows of the compact tensors
 * The raster kernels then run on the compact records unchanged.  Backward: d3gs_raster_backward on the compact
 * tensors, d3gs_sparse_expand (rows back to zero-filled dense radii / cov2d_vecs / sh_to_rgb_ne_0 / splat_grads),
 * d3gs_preprocess_backward on those, then the gradient rows of the Gaussians some view saw:
 *   d3gs_sparse_flags(dense radii, N, B, 1, flags) ; scan ; d3gs_flagged_indices -> unique ids (ascending) ;
 *   d3gs_gather_rows per gradient tensor. */
int32_t d3gs_sparse_flags(const int32_t* radii, int64_t num, int32_t views, int32_t per_gaussian, int32_t* flags,
                          void* stream);
int32_t d3gs_sparse_compact(const D3gsSplatContext* dense, int64_t num, int32_t views, const int32_t* scan,
                            const D3gsSplatContext* compact, int32_t* gaussian_ids, int32_t* batch_ids, void* stream);
int32_t d3gs_sparse_remap(int32_t* sorted_values, int64_t n, const int32_t* scan, void* stream);
int32_t d3gs_sparse_expand(int64_t kept, int64_t num, int32_t views, const int32_t* gaussian_ids,
                           const int32_t* batch_ids, const int32_t* radii, const float* cov2d_vecs,
                           const uint8_t* sh_to_rgb_ne_0, const float* splat_grads, int32_t* dense_radii,
                           float* dense_cov2d_vecs, uint8_t* dense_sh_to_rgb_ne_0, float* dense_splat_grads,
                           void* stream);
int32_t d3gs_flagged_indices(const int32_t* flags, const int32_t* scan, int64_t count, int32_t* out, void* stream);
int32_t d3gs_gather_rows(const float* src, int32_t row_floats, const int32_t* index, int64_t rows, float* dst,
                         void* stream);

/* ---- k nearest neighbours of a point cloud (d3sim/algos/d3gs/ops.py:14-183 simple_knn) --------------------------
 * out [n, k] = distances (not squared) from every point to its k nearest OTHER points, ascending; exact.  Used for
 * the initial scales (origin/model.py:26-28: the mean of the three squared distances).  points: n rows of
 * point_stride floats (xyz first); points_min / points_max: [3] on the device (the reference computes them with
 * torch, ops.py:21-22); morton_bits 10 (32-bit codes) or 21 (use_64bit); k in [1, 8].  The workspace holds the
 * codes, the sort's buffers, the sorted points and the box bounds. */
size_t d3gs_simple_knn_workspace_bytes(int64_t n, int32_t morton_bits);
int32_t d3gs_simple_knn(const float* points, int64_t point_stride, int64_t n, int32_t k, int32_t morton_bits,
                        const float* points_min, const float* points_max, float* out, void* workspace,
                        size_t workspace_bytes, uint32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* D3GS_B200_H_ */
