/*
 * fda_b200.h -- C ABI of the B200 (sm_100a) Flash Deformable 3D Attention kernels.
 *
 * Plain pointers and sizes only: every pointer is a DEVICE pointer unless its
 * comment says otherwise; `stream` is a cudaStream_t passed as void*; every
 * call is asynchronous on that stream and returns an fda_status_t.  The
 * library keeps no per-call state and allocates no device memory; the caller
 * provides outputs and (for the backward pass) a workspace.
 *
 * Tensor layouts (all dense / contiguous):
 *   value                 [batch][num_value][num_heads][head_dim]      value_dtype
 *                         num_value = sum_l D_l*H_l*W_l, level-major, cells (z,y,x) row-major
 *   spatial_shapes        [num_levels][3] = (D_l, H_l, W_l)            int64, device
 *   level_start_index     [num_levels]    first cell of each level      int64, device
 *   sampling_loc_attn     [batch][num_query][num_heads][num_levels*num_points*4]   packed_dtype
 *                         planar per (b,q,g): num_levels*num_points*3 normalised coordinates
 *                         (x,y,z per point, level-major) followed by num_levels*num_points raw
 *                         logits; soft-max over the logits happens inside the operator.
 *   output / grad_output  [batch][num_query][num_heads*head_dim]       value_dtype
 *   grad_value            like value                                   value_dtype
 *   grad_sampling_loc_attn like sampling_loc_attn                      packed_dtype
 *
 * Supported envelope: num_levels 1..5, num_points in {4, 8} (as the reference's
 * launch ladders, csrc/cuda/flash_deform_im2col_cuda.cuh:335-379,548-593),
 * head_dim a multiple of 16 bytes worth of elements (8 for 16-bit, 4 for fp32) with
 * head_dim*sizeof(value) <= 512, value_dtype in {f32, f16, bf16}; packed_dtype equal to
 * value_dtype (the reference's only form) or f32 beside a 16-bit value.
 */
#ifndef FDA_B200_H_
#define FDA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum fda_dtype {
    FDA_DTYPE_F32 = 0,
    FDA_DTYPE_F16 = 1,
    FDA_DTYPE_BF16 = 2
} fda_dtype_t;

typedef enum fda_status {
    FDA_OK = 0,
    FDA_ERR_NULL_POINTER = 1,
    FDA_ERR_BAD_DTYPE = 2,        /* unknown dtype, or a packed/value dtype pair outside the envelope */
    FDA_ERR_BAD_LEVELS = 3,       /* num_levels outside 1..5 */
    FDA_ERR_BAD_POINTS = 4,       /* num_points not 4 or 8 */
    FDA_ERR_BAD_HEAD_DIM = 5,     /* head_dim not a multiple of a 16-byte vector, or head row > 512 bytes */
    FDA_ERR_BAD_SHAPE = 6,        /* a non-positive dimension, or a tensor too large for the index width */
    FDA_ERR_IM2COL_STEP = 7,      /* batch % min(batch, im2col_step) != 0 */
    FDA_ERR_WORKSPACE = 8,        /* workspace missing or smaller than fda_backward_workspace_bytes() */
    FDA_ERR_MISALIGNED = 9,       /* a tensor base address is not 16-byte aligned */
    FDA_ERR_CUDA = 10,            /* a CUDA runtime call or the kernel launch failed; see fda_last_cuda_error() */
    FDA_ERR_TOO_LARGE_STATIC = 11 /* problem exceeds a compiled-in capacity */
} fda_status_t;

/* Human-readable name of a status code (static storage, never NULL). */
const char *fda_status_string(int status);

/* cudaError_t (as int) of the last failing CUDA call made by this library on the calling thread. */
int fda_last_cuda_error(void);

/* ABI version: major*1000 + minor. */
int fda_version(void);

/*
 * Forward:  output[b,q,g,:] = sum_i softmax(logits)_i * trilinear(value[b, level(i)], loc_i)[g,:]
 *
 * Replaces the reference launcher flash_deformable_im2col_cuda(stream, data_value,
 * data_spatial_shapes, data_level_start_index, data_sampling_loc_attn, data_col, batch_size,
 * spatial_size, num_heads, channels, num_levels, num_query, num_point, d_stride, block_thread,
 * use_reg) -- csrc/cuda/flash_deform_im2col_cuda.cuh:548-593 -- and the chunk loop around it in
 * flash_deform_attn_cuda_forward, csrc/cuda/flash_deform_attn_cuda.cu:46-88.
 *
 * im2col_step is validated exactly as there (batch % min(batch, im2col_step) == 0) and otherwise
 * unused: the whole batch is one launch.  d_stride and block_thread are the reference's launch
 * hints; they are accepted and ignored.  use_reg != 0 lets the library choose between its
 * register-staged and shared-memory-staged kernels per shape; use_reg == 0 forces the
 * shared-memory-staged kernel (the reference's meaning of the flag).
 * Every element of output is written (no pre-zeroing needed).
 */
int fda_forward(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                const void *sampling_loc_attn, void *output,
                int batch, int num_value, int num_heads, int head_dim, int num_levels,
                int num_query, int num_points, int value_dtype, int packed_dtype,
                int im2col_step, int d_stride, int block_thread, int use_reg, void *stream);

/*
 * Bytes of device workspace fda_backward needs for this problem: the fp32 accumulation image of
 * grad_value for 16-bit values (batch*num_value*num_heads*head_dim*4, rounded up to 256; none for
 * an fp32 value, which accumulates in place) plus, when the slab-binned path applies,
 * fda_backward_scratch_bytes().
 */
size_t fda_backward_workspace_bytes(int batch, int num_value, int num_heads, int head_dim, int num_levels, int num_query,
                                    int num_points, int value_dtype, int packed_dtype);

/*
 * Bytes of scratch for the backward launches that hand work to one another:
 *   - the slab-binned handling of the largest pyramid level: slab counters plus one 8-byte entry per
 *     (row, point) of one level; 0 when binning cannot pay off (the gradient image of one batch
 *     element fits the device's L2 budget) or is switched off (FDA_BINNING=0);
 *   - for 16-bit offsets/logits, an fp32 plane [batch][num_query*num_heads][num_levels*num_points]
 *     that carries the raw logit gradients from launch to launch unrounded (with fp32 offsets the
 *     logit slots of grad_sampling_loc_attn serve, bit for bit).
 * Without scratch the backward still works, through the plain scatter kernel alone.
 */
size_t fda_backward_scratch_bytes(int batch, int num_value, int num_heads, int head_dim, int num_levels, int num_query,
                                  int num_points, int packed_dtype);

/*
 * The cell-sorted backward (all points sorted by the cell they fall in; gathers and reductions once per run of equal
 * cells instead of once per point) applies to 16-bit values with 32 channels per head and enough points to pay for
 * its extra launches (FDA_BWD_SORT: 0 off, 1 by size, 2 always).  It needs more scratch than the slab-binned path:
 * fda_backward_sorted_scratch_bytes() (0 when it does not apply).  A caller that wants whichever path the library
 * prefers passes max(fda_backward_scratch_bytes, fda_backward_sorted_scratch_bytes) bytes; fda_backward_workspace_bytes
 * already includes it.  fda_backward_path tells which path such a call takes: 0 the plain scatter kernel, 1 the
 * slab-binned path for the largest level, 2 the cell-sorted path.  No counterpart in the reference.
 */
size_t fda_backward_sorted_scratch_bytes(int batch, int num_value, int num_heads, int head_dim, int num_levels, int num_query,
                                         int num_points, int value_dtype);

/*
 * Heads per group of the forward's row order for this problem: num_heads = plain row order (query by query); a smaller
 * divisor of num_heads = the grid walks all queries for that many heads at a time, so that the value rows it gathers stay
 * L2-resident (chosen when one batch element's value volume exceeds the L2 budget and the call is large;
 * FDA_FWD_HEAD_GROUPS).  Outputs do not depend on it.  Diagnostic; no counterpart in the reference.
 */
int fda_forward_head_group(int num_value, int num_heads, int head_dim, int num_levels, int num_query, int num_points,
                           int value_dtype);
int fda_backward_path(int batch, int num_value, int num_heads, int head_dim, int num_levels, int num_query, int num_points,
                      int value_dtype);

/*
 * The library reads its tuning knobs (FDA_* environment variables) once, when it is loaded;
 * fda_reload_config re-reads them.  Not thread-safe against concurrent launches.
 */
void fda_reload_config(void);

/*
 * Backward: grad_value (scatter-add of softmax_i * w_corner * grad_output through fp32 vector
 * reductions, then one cast pass for 16-bit values) and grad_sampling_loc_attn (coordinate
 * gradients and gradients w.r.t. the raw logits, written once each in packed_dtype).
 *
 * Replaces flash_deformable_col2im_cuda(stream, data_value, data_spatial_shapes,
 * data_level_start_index, data_sampling_loc_attn, grad_output, batch_size, spatial_size, num_heads,
 * channels, num_levels, num_query, num_point, grad_value, grad_sampling_loc, d_stride,
 * block_thread) -- csrc/cuda/flash_deform_col2im_cuda.cuh:689-731 -- together with the zero-fill,
 * chunk loop and cast-back of flash_deform_attn_cuda_backward, csrc/cuda/flash_deform_attn_cuda.cu:125-178.
 *
 * The library zero-fills what it accumulates into (workspace, or grad_value for fp32); both
 * outputs are fully written.  workspace must be 256-byte aligned and at least
 * fda_backward_workspace_bytes() long; it may be NULL when that is 0.  When the gradient image
 * of one batch element does not fit L2, the largest level is processed slab by slab (its points
 * are first sorted into z-slabs in the workspace) so that its part of the image stays L2-resident.
 */
int fda_backward(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                 const void *sampling_loc_attn, const void *grad_output,
                 void *grad_value, void *grad_sampling_loc_attn,
                 void *workspace, size_t workspace_bytes,
                 int batch, int num_value, int num_heads, int head_dim, int num_levels,
                 int num_query, int num_points, int value_dtype, int packed_dtype,
                 int im2col_step, int d_stride, int block_thread, void *stream);

/*
 * The two halves of fda_backward for callers that reduce the fp32 accumulation image across
 * devices before the cast (queries sharded over GPUs, value replicated): fda_backward_accumulate
 * zero-fills `accum` (fp32, value's shape) and scatter-adds into it, and writes
 * grad_sampling_loc_attn; fda_cast_grad_value converts an fp32 image to value_dtype.
 * Between the two the caller may sum `accum` over ranks.  No counterpart in the reference (it
 * has no multi-device path); semantics are those of fda_backward split at the cast.
 */
int fda_backward_accumulate(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                            const void *sampling_loc_attn, const void *grad_output,
                            float *accum, void *grad_sampling_loc_attn,
                            int batch, int num_value, int num_heads, int head_dim, int num_levels,
                            int num_query, int num_points, int value_dtype, int packed_dtype,
                            int im2col_step, void *stream);

int fda_cast_grad_value(const float *accum, void *grad_value, size_t num_elements, int value_dtype, void *stream);

/*
 * fda_backward_accumulate restricted to the pyramid levels [level_begin, level_end), so that a
 * multi-GPU caller can finish (and start exchanging) the largest level's part of the image while
 * the other levels are still computed.  Launches over disjoint level ranges that together cover
 * all levels, issued in stream order over the same buffers, give the result of one full call:
 *   first launch   flags = FDA_BWD_ZERO_IMAGE                    (zero-fill the whole image first)
 *   middle launch  flags = FDA_BWD_RESUME
 *   last launch    flags = FDA_BWD_RESUME | FDA_BWD_FINALIZE
 * (a single launch over all levels uses FDA_BWD_ZERO_IMAGE | FDA_BWD_FINALIZE).  Between launches
 * grad_sampling_loc_attn holds intermediate values; it is final after the FINALIZE launch.
 * scratch (256-byte aligned, may be NULL): with fda_backward_scratch_bytes() bytes it enables the
 * slab-binned path for the largest level when it is part of the range, and keeps the logit
 * gradients handed from launch to launch in fp32 when the offsets are 16-bit (without it they pass
 * through grad_sampling_loc_attn and are rounded to 16 bits once more on the way); with at least
 * fda_backward_sorted_scratch_bytes() bytes (when that is not 0) the launches take the cell-sorted
 * path instead: the first launch of a sequence (no FDA_BWD_RESUME) sorts the points of all levels
 * into the scratch, every launch walks its levels' part of the list, the FDA_BWD_FINALIZE launch
 * writes grad_sampling_loc_attn (it holds nothing meaningful before).  Pass the same scratch to
 * every launch of a sequence.
 * No counterpart in the reference.
 */
#define FDA_BWD_ZERO_IMAGE 1
#define FDA_BWD_RESUME 2
#define FDA_BWD_FINALIZE 4
#define FDA_BWD_BINNED_DONE 8 /* the largest level was already scattered with fda_backward_binned_part */
#define FDA_BWD_ZERO_TOUCHED 16 /* in place of FDA_BWD_ZERO_IMAGE: zero only the rows that points touch (see below) */
int fda_backward_accumulate_levels(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                                   const void *sampling_loc_attn, const void *grad_output,
                                   float *accum, void *grad_sampling_loc_attn,
                                   int batch, int num_value, int num_heads, int head_dim, int num_levels,
                                   int num_query, int num_points, int value_dtype, int packed_dtype,
                                   int im2col_step, int level_begin, int level_end, int flags,
                                   void *scratch, size_t scratch_bytes, void *stream);

/*
 * Sparse handling of the fp32 image, for calls whose sampling points reach only a part of the value
 * volume (a few hundred queries looking into a large volume).  FDA_BWD_ZERO_TOUCHED on the first
 * launch of a sequence zeroes, from the point list, exactly the image rows that the scatter can
 * touch -- the 8 corner cells of every point of every level, one head row each -- and leaves the
 * rest of the image as it is (it may hold anything).  Such an image must not be converted with
 * fda_cast_grad_value, which reads all of it; fda_cast_grad_value_touched zero-fills grad_value and
 * converts the same rows from the same point list.  With an fp32 value (image == grad_value) the
 * flag acts as FDA_BWD_ZERO_IMAGE, and fda_cast_grad_value_touched returns FDA_ERR_BAD_DTYPE.
 * fda_backward_touched_rows returns 1 when fda_backward itself works this way for a problem
 * (FDA_BWD_TOUCHED: 0 never, 1 when the points can touch at most 60 % of the image -- 8 corner rows
 * per point against num_value rows per head --, 2 always; never for a problem that
 * fda_backward_path sends down the cell-sorted path), so that a caller composing the backward
 * from the entry points above can follow the same rule.  The scatter adds the same terms to the same
 * zeros either way.
 * No counterpart in the reference (its grad_value is a zero-filled tensor in the value dtype that
 * the kernel adds to, csrc/cuda/flash_deform_attn_cuda.cu:145).
 */
int fda_backward_touched_rows(int batch, int num_value, int num_heads, int head_dim, int num_levels, int num_query,
                              int num_points, int value_dtype);
int fda_cast_grad_value_touched(const float *accum, void *grad_value, const int64_t *spatial_shapes,
                                const int64_t *level_start_index, const void *sampling_loc_attn,
                                int batch, int num_value, int num_heads, int head_dim, int num_levels,
                                int num_query, int num_points, int value_dtype, int packed_dtype, void *stream);

/*
 * The slab-binned scatter of the largest level in `parts` launches, so that a multi-GPU caller can
 * exchange the z-range of the image that a launch has finished while the next launch runs.
 * fda_backward_bin_plan answers, from a HOST copy of spatial_shapes, whether binning applies to a
 * problem (return value 1) and how: the level, its number of slabs S and planes per slab `depth`.
 * Launch `part` (0-based) covers slabs [S*part/parts, S*(part+1)/parts); after it, the image planes
 * [first_slab*depth, min(last_slab_end*depth, D_level)) of that level are final (the plane above is
 * still written by the next slab).  Part 0 also builds the slab lists and, with FDA_BWD_ZERO_IMAGE,
 * zero-fills the image.  After the last part call fda_backward_accumulate_levels over all levels
 * with FDA_BWD_RESUME | FDA_BWD_FINALIZE | FDA_BWD_BINNED_DONE and the same scratch.  Returns
 * FDA_ERR_WORKSPACE when scratch is missing or binning does not apply to the problem.
 * No counterpart in the reference.
 */
int fda_backward_bin_plan(const int64_t *spatial_shapes_host, int num_levels, int batch, int num_value, int num_heads,
                          int head_dim, int num_query, int num_points, int *level, int *slabs, int *depth);
int fda_backward_binned_part(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                             const void *sampling_loc_attn, const void *grad_output,
                             float *accum, void *grad_sampling_loc_attn,
                             int batch, int num_value, int num_heads, int head_dim, int num_levels,
                             int num_query, int num_points, int value_dtype, int packed_dtype,
                             int im2col_step, int part, int parts, int flags,
                             void *scratch, size_t scratch_bytes, void *stream);

/*
 * Cross-GPU sum + cast of the fp32 images over peer (NVLink) memory, for the query-sharded
 * backward: this rank sums slice `rank` (of `world` equal slices) of all ranks' images in fp32,
 * converts it to value_dtype and stores it into every rank's grad_value.  peer_images and
 * peer_outputs are HOST arrays of `world` DEVICE pointers, indexed by rank, that this GPU can
 * address (peer-mapped / symmetric memory); the local rank's own buffers are entry `rank`.
 * num_elements must be a multiple of 8.  The kernel only issues plain loads and stores and does
 * not wait on other ranks: the caller must place a cross-rank barrier on `stream` before the call
 * (all images complete) and after it (all pushes landed).  After the second barrier every rank's
 * grad_value holds the identical, fully reduced result.  world <= 16.
 * No counterpart in the reference (it has no multi-device path).
 */
int fda_peer_reduce_cast(const float *const *peer_images, void *const *peer_outputs, int world, int rank,
                         size_t num_elements, int value_dtype, void *stream);

/*
 * The same exchange when only a GROUP of ranks holds partial sums of this range of the image (the
 * batch-aligned partition: the ranks that share one batch element), while every rank of the job
 * needs the result: group_images is a HOST array of `group_size` DEVICE pointers indexed by rank
 * within the group (own image at `group_rank`); this rank sums slice `group_rank` of `group_size`
 * equal slices and stores the converted result into all `world` peer_outputs.  A group of one is a
 * cast + broadcast.  Same barrier contract as fda_peer_reduce_cast.  No counterpart in the reference.
 */
int fda_group_reduce_cast(const float *const *group_images, int group_size, int group_rank,
                          void *const *peer_outputs, int world, int rank,
                          size_t num_elements, int value_dtype, void *stream);

/*
 * Head-sharded backward (every rank of a group owns a slice of the heads of one batch element, so no sum is needed):
 * converts the cells [cell_begin, cell_begin + cell_count) of this rank's compact fp32 image [cells][slice_elements] to
 * value_dtype and stores them into every rank's full gradient [cells][full_elements] at element offset
 * head_offset_elements of each cell.  peer_outputs[r] points at the batch element inside rank r's grad_value (peer
 * memory, 16-byte aligned); all element counts are multiples of 8.  No waits inside; run one cross-rank barrier after
 * it before grad_value is read.  No counterpart in the reference.
 */
int fda_head_slice_cast_push(const float *image_slice, void *const *peer_outputs, int world, int rank,
                             size_t cell_begin, size_t cell_count, int slice_elements, int full_elements,
                             int head_offset_elements, int value_dtype, void *stream);

/*
 * Push variant of the same exchange, in two calls with a cross-rank barrier between them (and the
 * usual one after): fda_peer_push_partials stores the slices of the local image that other ranks
 * own into their staging areas (peer_staging: HOST array of `world` DEVICE pointers, each area
 * world * slot_stride_elements floats; this rank writes slot `rank` of every other area), then
 * fda_peer_reduce_staged_cast sums the own slice of the local image with the world-1 partials staged
 * locally, converts, and stores the result into every rank's grad_value.  slot_stride_elements is a
 * multiple of 8 and at least the longest slice.  No counterpart in the reference.
 */
int fda_peer_push_partials(const float *image, float *const *peer_staging, size_t slot_stride_elements,
                           int world, int rank, size_t num_elements, void *stream);
int fda_peer_reduce_staged_cast(const float *image, const float *staging, size_t slot_stride_elements,
                                void *const *peer_outputs, int world, int rank, size_t num_elements,
                                int value_dtype, void *stream);

/*
 * Same exchange through NVSwitch multicast (NVLS): mc_image and mc_output are the MULTICAST
 * addresses of the fp32 image and of grad_value (both bound on all `world` ranks).  This rank's
 * slice is summed in the switch (multimem.ld_reduce .add.f32), converted once, and written to
 * every rank's grad_value with multimem.st.  Same barrier contract as fda_peer_reduce_cast.
 * No counterpart in the reference.
 */
int fda_multimem_reduce_cast(const float *mc_image, void *mc_output, int world, int rank,
                             size_t num_elements, int value_dtype, void *stream);

/*
 * Builds the operator's planar input from what a multi-scale deformable-attention layer has after
 * its projections: offsets [B,Lq,G,L,K,3] (x,y,z, in cells of level l), reference_points [B,Lq,L,3]
 * (normalised), logits [B,Lq,G,L,K], all of `dtype`; packed [B,Lq,G,L*K*4] is fp32:
 * coordinates reference + offset / (W_l,H_l,D_l), then the logits.  One fused pass.  The reference
 * leaves this step to its callers (its tests build the tensor with torch.cat).
 */
int fda_pack_sampling(const void *offsets, const void *reference_points, const void *logits,
                      const int64_t *spatial_shapes, float *packed, int batch, int num_query, int num_heads,
                      int num_levels, int num_points, int dtype, void *stream);

/*
 * Backward of fda_pack_sampling: from grad_packed [B,Lq,G,L*K*4] (fp32, as the operator's backward returns it
 * for fp32 offsets) to grad_offsets [B,Lq,G,L,K,3] = coordinate gradients / (W_l,H_l,D_l),
 * grad_reference_points [B,Lq,L,3] = coordinate gradients summed over heads and points, and
 * grad_logits [B,Lq,G,L,K], all of `dtype`.  One fused pass.  No counterpart in the reference.
 */
int fda_pack_sampling_backward(const float *grad_packed, const int64_t *spatial_shapes, void *grad_offsets,
                               void *grad_reference_points, void *grad_logits, int batch, int num_query,
                               int num_heads, int num_levels, int num_points, int dtype, void *stream);

/*
 * DCNv4-3D (volumetric deformable convolution v4), forward and backward:
 *   output[b, q, g, :] = sum_k m_k * trilinear(value[b], p0(q) + (stencil_k * dilation + offset_k) * offset_scale)[g, :]
 * value [batch][depth_in][height_in][width_in][group*group_channels]; p_offset [batch][Q][padded_offset_dim] with
 * Q = depth_out*height_out*width_out and, per group g, K*3 offsets (x, y, z per point) then K mask values at
 * g*K*4 (K = kernel_d*kernel_h*kernel_w, minus one with remove_center; stencil order w outermost, d innermost);
 * output / grad_output [batch][Q][group*group_channels]; kernel / stride / pad / dilation are HOST arrays of three
 * ints in (d, h, w) order; one dtype for all tensors.  softmax != 0 soft-maxes the K masks of a (q, g).
 *
 * Replace dcnv4_im2col_cuda / dcnv4_col2im_cuda and the host code around them (reference
 * csrc/cuda/dcnv4_im2col_cuda.cuh, csrc/cuda/dcnv4_col2im_cuda.cuh, csrc/cuda/dcnv4_cuda.cu:19-189; entry points
 * csrc/dcnv4.h:7-61).  d_stride / block_thread of the reference are launch hints and have no counterpart here.
 * The backward zero-fills what it accumulates into and writes both gradients completely (offset-row padding = 0);
 * gradients come back in the tensors' own dtype.  workspace: fda_dcnv4_backward_workspace_bytes() (an fp32 image of
 * grad_value for 16-bit dtypes, none for fp32), 16-byte aligned.
 */
int fda_dcnv4_output_size(int depth_in, int height_in, int width_in, const int *kernel, const int *stride,
                          const int *pad, const int *dilation, int *depth_out, int *height_out, int *width_out);
int fda_dcnv4_forward(const void *value, const void *p_offset, void *output, int batch, int depth_in, int height_in,
                      int width_in, int group, int group_channels, const int *kernel, const int *stride,
                      const int *pad, const int *dilation, float offset_scale, int remove_center, int softmax,
                      int padded_offset_dim, int dtype, int im2col_step, void *stream);
size_t fda_dcnv4_backward_workspace_bytes(int batch, int depth_in, int height_in, int width_in, int group,
                                          int group_channels, int dtype);
int fda_dcnv4_backward(const void *value, const void *p_offset, const void *grad_output, void *grad_value,
                       void *grad_offset, void *workspace, size_t workspace_bytes, int batch, int depth_in,
                       int height_in, int width_in, int group, int group_channels, const int *kernel,
                       const int *stride, const int *pad, const int *dilation, float offset_scale,
                       int remove_center, int softmax, int padded_offset_dim, int dtype, int im2col_step,
                       void *stream);

/*
 * ROI-Align 3D.  features [N][C][D][H][W] (channels first, as the reference's op), rois [num_rois][7] =
 * (batch index, x1, y1, z1, x2, y2, z2) in input coordinates (scaled by spatial_scale), output
 * [num_rois][C][pooled_depth][pooled_height][pooled_width]; sampling_ratio <= 0 = adaptive (ceil(roi extent / bins)
 * samples per bin and axis); order 0 = nearest, 1 = trilinear.  Forward: features, rois and output share `dtype`,
 * accumulation in fp32.  Backward: grad_output of grad_output_dtype, rois and grad_features fp32; grad_features must
 * be zero-filled by the caller (the reference's contract) and is accumulated into with fp32 atomics.
 * Replace roi_align_3d_forward / roi_align_3d_backward (reference csrc/roi_align_3d.h,
 * csrc/cuda/roi_align_3d_cuda_kernel.cuh:31,110, csrc/cuda/interpolation_helpers_3d.h).
 */
int fda_roi_align3d_forward(const void *features, const void *rois, void *output, int num_rois, int channels,
                            int depth, int height, int width, int pooled_depth, int pooled_height,
                            int pooled_width, float spatial_scale, int sampling_ratio, int order, int dtype,
                            void *stream);
int fda_roi_align3d_backward(const void *grad_output, const float *rois, float *grad_features, int num_rois,
                             int channels, int depth, int height, int width, int pooled_depth,
                             int pooled_height, int pooled_width, float spatial_scale, int sampling_ratio,
                             int order, int grad_output_dtype, void *stream);

/*
 * NMS 3D on boxes ALREADY SORTED by decreasing score: boxes_sorted [num_boxes][6] = (x1, y1, z1, x2, y2, z2) fp32.
 * A box is dropped when its IoU with an earlier kept box exceeds iou_threshold.  keep [num_boxes] receives the
 * positions (in the sorted order) of the kept boxes, *num_keep (device int) their number; workspace holds the
 * pairwise bit matrix (fda_nms3d_workspace_bytes).  Both the matrix and the greedy sweep run on the device.
 * Replace nms_3d_cuda (reference csrc/cuda/nms_3d_cuda.cu:49-162; entry point csrc/nms_3d.h:28), whose sweep runs
 * on the host after copying the matrix back.
 */
size_t fda_nms3d_workspace_bytes(int num_boxes);
int fda_nms3d(const float *boxes_sorted, int num_boxes, float iou_threshold, void *workspace,
              size_t workspace_bytes, long long *keep, int *num_keep, void *stream);

/*
 * Backward pass that needs no workspace from the caller and allocates nothing: same inputs,
 * outputs and results as fda_backward, but the fp32 accumulation image sits in a fixed
 * FDA_NOALLOC_MAX_ELEMENTS-float (64 MiB) array inside the library, present on every GPU that
 * loads it.  Meant for callers that may not allocate device memory where they run (an engine
 * plug-in's execute hook, a process whose pool already owns the whole GPU, a loop that cannot
 * tolerate cudaMalloc's synchronisation).  No counterpart in the reference, whose backward
 * always allocates its fp32 buffers through torch.
 *
 * Returns FDA_ERR_TOO_LARGE_STATIC when a 16-bit grad_value has more than
 * FDA_NOALLOC_MAX_ELEMENTS elements (fp32 values accumulate in place and have no limit).
 * The first call on each device looks up the array's device address (that device must be
 * current); with lazy module loading that lookup is also what places the 64 MiB on the device,
 * so make that first call (any small problem will do) at start-up: before a memory pool takes
 * the rest of the GPU -- afterwards it can fail with FDA_ERR_CUDA / out of memory, see
 * fda_last_cuda_error() -- and before any stream capture starts.  All calls share the one
 * array: calls that overlap on a GPU race with each other, so keep them ordered.  The array is
 * not cleared between calls; each call zeroes the part it uses before accumulating.
 */
#define FDA_NOALLOC_MAX_ELEMENTS (16u * 1024u * 1024u)
int fda_backward_noalloc(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                         const void *sampling_loc_attn, const void *grad_output,
                         void *grad_value, void *grad_sampling_loc_attn,
                         int batch, int num_value, int num_heads, int head_dim, int num_levels,
                         int num_query, int num_points, int value_dtype, int packed_dtype,
                         int im2col_step, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* FDA_B200_H_ */
