/*
 * trigrad_b200 - C ABI of the B200 (sm_100a) differentiable triangle rasteriser.
 *
 * This is the drop-in boundary for the render path of Davidxdydz/trigrad.  In the reference
 * that boundary is a pybind11 module taking torch::Tensor by value
 * (src/trigrad/module.cu:8-10, src/trigrad/render.h:6-38); here it is plain C: raw device
 * pointers, sizes, a CUDA stream and an int status.  The library never allocates or frees
 * device memory: outputs, saved state and workspace belong to the caller.
 *
 * Conventions
 *   vertices   [V,4] float32  (x, y, z, w), x/y in NDC, row 0 of the image is y = -1
 *   indices    [T,3] int32
 *   colors     [V,3] float32, opacities [V] float32
 *   image      [H,W,4] float32 (rgb accumulated, a = remaining transmittance)
 *   tiles      tiles_x = ceil(W/tile_w), tiles_y = ceil(H/tile_h), tile id = ty*tiles_x + tx
 *   All pointers are device pointers unless named *_host.  `stream` is a cudaStream_t.
 *   Every function returns TG_OK (0) or one of the TG_ERR_* codes; tg_last_error() gives text.
 *   The number of (triangle, tile) pairs K must stay below 2^31.
 *
 * Threads and state.  Every entry point may be called from any host thread (the reference runs its
 * forward on the caller's thread and its backward on an autograd worker thread); work is ordered on
 * the stream that is passed, the device is the one current on the calling thread.  The library keeps
 * no state between calls that affects results.  What it caches, all of it invisible to the caller:
 *   - per host thread: the text behind tg_last_error(); one cudaEvent_t per device (marks "K has
 *     reached the host" inside tg_render_forward); the occupancy figures of the radix-sort kernels
 *     for the device last used by that thread;
 *   - per process: an atomic launch counter (tg_launch_count); per device, atomically, "the opt-in
 *     shared-memory size of the long tile sort has been set" and the device address of the fixed
 *     array behind tg_scan_static.  These belong to the device's primary context: a program that
 *     resets a device (cudaDeviceReset) must not call the library on it afterwards.
 */
#ifndef TRIGRAD_B200_H
#define TRIGRAD_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* tg_stream_t; /* cudaStream_t */

enum {
    TG_OK = 0,
    TG_ERR_BAD_ARG = 1,     /* null pointer, non-positive size, tile_w*tile_h > 1024 ... */
    TG_ERR_WORKSPACE = 2,   /* workspace / scratch smaller than tg_*_bytes() says */
    TG_ERR_CAPACITY = 3,    /* K exceeds the caller's list capacity; K is reported back */
    TG_ERR_DEVICE_FLAG = 4, /* a kernel raised its error word (a bounded wait ran out) */
    TG_ERR_CUDA = 5         /* a CUDA runtime call or launch failed */
};

/* Words per packed per-triangle record (float32 words). */
#define TG_GEO_WORDS 16  /* M[9] row-major, z[3], w[3], depth lower bound */
#define TG_ATTR_WORDS 24 /* opacity[3], colour a/b/c [9], 1/w [3], vertex ids [3] (as int bits), xy of a/b/c [6] */

int tg_version(void);
const char* tg_status_string(int status);
/* Text of the last failure on the calling thread ("" if none). */
const char* tg_last_error(void);
/* Number of kernels this library has launched in this process so far (diagnostic counter; the
 * reference has no counterpart). */
unsigned long long tg_launch_count(void);

/* ---- stage 1: per-triangle preprocess ------------------------------------------------------
 * Tile rectangle of the bounding box, tile-overlap count, barycentric matrix and packed records.
 * Replaces count_per_tile_kernel (src/trigrad/render.cu:90-121, rectangle rule :51-76) and
 * cartesian_to_bary_kernel (src/trigrad/render.cu:310-337).
 *   tri_counts [T] uint32      number of tiles in the rectangle, 0 for degenerate triangles
 *   tri_rects  [T,4] int32     (x0,y0,x1,y1) or (0,-1,0,-1); may be NULL
 *   tri_geo    [T,TG_GEO_WORDS], tri_attr [T,TG_ATTR_WORDS] float32, 16-byte aligned
 */
int tg_preprocess(const float* vertices, const int32_t* indices, const float* colors, const float* opacities,
                  int T, int W, int H, int tile_w, int tile_h, uint32_t* tri_counts, int32_t* tri_rects,
                  float* tri_geo, float* tri_attr, tg_stream_t stream);

/* ---- stage 2: device-wide exclusive prefix scan ---------------------------------------------
 * out[i] = sum(in[0..i)), out[n] = total.  Single pass, decoupled look-back with bounded waits.
 * Replaces offsets.sum() + torch::cumsum_out (src/trigrad/render.cu:290-295).
 * `status` is one device uint32 that the kernel sets non-zero if a wait ran out.
 */
size_t tg_scan_scratch_bytes(int n);
int tg_scan(const uint32_t* in, uint32_t* out, int n, void* scratch, size_t scratch_bytes, uint32_t* status,
            tg_stream_t stream);

/* Same scan for callers that cannot allocate device memory where they need it (a host with a fixed
 * memory plan, a loop that must stay clear of the allocator, a plugin inside an application that
 * owns all allocations).  This entry point has no counterpart in the reference.  The look-back words
 * live in a 64 KB array inside the library image, so every GPU that loads the library holds that
 * much until the process exits, and n is limited to 2^24 elements per call (larger n is refused with
 * TG_ERR_CAPACITY; use tg_scan).  It calls no allocating routine.  The first call on each device
 * looks up the array's device address, so make that call before starting any stream capture.  All
 * calls on a device share the array, which is cleared at the start of each call: two calls whose
 * kernels may overlap on the GPU (different streams) race, so order them on one stream.
 */
int tg_scan_static(const uint32_t* in, uint32_t* out, int n, uint32_t* status, tg_stream_t stream);

/* Self-test of the bounded device-side waits (the look-back of tg_scan / tg_scan_static and of the sort
 * gives up after a fixed number of polls, raises `status` and lets the host return
 * TG_ERR_DEVICE_FLAG instead of hanging).  One warp waits, at most `spin_limit` (1..4096) polls, for a
 * partition word that nothing ever publishes, so the wait is certain to run out: *status (device
 * uint32) becomes 1.  scratch: 32 bytes of device memory, 8-byte aligned.  The launch always ends; no
 * other kernel is involved.  No counterpart in the reference, whose kernels never wait on one another.
 */
int tg_selftest_bounded_wait(void* scratch, size_t scratch_bytes, uint32_t* status, uint32_t spin_limit,
                             tg_stream_t stream);

/* ---- stage 3: key emission --------------------------------------------------------------------
 * For triangle t and every tile (tx outer, ty inner) of its rectangle, entry e = tri_offsets[t] + n:
 *   keys[e] = (uint64)tile << 32 | ord(depth key),  ids[e] = t
 * depth key = min plane depth over the triangle clipped to the tile, 1e30f if the clip is empty;
 * ord() is the order-preserving float->uint32 map (-0 folded into +0).
 * Replaces fill_per_tile_lists_kernel (src/trigrad/render.cu:140-270).
 */
int tg_emit_keys(const float* vertices, const int32_t* indices, int T, int W, int H, int tile_w, int tile_h,
                 const uint32_t* tri_offsets, uint64_t* keys, uint32_t* ids, uint32_t capacity, tg_stream_t stream);

/* ---- stage 4: onesweep LSD radix sort of (uint64 key, uint32 value) pairs --------------------
 * Stable, ascending on key bits [begin_bit, end_bit), 8-bit digits.  Sorts n pairs from
 * (keys_a, vals_a); the other pair of buffers is scratch.  *result_in_b_host tells where the
 * sorted data ended up (0: a, 1: b).  Replaces cub::DeviceSegmentedSort::StableSortPairs
 * (src/trigrad/render.cu:272-284): one global sort on tile<<32|depth equals a stable sort per tile.
 */
size_t tg_sort_scratch_bytes(uint32_t n);
int tg_sort_pairs(uint64_t* keys_a, uint64_t* keys_b, uint32_t* vals_a, uint32_t* vals_b, uint32_t n,
                  int begin_bit, int end_bit, void* scratch, size_t scratch_bytes, uint32_t* status,
                  int* result_in_b_host, tg_stream_t stream);

/* ---- stage 5: tile ranges ----------------------------------------------------------------------
 * offsets[t] = first position in the sorted keys whose tile id is >= t; offsets[tiles] = n.
 * Same object as the reference's `offsets` (src/trigrad/render.cu:292-295).
 */
int tg_tile_ranges(const uint64_t* sorted_keys, uint32_t n, int tiles, int32_t* offsets, tg_stream_t stream);

/* ---- stages 3-5 as the forward entry point runs them: segmented sort --------------------------------
 * entries: uint64 words (ordered depth << 32 | triangle), grouped by tile: tile t owns
 * entries[offsets[t] .. offsets[t+1]).  Every segment is sorted ascending in place and its low words
 * are written to sorted_ids at the same positions.  The words of one segment must differ from one
 * another (short segments are sorted by counting smaller words).  A triangle occurs at most once per tile, so the
 * result equals the stable sort of (tile << 32 | depth) keys that
 * cub::DeviceSegmentedSort::StableSortPairs produces for entries emitted in triangle order
 * (src/trigrad/render.cu:272-284).  scratch: tg_tile_sort_scratch_bytes(tiles) bytes (work lists of the
 * longer segments), 4-byte aligned; need not be cleared.  No device-side waiting: a segment of any length
 * is handled by one warp or one CTA.
 */
size_t tg_tile_sort_scratch_bytes(int tiles);
int tg_sort_tile_lists(uint64_t* entries, const int32_t* offsets, int tiles, int32_t* sorted_ids, void* scratch,
                       size_t scratch_bytes, tg_stream_t stream);

/* ---- stage 6: forward compositing ---------------------------------------------------------------
 * One CTA per tile, one thread per pixel.  Replaces render_forward_kernel
 * (src/trigrad/render.cu:540-619 with :338-453).  max_layers must be >= 1.
 * selection: NULL, or [tg_selection_planes()][H*W] int32 that receives, per pixel, the triangle ids of
 * the fragments it blended, in blending order (plane k = k-th fragment, k < ends).  The backward pass
 * then needs no second search of the tile lists.  tg_selection_planes() is max_layers in per-pixel
 * mode with max_layers <= 32 and 0 otherwise (then `selection` is ignored).
 */
int tg_selection_planes(int per_pixel_sort, int max_layers);
int tg_blend_forward(const float* tri_geo, const float* tri_attr, const int32_t* sorted_ids, const int32_t* offsets,
                     int W, int H, int tile_w, int tile_h, float early_stopping_threshold, int per_pixel_sort,
                     int max_layers, float* image, float* depthmap, float* final_weights, int32_t* ends,
                     int32_t* selection, tg_stream_t stream);

/* ---- stage 7: backward ------------------------------------------------------------------------
 * Replaces render_backward_kernel (src/trigrad/render.cu:621-695 with :455-538).
 * grad_vertices [V,4] (z column stays 0; 16-byte aligned), grad_colors [V,3], grad_opacities [V].
 * grad_depthmap may be NULL (no gradient flows into the depth map: taken as zero, and 4 bytes per pixel less to read).
 * accumulate == 0: the three gradient buffers are overwritten; != 0: added to.
 * selection: what tg_blend_forward wrote, or NULL (the lists are then searched again).
 * scratch: tg_backward_scratch_bytes(V) bytes, 16-byte aligned (packed per-vertex accumulator).
 */
size_t tg_backward_scratch_bytes(int V);
int tg_blend_backward(const float* tri_geo, const float* tri_attr, const int32_t* sorted_ids, const int32_t* offsets,
                      int V, int W, int H, int tile_w, int tile_h, int per_pixel_sort, int max_layers,
                      const float* grad_image, const float* grad_depthmap, const float* image, const float* depthmap,
                      const float* final_weights, const int32_t* ends, const int32_t* selection, float* grad_vertices,
                      float* grad_colors, float* grad_opacities, int accumulate, void* scratch, size_t scratch_bytes,
                      tg_stream_t stream);

/* Gradients of what the forward pass blended, in every mode (an extension; no counterpart in the reference).
 * tg_blend_backward restates the reference's backward literally, and that kernel is only consistent with its
 * forward in the default mode: with per_pixel_sort = 0 it visits the first `ends` list entries front to back
 * with recurrences written for a back-to-front walk (src/trigrad/render.cu:659-666 against :478-497), and
 * beyond 32 layers it reverses the order inside each batch of 32 only (:673-693).  This entry point computes
 * the derivative of the forward outputs with respect to vertices (x, y, w), colours and opacities for any
 * per_pixel_sort / max_layers; in the default mode it agrees with tg_blend_backward.  Arguments as for
 * tg_blend_backward without `selection`; accumulate is 0 or 1.
 */
int tg_blend_backward_corrected(const float* tri_geo, const float* tri_attr, const int32_t* sorted_ids,
                                const int32_t* offsets, int V, int W, int H, int tile_w, int tile_h, int per_pixel_sort,
                                int max_layers, const float* grad_image, const float* grad_depthmap, const float* image,
                                const float* depthmap, const float* final_weights, const int32_t* ends,
                                float* grad_vertices, float* grad_colors, float* grad_opacities, int accumulate,
                                void* scratch, size_t scratch_bytes, tg_stream_t stream);

/* Backward of the mean-squared-error loss  loss = loss_scale * sum((image - target)^2)  fused into stage 7:
 * the upstream gradient grad_scale * (image - target) is formed per pixel inside the kernel (depth-map
 * gradient zero), so no gradient image is written or read, and the loss value is reduced on the way.
 * For mean(): loss_scale = 1/(4 W H), grad_scale = 2/(4 W H).  *loss_out (device) is overwritten, or added
 * to when accumulate != 0.  Needs the selection saved by the forward pass (default mode); otherwise form
 * the gradient image yourself and call tg_blend_backward.  The reference has no counterpart: its users
 * write the loss in torch (notebooks/renderer.ipynb:529-548).
 */
int tg_blend_backward_l2(const float* tri_geo, const float* tri_attr, const int32_t* sorted_ids, const int32_t* offsets,
                         int V, int W, int H, int tile_w, int tile_h, int per_pixel_sort, int max_layers,
                         const float* target, float grad_scale, float loss_scale, float* loss_out, const float* image,
                         const float* depthmap, const float* final_weights, const int32_t* ends, const int32_t* selection,
                         float* grad_vertices, float* grad_colors, float* grad_opacities, int accumulate, void* scratch,
                         size_t scratch_bytes, tg_stream_t stream);

/* The same with the target image as 8-bit RGBA [H,W,4] (4-byte aligned): target = value / 255 (correctly rounded,
 * i.e. what `u8.float() / 255` gives in torch), a quarter of the bytes to bring to the GPU per view.
 */
int tg_blend_backward_l2_u8(const float* tri_geo, const float* tri_attr, const int32_t* sorted_ids, const int32_t* offsets,
                            int V, int W, int H, int tile_w, int tile_h, int per_pixel_sort, int max_layers,
                            const uint8_t* target_rgba8, float grad_scale, float loss_scale, float* loss_out,
                            const float* image, const float* depthmap, const float* final_weights, const int32_t* ends,
                            const int32_t* selection, float* grad_vertices, float* grad_colors, float* grad_opacities,
                            int accumulate, void* scratch, size_t scratch_bytes, tg_stream_t stream);

/* ---- gradients of several views in one packed accumulator ------------------------------------------
 * With accumulate = TG_ACCUMULATE_PACKED the backward entry points (tg_blend_backward, tg_blend_backward_l2,
 * tg_blend_step_l2, tg_render_step_l2) neither clear `scratch` nor write the three gradient tensors
 * (which may then be NULL, like loss_out): the packed per-vertex sums and the loss partials stay in
 * `scratch` and keep growing call after call - also from calls on several streams, the additions are
 * atomic.  The caller clears the tg_backward_scratch_bytes(V) bytes once (cudaMemsetAsync), runs the
 * views, orders the streams, and calls tg_unpack_gradients once: grad_* = (accumulate ? grad_* : 0) +
 * sums, loss_out likewise with loss_scale (loss_out may be NULL).  No counterpart in the reference, which
 * writes three gradient tensors per call (src/trigrad/render.cu:789-791).
 */
#define TG_ACCUMULATE_PACKED 2
int tg_unpack_gradients(const void* scratch, size_t scratch_bytes, int V, float loss_scale, float* loss_out,
                        float* grad_vertices, float* grad_colors, float* grad_opacities, int accumulate,
                        tg_stream_t stream);

/* Packed input layout (see TG_INPUT_PACKED): rgba [V,4] = (colors, opacities), faces [T,4] = (indices, 0).
 * No counterpart in the reference, whose layouts are fixed by its tensor arguments (src/trigrad/wrapper.py:115-158).
 */
int tg_pack_inputs(const float* colors, const float* opacities, const int32_t* indices, int V, int T, float* rgba,
                   int32_t* faces, tg_stream_t stream);
/* tg_unpack_gradients for the packed layout: grad_vertices [V,4] and grad_rgba [V,4] = (dr, dg, db, dopacity). */
int tg_unpack_gradients_rgba(const void* scratch, size_t scratch_bytes, int V, float loss_scale, float* loss_out,
                             float* grad_vertices, float* grad_rgba, int accumulate, tg_stream_t stream);

/* ---- forward + backward of mean((image - target)^2) in one kernel --------------------------------
 * No counterpart in the reference: tg_blend_forward followed by tg_blend_backward_l2 for the default
 * mode (per-pixel sort, 1 <= max_layers <= 32, tiles of at most 256 pixels), fused so that the values
 * the forward interpolates feed the backward recurrence directly (no selection planes, no second
 * read of the image).  Outputs and gradient conventions as for those two calls; the image, depth map,
 * final weights and ends are bit-identical to tg_blend_forward's.
 */
int tg_blend_step_l2(const float* tri_geo, const float* tri_attr, const int32_t* sorted_ids, const int32_t* offsets,
                     int V, int W, int H, int tile_w, int tile_h, float early_stopping_threshold, int max_layers,
                     const float* target, float grad_scale, float loss_scale, float* loss_out, float* image,
                     float* depthmap, float* final_weights, int32_t* ends, float* grad_vertices, float* grad_colors,
                     float* grad_opacities, int accumulate, void* scratch, size_t scratch_bytes, tg_stream_t stream);

/* ---- whole forward path -------------------------------------------------------------------------
 * Replaces render_forward (src/trigrad/render.cu:713-763).  Runs stages 1-6 on `stream`.
 *   selection    as for tg_blend_forward (may be NULL)
 *   sorted_ids   [list_capacity] int32   out, first K entries valid
 *   offsets      [tiles+1] int32         out
 *   info_host    uint32[4] in (preferably pinned) host memory.  [0] receives K and [1] the length
 *                of the longest tile list; the call waits on the host until they have arrived (it watches
 *                the first word, so pinned memory makes this quick; the reference synchronises at the same
 *                point, src/trigrad/render.cu:290).  [2] receives the device error
 *                word (0 = fine) by an asynchronous copy: it is valid after the caller next
 *                synchronises the stream.  [3] is not used.
 *   stage_ms_host  NULL or float[5]: milliseconds of {init, per_tile_lists, sorting,
 *                bary_transforms, rasterization} measured with CUDA events (synchronises)
 * If K > list_capacity nothing past the scan is run and TG_ERR_CAPACITY is returned with info_host[0]
 * set; call again with a larger list and workspace.
 *   flags        0, or TG_FORWARD_CULL_TILES: a (triangle, tile) pair of the bounding rectangle is listed only if
 *                the triangle can cover the centre of some pixel of that tile - the exact overlap test the
 *                reference leaves as a TODO (src/trigrad/render.cu:110; its lists hold every tile of the bounding
 *                box, the useless pairs carrying the key 1e30, :254-261).  The test evaluates each barycentric at
 *                the corner of the tile's pixel-centre rectangle that maximises it with the operations of the
 *                per-pixel coverage test, so it never drops a pair that covers a pixel: image, depth map and
 *                gradients are bit-identical with and without it in the default mode; offsets, sorted_ids and K
 *                shrink (they then differ from the reference's).  Not for per_pixel_sort = 0, where the
 *                reference's backward indexes the list by position.  Ignored beyond 65536 tiles.
 */
#define TG_FORWARD_CULL_TILES 1u
/*                TG_INPUT_PACKED: `indices` is [T,4] int32 (fourth word ignored) and `colors` is [V,4] float32
 *                (r, g, b, opacity), both 16-byte aligned; `opacities` is ignored (may be NULL).  One 16-byte load
 *                per face and per vertex attribute instead of the reference's 12-byte strides
 *                (src/trigrad/util.h:457-573: color3 and id3 are packed 3-word types).  Results are identical;
 *                tg_pack_inputs converts, tg_unpack_gradients_rgba returns the gradients in the same layout.
 */
#define TG_INPUT_PACKED 2u
size_t tg_forward_workspace_bytes(int T, int tiles, uint32_t list_capacity);
int tg_render_forward(const float* vertices, const int32_t* indices, const float* colors, const float* opacities,
                      int T, int W, int H, int tile_w, int tile_h, float early_stopping_threshold,
                      int per_pixel_sort, int max_layers, float* image, float* depthmap, float* final_weights,
                      int32_t* ends, int32_t* selection, float* tri_geo, float* tri_attr, int32_t* sorted_ids,
                      uint32_t list_capacity, int32_t* offsets, void* workspace, size_t workspace_bytes, uint32_t* info_host,
                      float* stage_ms_host, unsigned flags, tg_stream_t stream);

/* ---- whole optimisation step of one view ------------------------------------------------------------
 * tg_render_forward with tg_blend_step_l2 in place of the compositing kernel: binning, tile lists,
 * forward, loss and gradients of one view in one call (same restrictions as tg_blend_step_l2).
 * Arguments as for tg_render_forward (workspace, info_host, stage_ms_host: "rasterization" then covers
 * forward + backward) and tg_blend_backward_l2 (target, scales, loss_out, gradients, scratch).
 */
int tg_render_step_l2(const float* vertices, const int32_t* indices, const float* colors, const float* opacities,
                      int T, int V, int W, int H, int tile_w, int tile_h, float early_stopping_threshold, int max_layers,
                      const float* target, float grad_scale, float loss_scale, float* loss_out, float* image,
                      float* depthmap, float* final_weights, int32_t* ends, float* tri_geo, float* tri_attr,
                      int32_t* sorted_ids, uint32_t list_capacity, int32_t* offsets, float* grad_vertices,
                      float* grad_colors, float* grad_opacities, int accumulate, void* workspace, size_t workspace_bytes,
                      void* scratch, size_t scratch_bytes, uint32_t* info_host, float* stage_ms_host, unsigned flags,
                      tg_stream_t stream);

/* ---- the step before the path: world -> render-space vertices and the VJP ------------------------------
 * points [V,3] world positions, pv_host: 16 floats in HOST memory, the row-major projection * view
 * matrix.  vertices[v] = (clip.x / clip.w, clip.y / clip.w, clip.z / clip.w, 1 / clip.w) with
 * clip = PV * (x, y, z, 1): the tensor operations of the reference's viewer (viewer.py:271-278) in one
 * kernel.  tg_project_backward: grad_points [V,3] receives (accumulate = 0) or is increased by
 * (accumulate = 1) the vector-Jacobian product with grad_vertices [V,4] - what torch autograd does for
 * those tensor operations.  No near-plane handling: points with clip.w = 0 give infinities, as in the
 * reference.
 */
int tg_project(const float* points, int V, const float* pv_host, float* vertices, tg_stream_t stream);
int tg_project_backward(const float* points, int V, const float* pv_host, const float* grad_vertices, float* grad_points,
                        int accumulate, tg_stream_t stream);

/* ---- projection with near-plane triangle splitting -----------------------------------------------------
 * The reference clips in its notebook, with a Python loop over triangles (split_clipped,
 * notebooks/renderer.ipynb, cell "Clip Test"), before it divides by w: with d = clip.z + clip.w per vertex, a
 * triangle with three vertices at d >= 0 is kept, one with none is dropped, one inside vertex gives the triangle
 * (in, new1, new2), two give (in1, in2, new1) and (new1, in2, new2); new = a + t (b - a) with t = d_a / (d_a - d_b)
 * from the inside vertex a to the outside vertex b, colours and opacities interpolated with the same t.
 * tg_project_clip does projection (clip = PV * (x, y, z, 1) as tg_project), splitting and the division in one
 * kernel.  Input triangle t owns output triangles 2t and 2t+1, i.e. soup vertices 6t .. 6t+5; slots that are not
 * needed hold the degenerate triangle (0,0,0,1) x 3 with zero colour and opacity, which the rasteriser drops.
 *   out_vertices [6T,4] (x/w, y/w, z/w, 1/w), 16-byte aligned; out_indices [2T,3] = 0, 1, 2, ...;
 *   out_colors [6T,3]; out_opacities [6T]
 * tg_project_clip_backward ADDS the vector-Jacobian product (atomic additions) to grad_points [V,3],
 * grad_colors [V,3], grad_opacities [V], which the caller clears; the interpolation parameters t are
 * differentiated too, as torch autograd does for the reference's tensor expression.
 */
int tg_project_clip(const float* points, const int32_t* indices, const float* colors, const float* opacities, int T,
                    const float* pv_host, float* out_vertices, int32_t* out_indices, float* out_colors,
                    float* out_opacities, tg_stream_t stream);
int tg_project_clip_backward(const float* points, const int32_t* indices, const float* colors, const float* opacities,
                             int T, const float* pv_host, const float* grad_out_vertices, const float* grad_out_colors,
                             const float* grad_out_opacities, float* grad_points, float* grad_colors,
                             float* grad_opacities, tg_stream_t stream);

/* One view's packed accumulator (filled by the backward entry points with TG_ACCUMULATE_PACKED) straight to
 * world space: tg_unpack_gradients and tg_project_backward in one kernel.  The render-space vertex gradient
 * of every vertex goes through the VJP of tg_project (same points, same pv_host) and is ADDED to
 * grad_points [V,3]; colour and opacity gradients are ADDED to grad_colors [V,3] / grad_opacities [V]; the
 * view's loss (sum of its partials * loss_scale) is ADDED to *loss_out (may be NULL).  All additions are
 * atomic, so views rendered on several streams may add into the same tensors; the caller clears them once
 * per batch.  The accumulator is zero again when the kernel ends: clear it once
 * (tg_backward_scratch_bytes(V) bytes) before the first view and reuse it, one accumulator per stream.
 * What a view through the reference's viewer pays in torch for this: the autograd of viewer.py:271-278 plus
 * three gradient tensors per view.
 */
int tg_unpack_project_backward(void* scratch, size_t scratch_bytes, int V, const float* points, const float* pv_host,
                               float loss_scale, float* loss_out, float* grad_points, float* grad_colors,
                               float* grad_opacities, tg_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TRIGRAD_B200_H */
