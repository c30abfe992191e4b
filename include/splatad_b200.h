/*
 * splatad_b200 - C ABI of the B200 (sm_100a) render hot path of SplatAD.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (cudaStream_t passed
 * as void*; NULL = the legacy default stream), enqueues its kernels on that stream, allocates
 * nothing and returns a status code. All tensors are contiguous, row-major FP32 unless noted;
 * ids are int32 (flatten ids, offsets, radii of the camera) or int64 (isect ids, packed
 * camera/gaussian ids). Optional pointers may be NULL where the comment says so. Outputs and
 * workspaces are owned by the caller.
 *
 * Each declaration names the function of the reference (carlinds/splatad, a gsplat fork) whose
 * pybind11 binding it replaces: gsplat/cuda/csrc/ext.cpp:4-52 registers them and
 * gsplat/cuda/csrc/bindings.h declares their torch::Tensor signatures.
 */
#ifndef SPLATAD_B200_H
#define SPLATAD_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPLATAD_B200_VERSION 100

/* status codes */
#define SPLATAD_OK 0
#define SPLATAD_ERR_BAD_ARG 1   /* null pointer, bad shape or size            -> ValueError / AssertionError */
#define SPLATAD_ERR_CHANNELS 2  /* unsupported channel count                  -> ValueError                  */
#define SPLATAD_ERR_KEY_BITS 3  /* sensor bits + tile bits exceed 32          -> RuntimeError                */
#define SPLATAD_ERR_WORKSPACE 4 /* workspace missing or too small             -> RuntimeError                */
#define SPLATAD_ERR_CUDA 5      /* a CUDA runtime call or launch failed       -> RuntimeError                */
#define SPLATAD_ERR_OVERFLOW 6  /* more intersections than the given capacity -> RuntimeError                */

/* Largest channel count one compositing launch renders; callers chunk above it
 * (gsplat/rendering.py:362-392 and 733-773 chunk at 32 as well). */
#define SPLATAD_MAX_CHANNELS 32

/* Message of the last error raised on the calling thread ("" if none). */
const char *splatad_last_error(void);
int splatad_version(void);

/* FP32 FMA throughput probe used to measure the CUDA-core roofline of the compositing
 * kernels: grid blocks x 256 threads x iters x 128 FMAs. `out` holds grid*256 floats.
 * No counterpart in the reference. */
int splatad_fma_probe(float *out, int32_t grid, int32_t iters, void *stream);

/* Per-kernel timing for benchmarks (no counterpart in the reference). While enabled, every
 * kernel launch of the library is bracketed by a CUDA event pair on its stream (this creates
 * events: a measurement mode only). _report waits for them and writes "name launches total_ms"
 * lines, one per kernel name in first-launch order, then clears the records. */
int splatad_profile_enable(int32_t enable);
int splatad_profile_report(char *buf, size_t cap);

/* ------------------------------------------------------------------------------------------
 * Projection
 * ---------------------------------------------------------------------------------------- */

/* fully_fused_lidar_projection_fwd_tensor - gsplat/cuda/csrc/bindings.h (lidar projection),
 * host function gsplat/cuda/csrc/projection.cu:2631-2713, kernel 2268-2417.
 * means [N,3]; covars [N,6] or NULL; quats [N,4], scales [N,3] (used when covars is NULL);
 * velocities [N,3] or NULL; viewmats [C,4,4]; linear/angular_velocity [C,3];
 * rolling_shutter_time [C].
 * Outputs [C,N,..]: radii [.,2] float degrees, means2d [.,2], depths (range), conics [.,3],
 * compensations (NULL = not computed), pix_vels [.,3], depth_compensations [.,2].
 * Entries of culled pairs are zero. With quats / scales inputs whose arrays start on 16-byte
 * boundaries the kernel prefetches slabs of 256 Gaussians with bulk asynchronous copies; any
 * other alignment and covars inputs take a plain kernel with bit-identical outputs (see
 * splatad_async_copy_timeouts for the copies' bounded waits). */
int splatad_lidar_projection_fwd(
    uint32_t C, uint32_t N, const float *means, const float *covars, const float *quats,
    const float *scales, const float *velocities, const float *viewmats, float min_elevation,
    float max_elevation, float min_azimuth, float max_azimuth, const float *linear_velocity,
    const float *angular_velocity, const float *rolling_shutter_time, float eps2d,
    float near_plane, float far_plane, float radius_clip, float *radii, float *means2d,
    float *depths, float *conics, float *compensations, float *pix_vels,
    float *depth_compensations, void *stream);

/* fully_fused_lidar_projection_bwd_tensor - gsplat/cuda/csrc/projection.cu:2715-2826, kernel
 * 2419-2629. Gradient outputs are overwritten (not accumulated) except v_viewmats [C,4,4],
 * which must be zero-initialised by the caller when requested. v_covars / (v_quats, v_scales),
 * v_viewmats and v_velocities may be NULL. v_velocities [N,3] is the gradient the reference
 * computes and discards (projection.cu:2538-2541). */
int splatad_lidar_projection_bwd(
    uint32_t C, uint32_t N, const float *means, const float *covars, const float *quats,
    const float *scales, const float *velocities, const float *viewmats,
    const float *linear_velocity, const float *angular_velocity,
    const float *rolling_shutter_time, float eps2d, const float *radii, const float *conics,
    const float *compensations, const float *v_means2d, const float *v_depths,
    const float *v_conics, const float *v_compensations, const float *v_pix_vels,
    const float *v_depth_compensations, float *v_means, float *v_covars, float *v_quats,
    float *v_scales, float *v_viewmats, float *v_velocities, void *stream);

/* fully_fused_projection_fwd_tensor - gsplat/cuda/csrc/projection.cu:966-1045, kernel 605-751.
 * Ks [C,3,3]. Outputs [C,N,..]: radii [.,2] int32 pixels, means2d, depths (z), conics,
 * compensations (NULL = not computed), pix_vels [.,2]. */
int splatad_projection_fwd(
    uint32_t C, uint32_t N, const float *means, const float *covars, const float *quats,
    const float *scales, const float *velocities, const float *viewmats, const float *Ks,
    int32_t image_width, int32_t image_height, const float *linear_velocity,
    const float *angular_velocity, const float *rolling_shutter_time, float eps2d,
    float near_plane, float far_plane, float radius_clip, int32_t *radii, float *means2d,
    float *depths, float *conics, float *compensations, float *pix_vels, void *stream);

/* fully_fused_projection_bwd_tensor - gsplat/cuda/csrc/projection.cu:1047-1155, kernel 753-964. */
int splatad_projection_bwd(
    uint32_t C, uint32_t N, const float *means, const float *covars, const float *quats,
    const float *scales, const float *velocities, const float *viewmats, const float *Ks,
    int32_t image_width, int32_t image_height, const float *linear_velocity,
    const float *angular_velocity, const float *rolling_shutter_time, float eps2d,
    const int32_t *radii, const float *conics, const float *compensations,
    const float *v_means2d, const float *v_depths, const float *v_conics,
    const float *v_compensations, const float *v_pix_vels, float *v_means, float *v_covars,
    float *v_quats, float *v_scales, float *v_viewmats, float *v_velocities, void *stream);

/* fully_fused_projection_packed_fwd_tensor - gsplat/cuda/csrc/projection.cu:1355-1464, kernel
 * 1157-1353. The reference sizes its outputs after a device->host read of nnz; here that is a
 * two-call protocol: _count writes indptr [C+1] and *nnz_device (int64, device memory; the
 * caller copies it to the host), _fill writes the nnz rows (camera-major, Gaussian-minor).
 * The same workspace must be passed to both calls. _fill does not need the count on the host:
 * with outputs of `capacity` rows (from an earlier frame, say) it can be enqueued right behind
 * _count; rows at or beyond the capacity are dropped, the caller then sees nnz > capacity and
 * fills again; the rows between nnz and the capacity get camera id 0, Gaussian id 0 and radii 0
 * (nothing lists or draws them). capacity < 0: the outputs hold nnz rows. */
size_t splatad_projection_packed_workspace_bytes(uint32_t C, uint32_t N);
int splatad_projection_packed_count(
    uint32_t C, uint32_t N, const float *means, const float *covars, const float *quats,
    const float *scales, const float *velocities, const float *viewmats, const float *Ks,
    int32_t image_width, int32_t image_height, const float *linear_velocity,
    const float *angular_velocity, const float *rolling_shutter_time, float eps2d,
    float near_plane, float far_plane, float radius_clip, void *workspace,
    size_t workspace_bytes, int32_t *indptr, int64_t *nnz_device, void *stream);
int splatad_projection_packed_fill(
    uint32_t C, uint32_t N, const float *means, const float *covars, const float *quats,
    const float *scales, const float *velocities, const float *viewmats, const float *Ks,
    int32_t image_width, int32_t image_height, const float *linear_velocity,
    const float *angular_velocity, const float *rolling_shutter_time, float eps2d,
    float near_plane, float far_plane, float radius_clip, const void *workspace, int64_t capacity,
    int64_t *camera_ids, int64_t *gaussian_ids, int32_t *radii, float *means2d, float *depths,
    float *conics, float *compensations, float *pix_vels, void *stream);

/* No counterpart in the reference. Same result as splatad_projection_packed_count (indptr [C+1]
 * and *nnz_device), but for hosts that must not allocate device memory at all: a plugin living
 * inside an engine that has already handed the whole GPU to its own arena, a control loop whose
 * certification forbids allocator calls after start-up, a process whose memory budget is fixed by
 * an outer scheduler. Such a caller has no workspace to pass, so the per-(camera, block) counters
 * live in a 512 KiB array compiled into the library (every GPU that loads the library keeps it
 * until the process exits). Limit: C * ceil(N / 256) <= 65536 (e.g. one camera and 16.7 M
 * Gaussians, or 8 cameras and 2 M); beyond it the call fails with SPLATAD_ERR_WORKSPACE and a
 * message, and touches nothing. The call makes no cudaMalloc / cudaFree and uses no allocating
 * library routine; inputs and outputs are still the caller's.
 * The first call on each device looks the array's device address up (cudaGetSymbolAddress, with
 * that device current). Under lazy module loading that lookup is also what makes the CUDA runtime
 * load this library's code onto the device and back the array with memory, so "allocates nothing"
 * holds from the second call on: make one call per device at start-up, while allocation is still
 * permitted, and outside any stream capture.
 * All calls on a device share the one array: nothing in it has to be cleared between calls
 * (every slot a call reads it has written first), but two calls that overlap on the GPU - on
 * different streams, or from different threads - race on it and corrupt each other's counts.
 * It answers "how many packed rows, and where does each camera start"; it does not feed
 * splatad_projection_packed_fill, which reads its offsets from a caller workspace. */
int splatad_projection_packed_count_noalloc(
    uint32_t C, uint32_t N, const float *means, const float *covars, const float *quats,
    const float *scales, const float *velocities, const float *viewmats, const float *Ks,
    int32_t image_width, int32_t image_height, const float *linear_velocity,
    const float *angular_velocity, const float *rolling_shutter_time, float eps2d,
    float near_plane, float far_plane, float radius_clip, int32_t *indptr, int64_t *nnz_device,
    void *stream);

/* fully_fused_projection_packed_bwd_tensor - gsplat/cuda/csrc/projection.cu:1718-1838, kernel
 * 1466-1716. sparse_grad != 0: parameter gradients are [nnz,..] rows (plain stores);
 * otherwise [N,..] accumulated with atomics, so the caller zero-initialises them.
 * v_viewmats (optional) is always accumulated. */
int splatad_projection_packed_bwd(
    uint32_t C, uint32_t N, uint32_t nnz, const float *means, const float *covars,
    const float *quats, const float *scales, const float *velocities, const float *viewmats,
    const float *Ks, int32_t image_width, int32_t image_height, const float *linear_velocity,
    const float *angular_velocity, const float *rolling_shutter_time, float eps2d,
    const int64_t *camera_ids, const int64_t *gaussian_ids, const float *conics,
    const float *compensations, const float *v_means2d, const float *v_depths,
    const float *v_conics, const float *v_compensations, const float *v_pix_vels,
    int32_t sparse_grad, float *v_means, float *v_covars, float *v_quats, float *v_scales,
    float *v_viewmats, float *v_velocities, void *stream);

/* ------------------------------------------------------------------------------------------
 * Spherical harmonics
 * ---------------------------------------------------------------------------------------- */

/* compute_sh_fwd_tensor - gsplat/cuda/csrc/sh.cu:408-433. dirs [n,3], coeffs [n,K,3],
 * masks [n] bytes (bool) or NULL, colors [n,3]. Masked-out rows are written as zero. */
int splatad_sh_fwd(uint32_t n_elems, uint32_t K, uint32_t degrees_to_use, const float *dirs,
                   const float *coeffs, const uint8_t *masks, float *colors, void *stream);

/* compute_sh_bwd_tensor - gsplat/cuda/csrc/sh.cu:435-468. v_coeffs [n,K,3] and v_dirs [n,3]
 * (NULL = not wanted) are overwritten. */
int splatad_sh_bwd(uint32_t n_elems, uint32_t K, uint32_t degrees_to_use, const float *dirs,
                   const float *coeffs, const uint8_t *masks, const float *v_colors,
                   float *v_coeffs, float *v_dirs, void *stream);

/* Camera centres campos [C,3] = inverse(viewmats)[:, :3, 3] (general 4 x 4 inverse by cofactors,
 * evaluated in double): what gsplat/rendering.py:345 takes from torch.inverse(viewmats). */
int splatad_camera_centers(uint32_t C, const float *viewmats, float *campos, void *stream);

/* View-dependent colours of the projected Gaussians in one pass - the torch chain around the SH
 * kernel in gsplat/rendering.py:345-373 (gathers by the packed ids, directions = means - camera
 * centres, spherical_harmonics with the radii mask, + 0.5, clamp at 0, depth appended for the
 * "+D" render modes). Entry e is (camera_ids[e], gaussian_ids[e]) (packed, int64) or
 * (e / N, e % N) (both NULL, n_elems = C * N). coeffs is [N,K,3], or [C,N,K,3] when
 * coeffs_per_camera != 0; campos [C,3]; radii [n_elems,2] int32; colors [n_elems,out_channels]
 * with out_channels 3, or 4 (then depths [n_elems] is the last channel). Entries with
 * radii[e][0] <= 0 hold 0.5 (the reference: uninitialised memory + 0.5). */
int splatad_sh_colors_fwd(uint32_t n_elems, uint32_t N, uint32_t K, uint32_t degrees_to_use,
                          const float *means, const float *campos, const float *coeffs,
                          uint32_t coeffs_per_camera, const int64_t *camera_ids,
                          const int64_t *gaussian_ids, const int32_t *radii, const float *depths,
                          uint32_t out_channels, float *colors, void *stream);
/* VJP: v_coeffs (shape of coeffs), v_means [N,3] and v_campos [C,3] are accumulated with atomics
 * (zero-initialise them), v_depths [n_elems] is overwritten; each may be NULL. */
int splatad_sh_colors_bwd(uint32_t n_elems, uint32_t N, uint32_t K, uint32_t degrees_to_use,
                          const float *means, const float *campos, const float *coeffs,
                          uint32_t coeffs_per_camera, const int64_t *camera_ids,
                          const int64_t *gaussian_ids, const int32_t *radii,
                          uint32_t out_channels, const float *v_colors, float *v_coeffs,
                          float *v_means, float *v_campos, float *v_depths, void *stream);

/* ------------------------------------------------------------------------------------------
 * Unfused building blocks of the projection (exported by the reference as separate ops,
 * gsplat/__init__.py:4-18). All tensors FP32 row-major; gradient outputs are written (not
 * accumulated) except v_viewmats, which is accumulated and must be zero-initialised.
 *
 * quat_scale_to_covar_preci_fwd/_bwd_tensor - gsplat/cuda/csrc/projection.cu:18-260. quats [N,4]
 *   (w,x,y,z, need not be normalised), scales [N,3]; covars / precis [N,3,3], or [N,6] upper
 *   triangles when triu != 0; either output (and its gradient) may be NULL.
 * world_to_cam_fwd/_bwd_tensor - projection.cu:466-599 (kernels in utils.cuh). means [N,3],
 *   covars [N,3,3], viewmats [C,4,4] -> means_c [C,N,3], covars_c [C,N,3,3]. In the backward any
 *   of v_means, v_covars, v_viewmats may be NULL.
 * persp_proj_fwd/_bwd_tensor - projection.cu:262-464. Sensor-frame means [C,N,3], covars
 *   [C,N,3,3], Ks [C,3,3] -> means2d [C,N,2], covars2d [C,N,2,2] (no blur added).
 * compute_pix_velocity_fwd/_bwd_tensor - projection.cu:2064-2266. p_view [C,N,3], lin_vel /
 *   ang_vel [C,3], velocities [C,N,3] (sensor frame) -> pixel velocities [C,N,2].
 * lidar_proj_fwd/_bwd_tensor - projection.cu:1841-2062. -> means2d [C,N,2] (azimuth, elevation in
 *   degrees), covars2d [C,N,2,2] (no blur added), depth_compensations [C,N,2].
 * compute_lidar_velocity_fwd/_bwd_tensor - projection.cu:2064-2266 (lidar variants). -> (azimuth,
 *   elevation, range) velocities [C,N,3].
 * ---------------------------------------------------------------------------------------- */
int splatad_quat_scale_to_covar_preci_fwd(uint32_t N, const float *quats, const float *scales,
                                          int32_t triu, float *covars, float *precis, void *stream);
int splatad_quat_scale_to_covar_preci_bwd(uint32_t N, const float *quats, const float *scales,
                                          const float *v_covars, const float *v_precis, int32_t triu,
                                          float *v_quats, float *v_scales, void *stream);
int splatad_world_to_cam_fwd(uint32_t C, uint32_t N, const float *means, const float *covars,
                             const float *viewmats, float *means_c, float *covars_c, void *stream);
int splatad_world_to_cam_bwd(uint32_t C, uint32_t N, const float *means, const float *covars,
                             const float *viewmats, const float *v_means_c, const float *v_covars_c,
                             float *v_means, float *v_covars, float *v_viewmats, void *stream);
int splatad_persp_proj_fwd(uint32_t C, uint32_t N, const float *means, const float *covars,
                           const float *Ks, uint32_t width, uint32_t height, float *means2d,
                           float *covars2d, void *stream);
int splatad_persp_proj_bwd(uint32_t C, uint32_t N, const float *means, const float *covars,
                           const float *Ks, uint32_t width, uint32_t height, const float *v_means2d,
                           const float *v_covars2d, float *v_means, float *v_covars, void *stream);
int splatad_compute_pix_velocity_fwd(uint32_t C, uint32_t N, const float *p_view, const float *lin_vel,
                                     const float *ang_vel, const float *velocities, const float *Ks,
                                     uint32_t width, uint32_t height, float *pix_vels, void *stream);
int splatad_compute_pix_velocity_bwd(uint32_t C, uint32_t N, const float *p_view, const float *lin_vel,
                                     const float *ang_vel, const float *velocities, const float *Ks,
                                     uint32_t width, uint32_t height, const float *v_pix_vels,
                                     float *v_p_view, float *v_velocities, void *stream);
int splatad_lidar_proj_fwd(uint32_t C, uint32_t N, const float *means, const float *covars, float eps2d,
                           float *means2d, float *covars2d, float *depth_compensations, void *stream);
int splatad_lidar_proj_bwd(uint32_t C, uint32_t N, const float *means, const float *covars, float eps2d,
                           const float *v_means2d, const float *v_covars2d,
                           const float *v_depth_compensations, float *v_means, float *v_covars,
                           void *stream);
int splatad_compute_lidar_velocity_fwd(uint32_t C, uint32_t N, const float *p_view, const float *lin_vel,
                                       const float *ang_vel, const float *velocities, float *lidar_vels,
                                       void *stream);
int splatad_compute_lidar_velocity_bwd(uint32_t C, uint32_t N, const float *p_view, const float *lin_vel,
                                       const float *ang_vel, const float *velocities,
                                       const float *v_lidar_vels, float *v_p_view, float *v_velocities,
                                       void *stream);

/* ------------------------------------------------------------------------------------------
 * Tile intersection
 *
 * isect_tiles_tensor (gsplat/cuda/csrc/rasterization.cu:92-216) and isect_lidar_tiles_tensor
 * (397-529) read the intersection count back to the host in the middle to size their outputs.
 * Here each is a two-call protocol on one stream:
 *   _plan  writes tiles_per_gauss, orders the visible Gaussians by depth, and copies
 *          host_counts[0..3] = {n_isects, n_visible, status bits, 0} to the host (pinned memory
 *          recommended; valid once the stream has reached that point). n_isects must fit
 *          int32 (flatten ids and offsets are int32): check it before calling _fill.
 *   _fill  writes isect_ids [capacity] int64 and flatten_ids [capacity] int32, sorted by
 *          (sensor, tile, depth bits, flatten index) when sort != 0, in flatten-index order
 *          otherwise. capacity >= n_isects; if it is smaller, status bit 1 is set in
 *          host_counts[2] (copied again by _fill) and the outputs are incomplete.
 *          tile_offsets (optional, [C * tiles + 1] int32, sort != 0 only) receives what
 *          splatad_isect_offset_encode would compute from isect_ids - the fill knows every
 *          tile's start already, so asking for it here saves that pass - followed by one more
 *          entry, the number of intersections written. With that entry in place the four
 *          compositing calls accept n_isects = -1 ("read the end of the last tile from
 *          tile_offsets[C * tiles]"), so a caller that passes a generous capacity can enqueue
 *          plan, fill and compositing without waiting for the count.
 * `sort`: 0 = lists in flatten-index order; 1 = sorted, with the depth order of the visible
 * Gaussians built by buckets (four kernels: count, scan, scatter, per-bucket order) - if more than
 * 1024 depths fall into one of the 65536 buckets that span the scene's depth range, the plan sets
 * status bit 4 in host_counts[2] and the order is not final: call _plan again with sort = 2;
 * 2 = sorted, depth order by four radix passes (twelve kernels, any depth distribution). Pass the
 * same value to _fill. Both give the same lists.
 * `total_elems` is C*N for the [C,N] layout (camera_ids NULL) or nnz for the packed layout
 * (camera_ids [nnz] int64 gives the sensor of each row, N is ignored).
 * Depths must be non-negative: their bit patterns are ordered as unsigned integers.
 * ---------------------------------------------------------------------------------------- */
size_t splatad_isect_plan_workspace_bytes(uint64_t total_elems);
size_t splatad_isect_fill_workspace_bytes(uint64_t capacity);

int splatad_isect_tiles_plan(
    uint32_t C, uint32_t N, uint64_t total_elems, const float *means2d, const int32_t *radii,
    const float *depths, const int64_t *camera_ids, uint32_t tile_size, uint32_t tile_width,
    uint32_t tile_height, int32_t sort, int32_t *tiles_per_gauss, void *workspace,
    size_t workspace_bytes, int64_t *host_counts, void *stream);
int splatad_isect_tiles_fill(
    uint32_t C, uint32_t N, uint64_t total_elems, const float *means2d, const int32_t *radii,
    const float *depths, const int64_t *camera_ids, uint32_t tile_size, uint32_t tile_width,
    uint32_t tile_height, int32_t sort, const int32_t *tiles_per_gauss, void *plan_workspace,
    void *fill_workspace, size_t fill_workspace_bytes, int64_t capacity, int64_t *isect_ids,
    int32_t *flatten_ids, int32_t *tile_offsets, int64_t *host_counts, void *stream);

/* elev_boundaries [n_boundaries] = tile boundaries in elevation (n_boundaries - 1 tile rows);
 * the number of azimuth tiles is ceil(360 / tile_azim_resolution) in float32 as in
 * gsplat/cuda/csrc/rasterization.cu:435; splatad_lidar_azimuth_tiles returns that number (to
 * size tile_offsets). */
uint32_t splatad_lidar_azimuth_tiles(float tile_azim_resolution);
int splatad_isect_lidar_tiles_plan(
    uint32_t C, uint32_t N, uint64_t total_elems, const float *means2d, const float *radii,
    const float *depths, const int64_t *camera_ids, const float *elev_boundaries,
    uint32_t n_boundaries, float tile_azim_resolution, float min_azim, int32_t sort,
    int32_t *tiles_per_gauss, void *workspace, size_t workspace_bytes, int64_t *host_counts,
    void *stream);
int splatad_isect_lidar_tiles_fill(
    uint32_t C, uint32_t N, uint64_t total_elems, const float *means2d, const float *radii,
    const float *depths, const int64_t *camera_ids, const float *elev_boundaries,
    uint32_t n_boundaries, float tile_azim_resolution, float min_azim, int32_t sort,
    const int32_t *tiles_per_gauss, void *plan_workspace, void *fill_workspace,
    size_t fill_workspace_bytes, int64_t capacity, int64_t *isect_ids, int32_t *flatten_ids,
    int32_t *tile_offsets, int64_t *host_counts, void *stream);

/* No counterpart in the reference. Arms a one-shot request for the NEXT _plan call of the calling
 * thread: when the lists will be built by the row / column split (sorted output, at most 128 tile
 * rows and 16384 tiles), a kernel stores host_pair[0] = n_isects, host_pair[2] = status bits and
 * then host_pair[1] = sequence into host_pair, four int64 of pinned (mapped) host memory, as soon
 * as they are known - before the depth order is built, with no copy in the stream. A host that only
 * needs the count polls host_pair[1] for `sequence` (a number it has not used for this triple
 * before) instead of waiting for the end of the plan. Otherwise (other list construction, memory not mapped for the
 * device) nothing is written and the host waits for host_counts as usual. NULL disarms. */
int splatad_isect_set_early_count(int64_t *host_pair, int64_t sequence);

/* No counterpart in the reference. Arms a one-shot hint for the NEXT _plan call of the calling
 * thread with sort = 1: the depths of the elements it will list are expected within
 * [depth_lo, depth_hi], given as the bit patterns of two non-negative finite floats (the range the
 * previous frame of the same sensor reported, widened a little). The depth buckets then span this
 * range, the rectangle count fills them as it goes and the separate bucket-count kernel is not
 * launched. The hint cannot change the result: depths outside it land in the end buckets and every
 * bucket is put in order by its full keys; a hint so wrong that an end bucket overflows shows as
 * status bit 4, exactly like crowded depths, and the caller repeats the plan without a hint. With
 * an early count armed as well, host_pair[3] receives dmin bits | dmax bits << 32 of the listed
 * elements of this plan (0 when the count comes from a kernel that does not know them). */
int splatad_isect_set_depth_range_hint(uint32_t depth_lo_bits, uint32_t depth_hi_bits);

/* isect_offset_encode_tensor - gsplat/cuda/csrc/rasterization.cu:264-285.
 * offsets [C, tile_height, tile_width] int32. */
int splatad_isect_offset_encode(const int64_t *isect_ids, int64_t n_isects, uint32_t C,
                                uint32_t tile_width, uint32_t tile_height, int32_t *offsets,
                                void *stream);

/* ------------------------------------------------------------------------------------------
 * Lidar points -> tiles -> raster image: prepares `raster_pts` from a point cloud, the step
 * before a lidar render (examples/lidar_rendering.ipynb cell 8).
 *
 * map_points_to_lidar_tiles_tensor - gsplat/cuda/csrc/rasterization.cu:596-747: tile of every
 * point (zero radius), tile_ids [total] int64 = sensor << 32 | tile, flatten_ids [total] int32 =
 * point index; with sort != 0 both are ordered by tile id, ties in point order (a stable sort, as
 * the reference's radix sort is). points2d [C,N,2] (camera_ids NULL) or [nnz,2] with camera_ids
 * [nnz] int64. The workspace (splatad_map_points_workspace_bytes) is only needed when sorting.
 * points_mapping_offset_encode_tensor - rasterization.cu:531-594. offsets [C, tile_height,
 * tile_width] int32 (zeros when there are no points).
 * populate_image_from_points_tensor - rasterization.cu:749-833. image [C, H, W, 5] is cleared
 * and then, per tile, the k-th point of the tile's list is written at the tile's k-th pixel
 * (row-major inside the tile; points beyond tile_width * tile_height per tile are dropped, as are
 * those whose pixel lies outside the image).
 * ---------------------------------------------------------------------------------------- */
size_t splatad_map_points_workspace_bytes(uint64_t total_elems);
int splatad_map_points_to_lidar_tiles(
    uint32_t C, uint32_t N, uint64_t total_elems, const float *points2d, const int64_t *camera_ids,
    const float *elev_boundaries, uint32_t n_boundaries, float tile_azim_resolution, float min_azim,
    int32_t sort, void *workspace, size_t workspace_bytes, int64_t *tile_ids, int32_t *flatten_ids,
    void *stream);
int splatad_points_mapping_offset_encode(const int64_t *point_ids, int64_t n_points, uint32_t C,
                                         uint32_t tile_width, uint32_t tile_height, int32_t *offsets,
                                         void *stream);
int splatad_populate_image_from_points(
    uint32_t C, int64_t n_points, const float *points, uint32_t image_width, uint32_t image_height,
    uint32_t tile_width, uint32_t tile_height, uint32_t tile_grid_width, uint32_t tile_grid_height,
    const int32_t *tile_offsets, const int32_t *flatten_ids, float *image, void *stream);


/* ------------------------------------------------------------------------------------------
 * Compositing. `channels` is the true channel count (1..SPLATAD_MAX_CHANNELS): no padding to
 * a supported size is needed, unlike gsplat/cuda/_wrapper.py:876-921.
 * ---------------------------------------------------------------------------------------- */

/* rasterize_to_pixels_fwd_tensor - gsplat/cuda/csrc/rasterization.cu:1520-2019, kernel
 * 1360-1518. Inputs are [C,N,..] or packed [nnz,..] (flatten_ids index either);
 * backgrounds [C,channels] or NULL. Outputs: render_colors [C,H,W,channels],
 * render_alphas [C,H,W], last_ids [C,H,W] int32; every pixel is written. */
int splatad_rasterize_to_pixels_fwd(
    uint32_t C, int64_t n_isects, const float *means2d, const float *conics, const float *colors,
    uint32_t channels, const float *opacities, const float *pix_vels,
    const float *rolling_shutter_time, const float *backgrounds, uint32_t image_width,
    uint32_t image_height, uint32_t tile_size, uint32_t tile_width, uint32_t tile_height,
    const int32_t *tile_offsets, const int32_t *flatten_ids, float *render_colors,
    float *render_alphas, int32_t *last_ids, void *stream);

/* rasterize_to_pixels_bwd_tensor - gsplat/cuda/csrc/rasterization.cu:3091-3726, kernel
 * 2833-3089. Gradient outputs are accumulated with atomics: zero-initialise them.
 * v_means2d_abs may be NULL. */
int splatad_rasterize_to_pixels_bwd(
    uint32_t C, int64_t n_isects, const float *means2d, const float *conics, const float *colors,
    uint32_t channels, const float *opacities, const float *pix_vels,
    const float *rolling_shutter_time, const float *backgrounds, uint32_t image_width,
    uint32_t image_height, uint32_t tile_size, uint32_t tile_width, uint32_t tile_height,
    const int32_t *tile_offsets, const int32_t *flatten_ids, const float *render_alphas,
    const int32_t *last_ids, const float *v_render_colors, const float *v_render_alphas,
    float *v_means2d_abs, float *v_means2d, float *v_conics, float *v_colors, float *v_opacities,
    float *v_pix_vels, void *stream);

/* rasterize_to_points_fwd_tensor - gsplat/cuda/csrc/rasterization.cu:2221-2831, kernel
 * 2021-2219. raster_pts [C,H,W,4] = (azimuth deg, elevation deg, range m, time offset s);
 * points with range <= 0 are not rendered and produce zeros. pix_vels [.,3],
 * depth_compensations [.,2]. depth_channel_idx names the channel that holds the Gaussian's
 * range. alpha_sum_until_points may be NULL when compute_alpha_sum_until_points == 0.
 * gaussian_ranges (optional): when given, lidar_features holds channels - 1 columns and the
 * last rendered channel (depth_channel_idx == channels - 1) is read from this [C,N] / [nnz]
 * array instead - this spares the caller the concatenation of features and range that
 * gsplat/rendering.py:746, 779 performs for every frame. */
int splatad_rasterize_to_points_fwd(
    uint32_t C, int64_t n_isects, const float *means2d, const float *conics,
    const float *lidar_features, const float *gaussian_ranges, uint32_t channels,
    const float *opacities,
    const float *pix_vels, const float *depth_compensations, const float *backgrounds,
    const float *raster_pts, uint32_t image_width, uint32_t image_height, uint32_t tile_width,
    uint32_t tile_height, uint32_t tile_grid_width, uint32_t tile_grid_height,
    int32_t compute_alpha_sum_until_points, float alpha_sum_threshold,
    const int32_t *tile_offsets, const int32_t *flatten_ids, uint32_t depth_channel_idx,
    float *render_features, float *render_alphas, float *alpha_sum_until_points,
    int32_t *last_ids, float *median_depths, void *stream);

/* rasterize_to_points_bwd_tensor - gsplat/cuda/csrc/rasterization.cu:4056-4851, kernel
 * 3728-4054. v_alpha_sum_until_points may be NULL (treated as zero). Gradient outputs are
 * accumulated with atomics: zero-initialise them. With gaussian_ranges, v_features has
 * channels - 1 columns and the range gradient goes to v_gaussian_ranges. */
int splatad_rasterize_to_points_bwd(
    uint32_t C, int64_t n_isects, const float *means2d, const float *conics,
    const float *lidar_features, const float *gaussian_ranges, uint32_t channels,
    const float *opacities,
    const float *pix_vels, const float *depth_compensations, const float *backgrounds,
    const float *raster_pts, uint32_t image_width, uint32_t image_height, uint32_t tile_width,
    uint32_t tile_height, uint32_t tile_grid_width, uint32_t tile_grid_height,
    int32_t compute_alpha_sum_until_points, float alpha_sum_threshold,
    const int32_t *tile_offsets, const int32_t *flatten_ids, uint32_t depth_channel_idx,
    const float *render_alphas, const int32_t *last_ids, const float *v_render_features,
    const float *v_render_alphas, const float *v_alpha_sum_until_points, float *v_means2d_abs,
    float *v_means2d, float *v_conics, float *v_features, float *v_opacities, float *v_pix_vels,
    float *v_depth_compensations, float *v_gaussian_ranges, void *stream);

/* ------------------------------------------------------------------------------------------
 * Indices of contributing (Gaussian, pixel) pairs within a range of list batches.
 * rasterize_to_indices_in_range_tensor - gsplat/cuda/csrc/rasterization.cu:992-1090 (kernel
 * 839-990) and rasterize_to_indices_in_range_lidar_tensor - 1264-1358 (kernel 1092-1262);
 * Python wrappers gsplat/cuda/_wrapper.py:1115-1281.
 *
 * A batch is tile_size^2 (lidar: tile_width * tile_height) consecutive entries of a tile's
 * list; batches [range_start, range_end) are walked from transmittances [C,H,W]. The
 * reference's two kernel passes with torch.cumsum in between become two calls:
 *   _count  counts per pixel, prefix-sums on the device and fills chunk_starts [C*H*W + 1]
 *           (int64, exclusive, the total in the last entry); if host_total is not NULL the
 *           total is also copied there and the stream is synchronised;
 *   _write  fills gaussian_ids / pixel_ids / camera_ids [total] (int64; pixel_ids are row-major
 *           inside their camera, i.e. already split the way _wrapper.py:1194-1196 does).
 * Pairs are ordered by camera, then pixel, then list position. workspace: device memory of
 * splatad_rasterize_to_indices_workspace_bytes(C, W, H) bytes (count pass only).
 * ---------------------------------------------------------------------------------------- */
size_t splatad_rasterize_to_indices_workspace_bytes(uint32_t C, uint32_t image_width,
                                                    uint32_t image_height);
int splatad_rasterize_to_indices_in_range_count(
    uint32_t range_start, uint32_t range_end, uint32_t C, uint32_t N, int64_t n_isects,
    const float *transmittances, const float *means2d, const float *conics, const float *opacities,
    const float *pix_vels, const float *rolling_shutter_time, uint32_t image_width,
    uint32_t image_height, uint32_t tile_size, uint32_t tile_width, uint32_t tile_height,
    const int32_t *tile_offsets, const int32_t *flatten_ids, void *workspace, size_t workspace_bytes,
    int64_t *chunk_starts, int64_t *host_total, void *stream);
int splatad_rasterize_to_indices_in_range_write(
    uint32_t range_start, uint32_t range_end, uint32_t C, uint32_t N, int64_t n_isects,
    const float *transmittances, const float *means2d, const float *conics, const float *opacities,
    const float *pix_vels, const float *rolling_shutter_time, uint32_t image_width,
    uint32_t image_height, uint32_t tile_size, uint32_t tile_width, uint32_t tile_height,
    const int32_t *tile_offsets, const int32_t *flatten_ids, const int64_t *chunk_starts,
    int64_t *gaussian_ids, int64_t *pixel_ids, int64_t *camera_ids, void *stream);
/* Lidar: raster_pts [C,H,W,4], pix_vels [C,N,3]; points with range <= 0 list nothing. */
int splatad_rasterize_to_indices_in_range_lidar_count(
    uint32_t range_start, uint32_t range_end, uint32_t C, uint32_t N, int64_t n_isects,
    const float *transmittances, const float *means2d, const float *conics, const float *opacities,
    const float *pix_vels, const float *raster_pts, uint32_t image_width, uint32_t image_height,
    uint32_t tile_width, uint32_t tile_height, uint32_t tile_grid_width, uint32_t tile_grid_height,
    const int32_t *tile_offsets, const int32_t *flatten_ids, void *workspace, size_t workspace_bytes,
    int64_t *chunk_starts, int64_t *host_total, void *stream);
int splatad_rasterize_to_indices_in_range_lidar_write(
    uint32_t range_start, uint32_t range_end, uint32_t C, uint32_t N, int64_t n_isects,
    const float *transmittances, const float *means2d, const float *conics, const float *opacities,
    const float *pix_vels, const float *raster_pts, uint32_t image_width, uint32_t image_height,
    uint32_t tile_width, uint32_t tile_height, uint32_t tile_grid_width, uint32_t tile_grid_height,
    const int32_t *tile_offsets, const int32_t *flatten_ids, const int64_t *chunk_starts,
    int64_t *gaussian_ids, int64_t *pixel_ids, int64_t *camera_ids, void *stream);

/* Measurement aid (no counterpart in the reference): walks every pixel's (point's) whole tile list
 * from transmittance `transmittances` [C,H,W] exactly as the compositing kernels do and adds up
 * counters[0] = (pixel, Gaussian) pairs evaluated (the one a pixel stops at included) and
 * counters[1] = pairs blended; pixel_counts [C*H*W] receives the blended pairs per pixel. These
 * are the "tested" and "contributing" pair counts of the compositing flop model. counters is a
 * device array of two uint64, zeroed by the call. */
int splatad_count_composited_pairs(
    uint32_t C, uint32_t N, int64_t n_isects, const float *transmittances, const float *means2d,
    const float *conics, const float *opacities, const float *pix_vels, const float *rolling_shutter_time,
    uint32_t image_width, uint32_t image_height, uint32_t tile_size, uint32_t tile_width, uint32_t tile_height,
    const int32_t *tile_offsets, const int32_t *flatten_ids, int32_t *pixel_counts, uint64_t *counters,
    void *stream);
int splatad_count_composited_pairs_lidar(
    uint32_t C, uint32_t N, int64_t n_isects, const float *transmittances, const float *means2d,
    const float *conics, const float *opacities, const float *pix_vels, const float *raster_pts,
    uint32_t image_width, uint32_t image_height, uint32_t tile_width, uint32_t tile_height,
    uint32_t tile_grid_width, uint32_t tile_grid_height, const int32_t *tile_offsets,
    const int32_t *flatten_ids, int32_t *pixel_counts, uint64_t *counters, void *stream);

/* ------------------------------------------------------------------------------------------
 * Densification hooks: what the training strategies do with the render path's outputs.
 * ---------------------------------------------------------------------------------------- */

/* DefaultStrategy._update_state - gsplat/strategy/default.py:203-258, fused. grads [total,2] is
 * means2d.grad or means2d.absgrad, radii [total,2] int32. gaussian_ids NULL: the [C,N] layout
 * (total = C * N; entries with radii[.,0] > 0 take part, Gaussian = entry % N); otherwise the
 * packed layout (int64 [total]). Accumulates into grad2d [N], count [N] and, unless NULL,
 * radii_state [N] (a true maximum, normalised by max(width, height)). */
int splatad_densify_update_state(
    uint64_t total, uint32_t N, const float *grads, const int32_t *radii, const int64_t *gaussian_ids,
    uint32_t image_width, uint32_t image_height, uint32_t n_cameras, float *grad2d, float *count,
    float *radii_state, void *stream);

/* compute_relocation_tensor - gsplat/cuda/csrc/relocation.cu:33-53 (kernel 4-31). ratios int32
 * [N] (clamped to 1..n_max), binoms [n_max,n_max]; outputs new_opacities [N], new_scales [N,3]. */
int splatad_compute_relocation(uint32_t N, const float *opacities, const float *scales,
                               const int32_t *ratios, const float *binoms, int32_t n_max,
                               float *new_opacities, float *new_scales, void *stream);

/* ------------------------------------------------------------------------------------------
 * Checks for hosts without a memory checker (no counterpart in the reference)
 * ---------------------------------------------------------------------------------------- */

/* The lidar forward projection prefetches its next slab of Gaussians with bulk asynchronous copies
 * and waits for them with a bounded number of polls; a wait that runs into its limit makes the
 * thread block give up (its outputs stay unwritten) and is counted. *count receives the number of
 * such give-ups since the last call, which resets it; 0 in any healthy run. Synchronises the device. */
int splatad_async_copy_timeouts(int64_t *count);

/* Validates the index lists the compositing kernels follow, without following them: every
 * flatten id of the listed part (up to tile_offsets[n_tiles] when total_follows, else n_isects)
 * is in [0, n_rows); tile_offsets (optional, [n_tiles] or [n_tiles + 1] with total_follows) are
 * non-decreasing and within [0, n_isects]; packed ids (optional, [n_packed]) are in range.
 * report (device, 4 x uint64, zeroed by the caller) receives {violations, site, index, limit} with
 * the last three describing the first violation seen (site 1 flatten id, 2 offsets out of order,
 * 3 offset out of range, 4 Gaussian id, 5 sensor id). Nothing is dereferenced through a bad index. */
int splatad_debug_validate_lists(int64_t n_isects, const int32_t *flatten_ids, uint64_t n_rows,
                                 const int32_t *tile_offsets, uint32_t n_tiles, int32_t total_follows,
                                 const int64_t *sensor_ids, const int64_t *gaussian_ids, uint64_t n_packed,
                                 uint32_t n_sensors, uint64_t n_gaussians, uint64_t *report, void *stream);

/* ------------------------------------------------------------------------------------------
 * Whole frame in one call
 * ---------------------------------------------------------------------------------------- */

/* The forward pass of lidar_rasterization (gsplat/rendering.py:443-819, classic mode, quats /
 * scales, D + 1 <= 32 channels) as ONE call: splatad_lidar_projection_fwd,
 * splatad_isect_lidar_tiles_plan / _fill at the given `capacity` and
 * splatad_rasterize_to_points_fwd (range channel taken from `depths`) enqueued back to back on
 * `stream` - same kernels, same results, one crossing of the language boundary per frame.
 * opacities_cn is [C, N] (the per-sensor opacities the compositing reads); lidar_features
 * [C, N, D]; every output, intermediate and workspace is the caller's: radii .. tiles_per_gauss as
 * in the projection / plan calls, isect_ids / flatten_ids [capacity], tile_offsets
 * [C * tiles + 1], images [C, H, W, .]. host_counts (pinned, 4 x int64) receives
 * {n_isects, n_visible, status, 0} once the stream has passed the plan: if n_isects > capacity the
 * lists and images are incomplete and the frame has to be repeated with more room.
 * early_count_pair / early_count_sequence (optional): see splatad_isect_set_early_count - the count
 * reaches the host while the depth sort, the fill and the compositing are still running. */
int splatad_lidar_frame_fwd(
    uint32_t C, uint32_t N, const float *means, const float *quats, const float *scales,
    const float *velocities, const float *opacities_cn, const float *lidar_features, uint32_t n_features,
    const float *viewmats, const float *linear_velocity, const float *angular_velocity,
    const float *rolling_shutter_time, const float *raster_pts, uint32_t image_width, uint32_t image_height,
    const float *elev_boundaries, uint32_t n_boundaries, float azimuth_resolution, uint32_t tile_width,
    uint32_t tile_height, float min_azimuth, float max_azimuth, float min_elevation, float max_elevation,
    float eps2d, float near_plane, float far_plane, float radius_clip, int32_t compute_alpha_sum,
    float alpha_sum_threshold, float *radii, float *means2d, float *depths, float *conics, float *pix_vels,
    float *depth_compensations, int32_t *tiles_per_gauss, int64_t capacity, int64_t *isect_ids,
    int32_t *flatten_ids, int32_t *tile_offsets, float *render_features, float *render_alphas,
    float *alpha_sum_until_points, int32_t *last_ids, float *median_depths, void *plan_workspace,
    size_t plan_workspace_bytes, void *fill_workspace, size_t fill_workspace_bytes, int64_t *host_counts,
    int64_t *early_count_pair, int64_t early_count_sequence, void *stream);

/* ------------------------------------------------------------------------------------------
 * Gaussian-sharded exchange (one process per GPU): every rank projects its slice of the Gaussians
 * for all sensors and sends the visible (sensor, Gaussian) records to the rank owning the sensor.
 * The reference leaves this to torch code around its collectives (gsplat/distributed.py:170-257:
 * all_to_all_int32 size exchange + all_to_all_tensor_list row exchange); these entry points build
 * the fixed-width send rows on the device and place received rows in single-GPU order. The
 * transport itself (one all-to-all of [rows, width] 32-bit words) stays with the caller.
 * ---------------------------------------------------------------------------------------- */

/* Which pairs of a [C, N] projection travel: those with radii[c, n, 0] > 0 (radii [C,N,2], float
 * degrees or int32 pixels - the sign test is the same on either bit pattern). _count writes
 * indptr [C+1] (first row of every sensor, total last) and *total_device (may be NULL); _fill
 * writes row_index[k] = c * N + n of the k-th pair in (sensor, Gaussian) order, dropping rows at
 * or beyond `capacity`. workspace: splatad_visible_rows_workspace_bytes(C, N) bytes, shared by
 * the two calls. C * N must fit int32. */
size_t splatad_visible_rows_workspace_bytes(uint32_t C, uint32_t N);
int splatad_visible_rows_count(uint32_t C, uint32_t N, const void *radii, void *workspace,
                               size_t workspace_bytes, int32_t *indptr, int64_t *total_device,
                               void *stream);
int splatad_visible_rows_fill(uint32_t C, uint32_t N, const void *radii, const void *workspace,
                              int64_t capacity, int32_t *row_index, void *stream);

/* out[i, :] = concatenation over the fields k of field_ptrs[k][index[i], 0:field_widths[k]]
 * (index NULL: row i). Fields are arrays of 32-bit words (float or int32), at most 12; a NULL
 * field pointer yields zeros. With sensor_table (int32 [C]) two id columns lead every row: the
 * global sensor id sensor_table[index[i] / n_per_sensor] and the global Gaussian id
 * gaussian_start + index[i] % n_per_sensor, as int32 bit patterns. field_ptrs / field_widths are
 * HOST arrays read during the call. */
int splatad_rows_gather(int64_t n_rows, const int32_t *index, int32_t n_fields,
                        const void *const *field_ptrs, const int32_t *field_widths,
                        const int32_t *sensor_table, uint32_t n_per_sensor, int32_t gaussian_start,
                        void *out, void *stream);

/* The inverse placement: field_ptrs[k][index[i], :] = columns of field k of in[i, :] (index NULL:
 * row i; index must not repeat a row). id_cols = 2 widens the two leading id columns to int64
 * into sensor_ids_out / gaussian_ids_out (either may be NULL), id_cols = 0 means rows without
 * them. A NULL field pointer skips that field. */
int splatad_rows_scatter(int64_t n_rows, const int32_t *index, int32_t n_fields,
                         void *const *field_ptrs, const int32_t *field_widths, int32_t id_cols,
                         int64_t *sensor_ids_out, int64_t *gaussian_ids_out, const void *in,
                         void *stream);

/* Received rows arrive as n_segments <= 128 contiguous segments, one per (source rank, owned
 * sensor) with the sensor index running fastest (n_sensors per source); segment s begins at row
 * src_start[s] of the receive buffer (ascending) and at row dst_start[s] of the final (sensor,
 * source rank) order. src_start / dst_start are HOST arrays read during the call. row_map[i] =
 * final row of received row i, for splatad_rows_scatter; local_sensor_ids (optional, int64
 * [n_rows]) receives, per FINAL row, the index of its sensor among the owned sensors. */
int splatad_segment_row_map(int32_t n_segments, int32_t n_sensors, const int64_t *src_start,
                            const int64_t *dst_start, int64_t n_rows, int32_t *row_map,
                            int64_t *local_sensor_ids, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* SPLATAD_B200_H */
