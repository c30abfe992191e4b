// Whole-frame entry points: one call enqueues every kernel of a forward render - projection, tile
// intersection (plan + fill at a caller-chosen capacity) and compositing - on one stream, with all
// outputs, intermediates and workspaces supplied by the caller. Same kernels and results as the
// individual entry points called in sequence (gsplat/rendering.py:616-819 is the reference's
// orchestration of the lidar frame); what goes away is the host work between the launches, which
// is what bounds the frame rate once a frame takes less than half a millisecond on the device.
#include "common.cuh"

using namespace splatad;

extern "C" int splatad_lidar_frame_fwd(
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
    int64_t *early_count_pair, int64_t early_count_sequence, void *stream) {
    SPL_REQUIRE(C > 0 && N > 0 && image_width > 0 && image_height > 0, SPLATAD_ERR_BAD_ARG,
                "lidar_frame_fwd: empty input");
    SPL_REQUIRE(n_features + 1 <= SPLATAD_MAX_CHANNELS, SPLATAD_ERR_CHANNELS,
                "lidar_frame_fwd: %u features + range exceed %d channels; render in chunks with the individual "
                "entry points", n_features, SPLATAD_MAX_CHANNELS);
    SPL_REQUIRE(opacities_cn && tile_offsets && capacity > 0 && host_counts, SPLATAD_ERR_BAD_ARG,
                "lidar_frame_fwd: null argument");
    int rc = splatad_lidar_projection_fwd(C, N, means, nullptr, quats, scales, velocities, viewmats, min_elevation,
                                          max_elevation, min_azimuth, max_azimuth, linear_velocity,
                                          angular_velocity, rolling_shutter_time, eps2d, near_plane, far_plane,
                                          radius_clip, radii, means2d, depths, conics, nullptr, pix_vels,
                                          depth_compensations, stream);
    if (rc != SPLATAD_OK) return rc;
    const float tile_azim_res = azimuth_resolution * (float)tile_width;
    const uint64_t total = (uint64_t)C * N;
    splatad_isect_set_early_count(early_count_pair, early_count_sequence);
    rc = splatad_isect_lidar_tiles_plan(C, N, total, means2d, radii, depths, nullptr, elev_boundaries, n_boundaries,
                                        tile_azim_res, min_azimuth, 1, tiles_per_gauss, plan_workspace,
                                        plan_workspace_bytes, host_counts, stream);
    splatad_isect_set_early_count(nullptr, 0);
    if (rc != SPLATAD_OK) return rc;
    rc = splatad_isect_lidar_tiles_fill(C, N, total, means2d, radii, depths, nullptr, elev_boundaries, n_boundaries,
                                        tile_azim_res, min_azimuth, 1, tiles_per_gauss, plan_workspace,
                                        fill_workspace, fill_workspace_bytes, capacity, isect_ids, flatten_ids,
                                        tile_offsets, nullptr, stream);
    if (rc != SPLATAD_OK) return rc;
    const uint32_t grid_w = splatad_lidar_azimuth_tiles(tile_azim_res);
    const uint32_t grid_h = n_boundaries - 1;
    // n_isects = -1: the end of the last tile is read from tile_offsets[C * tiles], written by the fill
    return splatad_rasterize_to_points_fwd(C, -1, means2d, conics, lidar_features, depths, n_features + 1,
                                           opacities_cn, pix_vels, depth_compensations, nullptr, raster_pts,
                                           image_width, image_height, tile_width, tile_height, grid_w, grid_h,
                                           compute_alpha_sum, alpha_sum_threshold, tile_offsets, flatten_ids,
                                           n_features, render_features, render_alphas, alpha_sum_until_points,
                                           last_ids, median_depths, stream);
}
