"""``rasterization()`` and ``lidar_rasterization()``: drop-in replacements for the two render
entry points of the reference (gsplat/rendering.py:22-440 and 443-819) with the same
signatures, return tuples and ``meta`` keys, running on the B200 CUDA library of this package.

Both are orchestration only: project -> (spherical harmonics) -> tile intersection -> per-tile
offsets -> compositing, with the channel chunking rules of the reference.
"""

from __future__ import annotations

import math
from typing import Dict, Optional, Tuple, Union

import torch
from torch import Tensor

try:  # Python >= 3.8 has Literal in typing; keep the reference's import order of preference
    from typing_extensions import Literal
except ImportError:  # pragma: no cover
    from typing import Literal

from .ops import (
    PendingPackedCount,
    lidar_frame_fwd,
    camera_centers,
    fully_fused_lidar_projection,
    fully_fused_projection,
    gather_rows,
    isect_lidar_tiles_deferred,
    isect_tiles_deferred,
    rasterize_to_pixels,
    rasterize_to_points,
    rasterize_to_points_split,
    view_dependent_colors,
)


def _check_gaussians(means: Tensor, quats: Tensor, scales: Tensor, opacities: Tensor,
                     velocities: Optional[Tensor], viewmats: Tensor) -> Tuple[int, int]:
    """Shape checks shared by both entry points; returns (N, C)."""
    N, C = means.shape[0], viewmats.shape[0]
    for name, tensor, shape in (("means", means, (N, 3)), ("quats", quats, (N, 4)), ("scales", scales, (N, 3)),
                                ("opacities", opacities, (N,)), ("viewmats", viewmats, (C, 4, 4))):
        assert tensor.shape == shape, f"{name}: {tuple(tensor.shape)}"
    if velocities is not None:
        assert velocities.shape == (N, 3), velocities.shape
    return N, C


def _sensor_motion(C: int, device, linear_velocity: Optional[Tensor], angular_velocity: Optional[Tensor],
                   rolling_shutter_time: Optional[Tensor]) -> Tuple[Tensor, Tensor, Tensor]:
    """Ego motion of the C sensors during read-out; a sensor without one stands still."""
    out = []
    for value, shape in ((linear_velocity, (C, 3)), (angular_velocity, (C, 3)), (rolling_shutter_time, (C,))):
        if value is None:
            value = torch.zeros(shape, device=device)
        assert value.shape == shape, value.shape
        out.append(value)
    return tuple(out)


def _composite_with_count_check(isect, grid: Tuple[int, int], composite):
    """Runs ``composite(isect_offsets, flatten_ids, total_follows)`` on a deferred tile intersection and returns
    (outputs, isect_ids, flatten_ids, isect_offsets): if the intersection count turns out to exceed
    the room it was given, intersection and compositing are repeated the two-step way."""
    outputs = composite(isect.offsets(*grid), isect.flatten_ids, isect.total_follows(*grid))
    resolved = isect.resolve()
    if resolved is None:
        isect = isect.redo()
        outputs = composite(isect.offsets(*grid), isect.flatten_ids, isect.total_follows(*grid))
        resolved = isect.resolve()
    return outputs, resolved[0], resolved[1], isect.offsets(*grid), isect.tiles_per_gauss


def rasterization(
    means: Tensor,  # [N, 3]
    quats: Tensor,  # [N, 4]
    scales: Tensor,  # [N, 3]
    opacities: Tensor,  # [N]
    colors: Tensor,  # [(C,) N, D] or [(C,) N, K, 3]
    velocities: Optional[Tensor],  # [N, 3]
    viewmats: Tensor,  # [C, 4, 4]
    Ks: Tensor,  # [C, 3, 3]
    width: int,
    height: int,
    linear_velocity: Optional[Tensor] = None,  # [C, 3]
    angular_velocity: Optional[Tensor] = None,  # [C, 3]
    rolling_shutter_time: Optional[Tensor] = None,  # [C]
    near_plane: float = 0.01,
    far_plane: float = 1e10,
    radius_clip: float = 0.0,
    eps2d: float = 0.3,
    sh_degree: Optional[int] = None,
    packed: bool = True,
    tile_size: int = 16,
    backgrounds: Optional[Tensor] = None,
    render_mode: Literal["RGB", "D", "ED", "RGB+D", "RGB+ED"] = "RGB",
    sparse_grad: bool = False,
    absgrad: bool = False,
    rasterize_mode: Literal["classic", "antialiased"] = "classic",
    channel_chunk: int = 32,
) -> Tuple[Tensor, Tensor, Dict]:
    """Rasterizes N 3-D Gaussians to C rolling-shutter pinhole cameras.

    Arguments, defaults and behaviour are those of the reference function of the same name
    (gsplat/rendering.py:22-440): ``colors`` is [(C,) N, D] post-activation values, or
    [(C,) N, K, 3] SH coefficients when ``sh_degree`` is given; ``render_mode`` selects colour
    and / or (expected) depth as the last channel; ``packed`` selects COO intermediates;
    ``rasterize_mode="antialiased"`` multiplies opacities by the blur compensation;
    ``absgrad`` stores |d loss / d means2d| in ``meta["means2d"].absgrad`` during backward.

    Returns (render_colors [C,H,W,X], render_alphas [C,H,W,1], meta).
    """
    args = (means, quats, scales, opacities, colors, velocities, viewmats, Ks, width, height, linear_velocity,
            angular_velocity, rolling_shutter_time, near_plane, far_plane, radius_clip, eps2d, sh_degree, packed,
            tile_size, backgrounds, render_mode, sparse_grad, absgrad, rasterize_mode, channel_chunk)
    # packed: the frame is enqueued without waiting for the number of packed rows (once a frame of
    # this shape has been seen); if the rows outgrow the room they were given, the frame is redone
    out = _rasterization(*args, wait_for_packed_count=not packed)
    return out if out is not None else _rasterization(*args, wait_for_packed_count=True)


def _rasterization(means, quats, scales, opacities, colors, velocities, viewmats, Ks, width, height,
                   linear_velocity, angular_velocity, rolling_shutter_time, near_plane, far_plane, radius_clip,
                   eps2d, sh_degree, packed, tile_size, backgrounds, render_mode, sparse_grad, absgrad,
                   rasterize_mode, channel_chunk, wait_for_packed_count):
    N, C = _check_gaussians(means, quats, scales, opacities, velocities, viewmats)
    assert Ks.shape == (C, 3, 3), Ks.shape
    assert render_mode in ("RGB", "D", "ED", "RGB+D", "RGB+ED"), render_mode
    linear_velocity, angular_velocity, rolling_shutter_time = _sensor_motion(
        C, means.device, linear_velocity, angular_velocity, rolling_shutter_time)

    if sh_degree is None:
        assert (colors.dim() == 2 and colors.shape[0] == N) or (
            colors.dim() == 3 and colors.shape[:2] == (C, N)
        ), colors.shape
    else:
        assert (colors.dim() == 3 and colors.shape[0] == N and colors.shape[2] == 3) or (
            colors.dim() == 4 and colors.shape[:2] == (C, N) and colors.shape[3] == 3
        ), colors.shape
        assert (sh_degree + 1) ** 2 <= colors.shape[-2], colors.shape

    pending = None if wait_for_packed_count else PendingPackedCount()
    proj_results = fully_fused_projection(
        means, None, quats, scales, velocities, viewmats, Ks, width, height, linear_velocity,
        angular_velocity, rolling_shutter_time, eps2d=eps2d, packed=packed, near_plane=near_plane,
        far_plane=far_plane, radius_clip=radius_clip, sparse_grad=sparse_grad,
        calc_compensations=(rasterize_mode == "antialiased"), pending=pending,
    )
    if packed:
        (camera_ids, gaussian_ids, radii, means2d, depths, conics, compensations, pix_vels) = proj_results
        opacities = gather_rows(opacities, gaussian_ids)  # [nnz]
    else:
        radii, means2d, depths, conics, compensations, pix_vels = proj_results
        opacities = opacities[None] if C == 1 else opacities.repeat(C, 1)  # [C, N], no copy for one sensor
        camera_ids, gaussian_ids = None, None

    if compensations is not None:
        opacities = opacities * compensations

    tile_width = math.ceil(width / float(tile_size))
    tile_height = math.ceil(height / float(tile_size))
    # plan + fill are enqueued without waiting for the intersection count (once a frame of this
    # shape has been seen); the exact-length isect_ids / flatten_ids are cut out after compositing
    isect = isect_tiles_deferred(means2d, radii, depths, tile_size, tile_width, tile_height, packed=packed,
                                 n_cameras=C, camera_ids=camera_ids, gaussian_ids=gaussian_ids)

    if sh_degree is None:
        if packed:
            if colors.dim() == 2:
                colors = gather_rows(colors, gaussian_ids)
            else:
                colors = colors[camera_ids, gaussian_ids]
        else:
            if colors.dim() == 2:
                colors = colors.expand(C, -1, -1)
    else:
        # camera centres (the translation of inverse(viewmats)), then gathers, directions, SH, + 0.5,
        # clamp and the depth channel in one kernel
        colors = view_dependent_colors(
            sh_degree, means, camera_centers(viewmats), colors, radii, camera_ids, gaussian_ids,
            depths=depths if render_mode in ["RGB+D", "RGB+ED"] else None)

    if render_mode in ["RGB+D", "RGB+ED"]:
        if sh_degree is None:
            colors = torch.cat((colors, depths[..., None]), dim=-1)
        if backgrounds is not None:
            backgrounds = torch.cat([backgrounds, torch.zeros(C, 1, device=backgrounds.device)], dim=-1)
    elif render_mode in ["D", "ED"]:
        colors = depths[..., None]
        if backgrounds is not None:
            backgrounds = torch.zeros(C, 1, device=backgrounds.device)

    tiles_per_gauss_cut = None
    if pending is not None and pending.active:
        # everything up to here ran on padded rows; the count has long arrived by now
        nnz = pending.resolve()
        if nnz is None:
            return None
        camera_ids, gaussian_ids, radii = camera_ids[:nnz], gaussian_ids[:nnz], radii[:nnz]
        means2d, depths, conics, pix_vels = means2d[:nnz], depths[:nnz], conics[:nnz], pix_vels[:nnz]
        opacities, colors = opacities[:nnz], colors[:nnz]
        tiles_per_gauss_cut = nnz

    def composite(isect_offsets, flatten_ids, total_follows):
        if colors.shape[-1] > channel_chunk:
            n_chunks = (colors.shape[-1] + channel_chunk - 1) // channel_chunk
            chunk_colors, chunk_alphas = [], []
            for i in range(n_chunks):
                colors_chunk = colors[..., i * channel_chunk : (i + 1) * channel_chunk]
                backgrounds_chunk = (
                    backgrounds[..., i * channel_chunk : (i + 1) * channel_chunk]
                    if backgrounds is not None
                    else None
                )
                render_colors_, render_alphas_ = rasterize_to_pixels(
                    means2d, conics, colors_chunk, opacities, pix_vels, width, height, tile_size,
                    isect_offsets, flatten_ids, rolling_shutter_time, backgrounds=backgrounds_chunk,
                    packed=packed, absgrad=absgrad, total_follows=total_follows,
                )
                chunk_colors.append(render_colors_)
                chunk_alphas.append(render_alphas_)
            return torch.cat(chunk_colors, dim=-1), chunk_alphas[0]  # alphas are the same for every chunk
        return rasterize_to_pixels(
            means2d, conics, colors, opacities, pix_vels, width, height, tile_size, isect_offsets,
            flatten_ids, rolling_shutter_time, backgrounds=backgrounds, packed=packed, absgrad=absgrad,
            total_follows=total_follows,
        )

    (render_colors, render_alphas), isect_ids, flatten_ids, isect_offsets, tiles_per_gauss = (
        _composite_with_count_check(isect, (tile_height, tile_width), composite))
    if tiles_per_gauss_cut is not None:
        tiles_per_gauss = tiles_per_gauss[:tiles_per_gauss_cut]
    if render_mode in ["ED", "RGB+ED"]:
        render_colors = torch.cat(
            [render_colors[..., :-1], render_colors[..., -1:] / render_alphas.clamp(min=1e-10)],
            dim=-1,
        )

    meta = dict(
        camera_ids=camera_ids, gaussian_ids=gaussian_ids, radii=radii, means2d=means2d, depths=depths,
        conics=conics, opacities=opacities, pix_vels=pix_vels, tile_width=tile_width, tile_height=tile_height,
        tiles_per_gauss=tiles_per_gauss, isect_ids=isect_ids, flatten_ids=flatten_ids,
        isect_offsets=isect_offsets, width=width, height=height, tile_size=tile_size, n_cameras=C,
    )
    return render_colors, render_alphas, meta


def lidar_rasterization(
    means: Tensor,  # [N, 3]
    quats: Tensor,  # [N, 4]
    scales: Tensor,  # [N, 3]
    opacities: Tensor,  # [N]
    lidar_features: Tensor,  # [C, N, D]
    velocities: Optional[Tensor],  # [N, 3]
    viewmats: Tensor,  # [C, 4, 4]
    raster_pts: Tensor,  # [C, H, W, 4]
    tile_elevation_boundaries: Tensor,  # [ceil(n_elevation_channels / tile_height) + 1]
    linear_velocity: Optional[Tensor] = None,  # [C, 3]
    angular_velocity: Optional[Tensor] = None,  # [C, 3]
    rolling_shutter_time: Optional[Tensor] = None,  # [C]
    min_azimuth: float = -180,
    max_azimuth: float = 180,
    min_elevation: float = -80,
    max_elevation: float = 80,
    n_elevation_channels: int = 32,
    azimuth_resolution: float = 0.1,
    tile_width: int = 32,
    tile_height: int = 8,
    near_plane: float = 0.01,
    far_plane: float = 1e10,
    radius_clip: float = 0.0,
    eps2d: float = 0.017,
    compute_alpha_sum_until_points: bool = True,
    compute_alpha_sum_until_points_threshold: float = 0.2,
    packed: bool = False,  # packed mode is not supported (as in the reference)
    sparse_grad: bool = False,
    absgrad: bool = False,
    rasterize_mode: Literal["classic", "antialiased"] = "classic",
    channel_chunk: int = 32,
    use_depth_compensation: bool = True,
) -> Tuple[Tensor, Tensor, Union[Tensor, None], Dict]:
    """Rasterizes N 3-D Gaussians to C spinning-lidar range images given as ``raster_pts``
    [C, H, W, 4] = (azimuth deg, elevation deg, range m, time offset s).

    Arguments, defaults and behaviour are those of the reference function of the same name
    (gsplat/rendering.py:443-819). Returns (features with the expected range appended as last
    channel [C,H,W,D+1], alphas [C,H,W,1], alpha_sum_until_points [C,H,W,1] or None, meta);
    ``meta["median_depths"]`` holds the median range.
    """
    N, C = _check_gaussians(means, quats, scales, opacities, velocities, viewmats)
    assert lidar_features.shape[:2] == (C, N) and lidar_features.dim() == 3, lidar_features.shape
    assert -180.0 <= min_azimuth < max_azimuth <= 180.0, (min_azimuth, max_azimuth)
    assert -85.0 <= min_elevation < max_elevation <= 85.0, (min_elevation, max_elevation)
    assert tile_width * tile_height <= 256, (tile_width, tile_height)
    assert n_elevation_channels > 0 and azimuth_resolution > 0.0, (n_elevation_channels, azimuth_resolution)
    n_elevation_tiles = math.ceil(n_elevation_channels / tile_height)
    assert tile_elevation_boundaries.shape == (n_elevation_tiles + 1,), tile_elevation_boundaries.shape
    assert raster_pts.dim() == 4 and raster_pts.shape[0] == C and raster_pts.shape[-1] == 4, raster_pts.shape
    if packed:
        raise NotImplementedError("Packed mode is not supported for lidar_rasterization")
    linear_velocity, angular_velocity, rolling_shutter_time = _sensor_motion(
        C, means.device, linear_velocity, angular_velocity, rolling_shutter_time)

    # A frame that fits one compositing launch and has a predecessor of its shape goes through one
    # library call that enqueues all of its forward pass (same kernels, same results). With gradients
    # wanted, the projection and compositing ops then adopt the frame's outputs - they launch nothing
    # and only put their backward passes into the graph, so that the graph, `meta` and the gradient
    # slots of `meta["means2d"]` are those of the op-by-op path.
    needs_grad = torch.is_grad_enabled() and any(
        t is not None and t.requires_grad
        for t in (means, quats, scales, opacities, lidar_features, velocities, viewmats))
    if (rasterize_mode == "classic" and use_depth_compensation
            and lidar_features.shape[-1] + 1 <= min(channel_chunk, 32) and N > 0 and C > 0
            and raster_pts.shape[1] * raster_pts.shape[2] > 0):
        with torch.no_grad():
            frame = lidar_frame_fwd(
                means, quats, scales, velocities, opacities[None] if C == 1 else opacities.repeat(C, 1),
                lidar_features, viewmats, linear_velocity, angular_velocity, rolling_shutter_time, raster_pts,
                tile_elevation_boundaries, azimuth_resolution, tile_width, tile_height, min_azimuth, max_azimuth,
                min_elevation, max_elevation, eps2d, near_plane, far_plane, radius_clip,
                compute_alpha_sum_until_points, compute_alpha_sum_until_points_threshold,
                expected_grid=(n_elevation_tiles,
                               math.ceil((max_azimuth - min_azimuth) / (azimuth_resolution * tile_width))))
        lists = frame.finish() if frame is not None else None
        if lists is not None and needs_grad:
            n_elevation_tiles_, n_azimuth_tiles_ = frame.grid
            isect_offsets = frame.offsets_buf[:-1].view(C, n_elevation_tiles_, n_azimuth_tiles_)
            radii, means2d, depths, conics, _, pix_vels, depth_compensations = fully_fused_lidar_projection(
                means, None, quats, scales, velocities, viewmats, linear_velocity, angular_velocity,
                rolling_shutter_time, min_elevation=min_elevation, max_elevation=max_elevation,
                min_azimuth=min_azimuth, max_azimuth=max_azimuth, eps2d=eps2d, packed=False,
                near_plane=near_plane, far_plane=far_plane, radius_clip=radius_clip, sparse_grad=sparse_grad,
                calc_compensations=False, frame=frame)
            opacities_cn = opacities[None] if C == 1 else opacities.repeat(C, 1)
            render, alphas, alpha_sum, median = rasterize_to_points_split(
                means2d, conics, lidar_features, depths, opacities_cn, pix_vels, depth_compensations, raster_pts,
                raster_pts.shape[-2], raster_pts.shape[-3], tile_width, tile_height, isect_offsets, lists[1],
                compute_alpha_sum_until_points, compute_alpha_sum_until_points_threshold, absgrad=absgrad,
                total_follows=True, frame=frame)
            meta = dict(
                camera_ids=None, gaussian_ids=None, radii=radii, means2d=means2d, depths=depths, conics=conics,
                opacities=opacities_cn, pix_vels=pix_vels, tile_grid_width=n_azimuth_tiles_,
                tile_grid_height=n_elevation_tiles_, tiles_per_gauss=frame.tiles_per_gauss, isect_ids=lists[0],
                flatten_ids=lists[1], isect_offsets=isect_offsets, width=raster_pts.shape[-2],
                height=raster_pts.shape[-3], tile_width=tile_width, tile_height=tile_height, n_cameras=C,
                median_depths=median,
            )
            return render, alphas, alpha_sum, meta
        if lists is not None:
            n_elevation_tiles_, n_azimuth_tiles_ = frame.grid
            meta = dict(
                camera_ids=None, gaussian_ids=None, radii=frame.radii, means2d=frame.means2d, depths=frame.depths,
                conics=frame.conics, opacities=opacities[None] if C == 1 else opacities.repeat(C, 1),
                pix_vels=frame.pix_vels, tile_grid_width=n_azimuth_tiles_, tile_grid_height=n_elevation_tiles_,
                tiles_per_gauss=frame.tiles_per_gauss, isect_ids=lists[0], flatten_ids=lists[1],
                isect_offsets=frame.offsets_buf[:-1].view(C, n_elevation_tiles_, n_azimuth_tiles_),
                width=raster_pts.shape[-2], height=raster_pts.shape[-3], tile_width=tile_width,
                tile_height=tile_height, n_cameras=C, median_depths=frame.median_depths,
            )
            return frame.render, frame.alphas, frame.alpha_sum, meta

    radii, means2d, depths, conics, compensations, pix_vels, depth_compensations = fully_fused_lidar_projection(
        means, None, quats, scales, velocities, viewmats, linear_velocity, angular_velocity,
        rolling_shutter_time, min_elevation=min_elevation, max_elevation=max_elevation,
        min_azimuth=min_azimuth, max_azimuth=max_azimuth, eps2d=eps2d, packed=False, near_plane=near_plane,
        far_plane=far_plane, radius_clip=radius_clip, sparse_grad=sparse_grad,
        calc_compensations=(rasterize_mode == "antialiased"),
    )
    opacities = opacities[None] if C == 1 else opacities.repeat(C, 1)  # [C, N], no copy for one sensor
    camera_ids, gaussian_ids = None, None

    if not use_depth_compensation:
        depth_compensations = depth_compensations * 0

    if compensations is not None:
        opacities = opacities * compensations

    tile_azimuth_resolution = azimuth_resolution * tile_width
    n_azimuth_tiles = math.ceil((max_azimuth - min_azimuth) / tile_azimuth_resolution)
    # plan + fill are enqueued without waiting for the intersection count (once a frame of this
    # shape has been seen); the exact-length isect_ids / flatten_ids are cut out after compositing
    isect = isect_lidar_tiles_deferred(
        means2d, radii, depths, elev_boundaries=tile_elevation_boundaries,
        tile_azim_resolution=tile_azimuth_resolution, min_azim=min_azimuth, packed=False, n_cameras=C)

    image_width = raster_pts.shape[-2]
    image_height = raster_pts.shape[-3]

    def composite(isect_offsets, flatten_ids, total_follows):
        common = dict(
            compute_alpha_sum_until_points=compute_alpha_sum_until_points,
            compute_alpha_sum_until_points_threshold=compute_alpha_sum_until_points_threshold,
            absgrad=absgrad,
            total_follows=total_follows,
        )
        geometry = (raster_pts, image_width, image_height, tile_width, tile_height, isect_offsets, flatten_ids)
        if (lidar_features.shape[-1] + 1) <= channel_chunk:
            # one launch: the range channel is read from `depths` directly (no [C,N,D+1] concatenation)
            return rasterize_to_points_split(
                means2d, conics, lidar_features, depths, opacities, pix_vels, depth_compensations,
                *geometry, **common,
            )
        # every chunk carries channel_chunk - 1 features and the range as its last channel
        n_chunks = (lidar_features.shape[-1] + channel_chunk) // channel_chunk
        chunks, medians, first = [], [], None
        for i in range(n_chunks):
            lidar_features_chunk = lidar_features[..., i * (channel_chunk - 1) : (i + 1) * (channel_chunk - 1)]
            features_, alphas_, alpha_sum_, median_ = rasterize_to_points(
                means2d, conics, torch.cat([lidar_features_chunk, depths[..., None]], dim=-1), opacities,
                pix_vels, depth_compensations, *geometry, packed=packed, **common,
            )
            chunks.append(features_ if i == n_chunks - 1 else features_[..., :-1])
            medians.append(median_)
            if first is None:
                first = (alphas_, alpha_sum_)  # the same for every chunk
        return torch.cat(chunks, dim=-1), first[0], first[1], torch.cat(medians, dim=-1)

    (render_lidar_features, render_alphas, alpha_sum_until_points, median_depths), isect_ids, flatten_ids, \
        isect_offsets, tiles_per_gauss = _composite_with_count_check(
            isect, (n_elevation_tiles, n_azimuth_tiles), composite)

    meta = dict(
        camera_ids=camera_ids, gaussian_ids=gaussian_ids, radii=radii, means2d=means2d, depths=depths,
        conics=conics, opacities=opacities, pix_vels=pix_vels, tile_grid_width=n_azimuth_tiles,
        tile_grid_height=n_elevation_tiles, tiles_per_gauss=tiles_per_gauss, isect_ids=isect_ids,
        flatten_ids=flatten_ids, isect_offsets=isect_offsets, width=image_width, height=image_height,
        tile_width=tile_width, tile_height=tile_height, n_cameras=C, median_depths=median_depths,
    )
    return render_lidar_features, render_alphas, alpha_sum_until_points, meta
