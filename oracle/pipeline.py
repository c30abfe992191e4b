"""End-to-end CPU restatement of ``lidar_rasterization`` and ``rasterization`` assembled from the
oracle pieces. TEST INFRASTRUCTURE ONLY - see ``oracle/__init__.py``. Also the CPU baseline
timed by ``bench.py`` (the reference has no CPU backend for these two functions: its torch
compositing calls CUDA kernels, so the compositing leg is this restatement).

Orchestration follows gsplat/rendering.py:205-440 (camera) and 616-819 (lidar).
"""

from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np
import torch

from . import composite, isect, projection


def _np(t):
    return None if t is None else t.detach().cpu().numpy()


def _zeros(C, n, ref):
    return torch.zeros(C, n, dtype=ref.dtype)


def lidar_rasterization(
    means, quats, scales, opacities, lidar_features, velocities, viewmats, raster_pts,
    tile_elevation_boundaries, linear_velocity=None, angular_velocity=None, rolling_shutter_time=None,
    min_azimuth=-180, max_azimuth=180, min_elevation=-80, max_elevation=80, n_elevation_channels=32,
    azimuth_resolution=0.1, tile_width=32, tile_height=8, near_plane=0.01, far_plane=1e10,
    radius_clip=0.0, eps2d=0.017, compute_alpha_sum_until_points=True,
    compute_alpha_sum_until_points_threshold=0.2, rasterize_mode="classic", use_depth_compensation=True,
    dtype=np.float32, timings: Optional[Dict] = None,
):
    """CPU lidar render. Returns (features+range [C,H,W,D+1], alphas, alpha_sum, meta) as numpy;
    ``meta`` additionally carries ``ambiguous`` (see oracle/composite_impl.h), ``tested`` and
    ``contributing`` pair counts."""
    import time

    tdt = torch.float32 if dtype == np.float32 else torch.float64
    cast = lambda x: None if x is None else torch.as_tensor(x).to(tdt)  # noqa: E731
    C = viewmats.shape[0]
    lin = cast(linear_velocity) if linear_velocity is not None else torch.zeros(C, 3, dtype=tdt)
    ang = cast(angular_velocity) if angular_velocity is not None else torch.zeros(C, 3, dtype=tdt)
    rs = cast(rolling_shutter_time) if rolling_shutter_time is not None else torch.zeros(C, dtype=tdt)
    t0 = time.perf_counter()
    with torch.no_grad():
        radii, means2d, depths, conics, comps, pix_vels, dcomp = projection.fully_fused_lidar_projection(
            cast(means), None, cast(quats), cast(scales), cast(velocities), cast(viewmats), lin, ang, rs,
            min_elevation, max_elevation, min_azimuth, max_azimuth, eps2d, near_plane, far_plane,
            radius_clip, rasterize_mode == "antialiased")
    opac = cast(opacities)[None].repeat(C, 1)
    if comps is not None:
        opac = opac * comps
    if not use_depth_compensation:
        dcomp = dcomp * 0
    t1 = time.perf_counter()
    n_el = math.ceil(n_elevation_channels / tile_height)
    tile_az = azimuth_resolution * tile_width
    n_az = math.ceil((max_azimuth - min_azimuth) / tile_az)
    r32 = _np(radii).astype(np.float32)
    m32 = _np(means2d).astype(np.float32)
    d32 = _np(depths).astype(np.float32)
    tpg, ids, flat = isect.isect_lidar_tiles(m32, r32, d32, _np(torch.as_tensor(tile_elevation_boundaries)),
                                             tile_az, min_azimuth)
    offsets = isect.isect_offset_encode(ids, C, n_az, n_el)
    t2 = time.perf_counter()
    H, W = raster_pts.shape[1:3]
    feats = torch.cat([cast(lidar_features), depths[..., None]], dim=-1)
    out = composite.rasterize_to_points_fwd(
        _np(means2d), _np(conics), _np(feats), _np(opac), _np(pix_vels), _np(dcomp), None,
        _np(torch.as_tensor(raster_pts)), W, H, tile_width, tile_height, offsets, flat,
        compute_alpha_sum_until_points, compute_alpha_sum_until_points_threshold, dtype=dtype)
    t3 = time.perf_counter()
    if timings is not None:
        timings.update(projection=t1 - t0, isect=t2 - t1, composite=t3 - t2, total=t3 - t0)
    meta = dict(radii=_np(radii), means2d=_np(means2d), depths=_np(depths), conics=_np(conics),
                opacities=_np(opac), pix_vels=_np(pix_vels), depth_compensations=_np(dcomp),
                tiles_per_gauss=tpg, isect_ids=ids, flatten_ids=flat, isect_offsets=offsets,
                tile_grid_width=n_az, tile_grid_height=n_el, median_depths=out["median_depths"],
                last_ids=out["last_ids"], ambiguous=out["ambiguous"], tested=out["tested"],
                contributing=out["contributing"])
    return out["render_colors"], out["render_alphas"], out["alpha_sum"], meta


def lidar_from_projection(radii, means2d, depths, conics, opacities, pix_vels, depth_compensations,
                          lidar_features, raster_pts, tile_elevation_boundaries, min_azimuth=-180,
                          max_azimuth=180, n_elevation_channels=32, azimuth_resolution=0.1, tile_width=32,
                          tile_height=8, compute_alpha_sum_until_points=True,
                          compute_alpha_sum_until_points_threshold=0.2, dtype=np.float32):
    """Tile intersection + compositing of the oracle on GIVEN projection outputs ([C,N,..] numpy
    arrays, e.g. the product's own), so that the list stages are compared on identical inputs.
    Returns dict(tiles_per_gauss, isect_ids, flatten_ids, isect_offsets, out=<composite dict>)."""
    C = means2d.shape[0]
    n_el = math.ceil(n_elevation_channels / tile_height)
    tile_az = azimuth_resolution * tile_width
    n_az = math.ceil((max_azimuth - min_azimuth) / tile_az)
    tpg, ids, flat = isect.isect_lidar_tiles(np.asarray(means2d, np.float32), np.asarray(radii, np.float32),
                                             np.asarray(depths, np.float32),
                                             np.asarray(tile_elevation_boundaries, np.float32), tile_az,
                                             min_azimuth)
    offsets = isect.isect_offset_encode(ids, C, n_az, n_el)
    H, W = raster_pts.shape[1:3]
    feats = np.concatenate([np.asarray(lidar_features), np.asarray(depths)[..., None]], axis=-1)
    out = composite.rasterize_to_points_fwd(means2d, conics, feats, opacities, pix_vels, depth_compensations,
                                            None, np.asarray(raster_pts), W, H, tile_width, tile_height, offsets,
                                            flat, compute_alpha_sum_until_points,
                                            compute_alpha_sum_until_points_threshold, dtype=dtype)
    return dict(tiles_per_gauss=tpg, isect_ids=ids, flatten_ids=flat, isect_offsets=offsets, out=out)


def camera_from_projection(radii, means2d, depths, conics, opacities, pix_vels, colors, rolling_shutter_time,
                           width, height, tile_size, n_cameras, camera_ids=None, backgrounds=None,
                           dtype=np.float32):
    """Tile intersection + compositing of the oracle on GIVEN camera projection outputs and colours
    ([C,N,..] arrays, or [nnz,..] rows with ``camera_ids`` for the packed layout), so that the list
    stages and the image are compared on identical stage inputs. ``colors`` already carries every
    rendered channel (e.g. RGB + depth). Returns dict(tiles_per_gauss, isect_ids, flatten_ids,
    isect_offsets, out=<composite dict>)."""
    tw = math.ceil(width / float(tile_size))
    th = math.ceil(height / float(tile_size))
    tpg, ids, flat = isect.isect_tiles(np.asarray(means2d, np.float32), np.asarray(radii),
                                       np.asarray(depths, np.float32), tile_size, tw, th,
                                       n_cameras=n_cameras, camera_ids=camera_ids)
    offsets = isect.isect_offset_encode(ids, n_cameras, tw, th)
    out = composite.rasterize_to_pixels_fwd(means2d, conics, np.ascontiguousarray(colors), opacities, pix_vels,
                                            np.asarray(rolling_shutter_time), backgrounds, width, height,
                                            tile_size, offsets, flat, dtype=dtype)
    return dict(tiles_per_gauss=tpg, isect_ids=ids, flatten_ids=flat, isect_offsets=offsets, out=out)


def rasterization(
    means, quats, scales, opacities, colors, velocities, viewmats, Ks, width, height,
    linear_velocity=None, angular_velocity=None, rolling_shutter_time=None, near_plane=0.01,
    far_plane=1e10, radius_clip=0.0, eps2d=0.3, sh_degree=None, packed=True, tile_size=16,
    backgrounds=None, render_mode="RGB", rasterize_mode="classic", dtype=np.float32,
    timings: Optional[Dict] = None,
):
    """CPU camera render (always in the [C, N] layout; ``packed`` only changes intermediate
    layouts in the product, not the image). Returns (colors [C,H,W,X], alphas [C,H,W,1], meta)."""
    import time

    tdt = torch.float32 if dtype == np.float32 else torch.float64
    cast = lambda x: None if x is None else torch.as_tensor(x).to(tdt)  # noqa: E731
    C = viewmats.shape[0]
    N = means.shape[0]
    lin = cast(linear_velocity) if linear_velocity is not None else torch.zeros(C, 3, dtype=tdt)
    ang = cast(angular_velocity) if angular_velocity is not None else torch.zeros(C, 3, dtype=tdt)
    rs = cast(rolling_shutter_time) if rolling_shutter_time is not None else torch.zeros(C, dtype=tdt)
    t0 = time.perf_counter()
    with torch.no_grad():
        radii, means2d, depths, conics, comps, pix_vels = projection.fully_fused_projection(
            cast(means), None, cast(quats), cast(scales), cast(velocities), cast(viewmats), cast(Ks),
            width, height, lin, ang, rs, eps2d, near_plane, far_plane, radius_clip,
            rasterize_mode == "antialiased")
        opac = cast(opacities)[None].repeat(C, 1)
        if comps is not None:
            opac = opac * comps
        col = cast(colors)
        if sh_degree is not None:
            camtoworlds = torch.inverse(cast(viewmats))
            dirs = cast(means)[None] - camtoworlds[:, None, :3, 3]
            shs = col[None].expand(C, -1, -1, -1) if col.dim() == 3 else col
            col = projection.spherical_harmonics(sh_degree, dirs, shs, masks=radii[..., 0] > 0)
            col = torch.clamp_min(col + 0.5, 0.0)
        elif col.dim() == 2:
            col = col[None].expand(C, -1, -1)
        if render_mode in ("RGB+D", "RGB+ED"):
            col = torch.cat([col, depths[..., None]], dim=-1)
        elif render_mode in ("D", "ED"):
            col = depths[..., None]
    t1 = time.perf_counter()
    tw = math.ceil(width / float(tile_size))
    th = math.ceil(height / float(tile_size))
    tpg, ids, flat = isect.isect_tiles(_np(means2d).astype(np.float32), _np(radii), _np(depths).astype(np.float32),
                                       tile_size, tw, th)
    offsets = isect.isect_offset_encode(ids, C, tw, th)
    t2 = time.perf_counter()
    bg = None
    if backgrounds is not None:
        bg = _np(cast(backgrounds))
        if render_mode in ("RGB+D", "RGB+ED"):
            bg = np.concatenate([bg, np.zeros((C, 1), bg.dtype)], axis=-1)
        elif render_mode in ("D", "ED"):
            bg = np.zeros((C, 1), bg.dtype)
    out = composite.rasterize_to_pixels_fwd(_np(means2d), _np(conics), _np(col.contiguous()), _np(opac),
                                            _np(pix_vels), _np(rs), bg, width, height, tile_size, offsets,
                                            flat, dtype=dtype)
    t3 = time.perf_counter()
    render = out["render_colors"]
    if render_mode in ("ED", "RGB+ED"):
        render = np.concatenate([render[..., :-1], render[..., -1:] / np.maximum(out["render_alphas"], 1e-10)], axis=-1)
    if timings is not None:
        timings.update(projection=t1 - t0, isect=t2 - t1, composite=t3 - t2, total=t3 - t0)
    meta = dict(radii=_np(radii), means2d=_np(means2d), depths=_np(depths), conics=_np(conics),
                opacities=_np(opac), pix_vels=_np(pix_vels), colors=_np(col), tiles_per_gauss=tpg,
                isect_ids=ids, flatten_ids=flat, isect_offsets=offsets, tile_width=tw, tile_height=th,
                last_ids=out["last_ids"], ambiguous=out["ambiguous"], tested=out["tested"],
                contributing=out["contributing"])
    return render, out["render_alphas"], meta


# ---------------------------------------------------------------------------------------------
# Float64 gradient chains: projection (torch autograd) -> [SH colours] -> analytic compositing
# backward (C), on GIVEN tile lists. What an end-to-end training step is checked against.
# ---------------------------------------------------------------------------------------------
def _leaf64(x):
    return None if x is None else torch.as_tensor(x).detach().to(torch.float64).cpu().clone().requires_grad_(True)


def lidar_gradients_f64(cfg, offsets, flatten_ids, cotangents, names, mask_f32=None, amb_tol=1e-4, **kw):
    """Gradients of ``sum(features * cot[0] * mask) + sum(alphas * cot[1] * mask) + sum(alpha_sum *
    cot[2] * mask)`` with respect to ``cfg[name]`` for ``name in names``, in float64, through the
    oracle's differentiable lidar projection and the analytic compositing backward, on the given
    tile lists ([C, grid_h, grid_w] offsets, flatten ids into the [C, N] layout).

    ``mask`` [C, H, W] keeps the points whose include / skip / stop decisions are the same in
    float32 (``mask_f32``: oracle compositing dict of a float32 run with the same ``amb_tol``, or
    None to compute one on the float32 cast of this projection) and float64. Returns (grads dict,
    mask, float64 forward dict)."""
    C = cfg["viewmats"].shape[0]
    L = {k: _leaf64(cfg[k]) for k in names}
    get = lambda k: L[k] if k in L else (None if cfg.get(k) is None else torch.as_tensor(cfg[k]).double())  # noqa: E731
    zeros = lambda *s: torch.zeros(*s, dtype=torch.float64)  # noqa: E731
    lin = get("linear_velocity") if cfg.get("linear_velocity") is not None else zeros(C, 3)
    ang = get("angular_velocity") if cfg.get("angular_velocity") is not None else zeros(C, 3)
    rs = get("rolling_shutter_time") if cfg.get("rolling_shutter_time") is not None else zeros(C)
    radii, means2d, depths, conics, comps, pix_vels, dcomp = projection.fully_fused_lidar_projection(
        get("means"), None, get("quats"), get("scales"), get("velocities"), get("viewmats"), lin, ang, rs,
        cfg.get("min_elevation", -80), cfg.get("max_elevation", 80), cfg.get("min_azimuth", -180),
        cfg.get("max_azimuth", 180), cfg.get("eps2d", 0.017), cfg.get("near_plane", 0.01),
        cfg.get("far_plane", 1e10), cfg.get("radius_clip", 0.0), kw.get("rasterize_mode") == "antialiased")
    opac = get("opacities")[None].repeat(C, 1)
    if comps is not None:
        opac = opac * comps
    if not kw.get("use_depth_compensation", True):
        dcomp = dcomp * 0
    feats = torch.cat([get("lidar_features"), depths[..., None]], dim=-1)
    pts = np.asarray(torch.as_tensor(cfg["raster_pts"]).double())
    H, W = pts.shape[1:3]
    asum = kw.get("compute_alpha_sum_until_points", True)
    thr = kw.get("compute_alpha_sum_until_points_threshold", 0.2)
    stage = [means2d, conics, feats, opac, pix_vels, dcomp]
    vals = [_np(x) for x in stage]
    geom = (pts, W, H, cfg["tile_width"], cfg["tile_height"], np.asarray(offsets), np.asarray(flatten_ids), asum, thr)
    f64 = composite.rasterize_to_points_fwd(*vals, None, *geom, dtype=np.float64)
    if mask_f32 is None:
        mask_f32 = composite.rasterize_to_points_fwd(*[v.astype(np.float32) for v in vals], None, *geom,
                                                     dtype=np.float32, amb_tol=amb_tol)
    mask = (mask_f32["last_ids"] == f64["last_ids"]) & ~mask_f32["ambiguous"]
    mk = mask[..., None].astype(np.float64)
    v_c, v_a = np.asarray(cotangents[0], np.float64) * mk, np.asarray(cotangents[1], np.float64) * mk
    v_s = np.asarray(cotangents[2], np.float64) * mk if (asum and cotangents[2] is not None) else None
    g = composite.rasterize_to_points_bwd(*vals, None, *geom, f64["render_alphas"], f64["last_ids"], v_c, v_a, v_s)
    grads_in = [g["v_means2d"], g["v_conics"], g["v_colors"], g["v_opacities"], g["v_pix_vels"], g["v_depth_comps"]]
    torch.autograd.backward(stage, [torch.from_numpy(x) for x in grads_in])
    return {k: L[k].grad for k in names}, mask, f64


def camera_gradients_f64(cfg, offsets, flatten_ids, cotangents, names, camera_ids=None, gaussian_ids=None,
                         mask_f32=None, amb_tol=1e-4):
    """Camera counterpart of :func:`lidar_gradients_f64`: gradients of ``sum(image * cot[0] * mask)
    + sum(alphas * cot[1] * mask)`` through the oracle's camera projection, SH colours
    (``sh_degree``) or plain colours, the render-mode channel rules, and the analytic compositing
    backward. ``flatten_ids`` index the [C, N] layout, or packed rows when ``camera_ids`` /
    ``gaussian_ids`` are given."""
    C, N = cfg["viewmats"].shape[0], cfg["means"].shape[0]
    L = {k: _leaf64(cfg[k]) for k in names}
    get = lambda k: L[k] if k in L else (None if cfg.get(k) is None else torch.as_tensor(cfg[k]).double())  # noqa: E731
    zeros = lambda *s: torch.zeros(*s, dtype=torch.float64)  # noqa: E731
    lin = get("linear_velocity") if cfg.get("linear_velocity") is not None else zeros(C, 3)
    ang = get("angular_velocity") if cfg.get("angular_velocity") is not None else zeros(C, 3)
    rs = get("rolling_shutter_time") if cfg.get("rolling_shutter_time") is not None else zeros(C)
    mode = cfg.get("render_mode", "RGB")
    assert mode in ("RGB", "RGB+D", "D"), mode
    aa = cfg.get("rasterize_mode", "classic") == "antialiased"
    radii, means2d, depths, conics, comps, pix_vels = projection.fully_fused_projection(
        get("means"), None, get("quats"), get("scales"), get("velocities"), get("viewmats"), get("Ks"),
        cfg["width"], cfg["height"], lin, ang, rs, cfg.get("eps2d", 0.3), cfg.get("near_plane", 0.01),
        cfg.get("far_plane", 1e10), cfg.get("radius_clip", 0.0), aa)
    opac = get("opacities")[None].repeat(C, 1)
    if comps is not None:
        opac = opac * comps
    col = get("colors")
    if cfg.get("sh_degree") is not None:
        dirs = get("means")[None] - torch.inverse(get("viewmats"))[:, None, :3, 3]
        shs = col[None].expand(C, -1, -1, -1) if col.dim() == 3 else col
        col = torch.clamp_min(projection.spherical_harmonics(cfg["sh_degree"], dirs, shs, masks=radii[..., 0] > 0)
                              + 0.5, 0.0)
    elif col.dim() == 2:
        col = col[None].expand(C, -1, -1)
    if mode == "RGB+D":
        col = torch.cat([col, depths[..., None]], dim=-1)
    elif mode == "D":
        col = depths[..., None]
    col = col.contiguous()
    flat = np.asarray(flatten_ids).astype(np.int64)
    if camera_ids is not None:
        flat = np.asarray(camera_ids).astype(np.int64)[flat] * N + np.asarray(gaussian_ids).astype(np.int64)[flat]
    stage = [means2d, conics, col, opac, pix_vels]
    vals = [_np(x) for x in stage]
    bg = None if cfg.get("backgrounds") is None else np.asarray(torch.as_tensor(cfg["backgrounds"]).double())
    if bg is not None and mode == "RGB+D":
        bg = np.concatenate([bg, np.zeros((C, 1))], axis=-1)
    geom = (cfg["width"], cfg["height"], cfg.get("tile_size", 16), np.asarray(offsets), flat.astype(np.int32))
    rs_np = _np(rs)
    f64 = composite.rasterize_to_pixels_fwd(*vals, rs_np, bg, *geom, dtype=np.float64)
    if mask_f32 is None:
        mask_f32 = composite.rasterize_to_pixels_fwd(*[v.astype(np.float32) for v in vals], rs_np, bg, *geom,
                                                     dtype=np.float32, amb_tol=amb_tol)
    mask = (mask_f32["last_ids"] == f64["last_ids"]) & ~mask_f32["ambiguous"]
    mk = mask[..., None].astype(np.float64)
    v_c, v_a = np.asarray(cotangents[0], np.float64) * mk, np.asarray(cotangents[1], np.float64) * mk
    g = composite.rasterize_to_pixels_bwd(*vals, rs_np, bg, *geom, f64["render_alphas"], f64["last_ids"], v_c, v_a)
    grads_in = [g["v_means2d"], g["v_conics"], g["v_colors"], g["v_opacities"], g["v_pix_vels"]]
    torch.autograd.backward(stage, [torch.from_numpy(x) for x in grads_in])
    return {k: L[k].grad for k in names}, mask, f64
