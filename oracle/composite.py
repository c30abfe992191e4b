"""ctypes front end of the C compositing oracle (``oracle/composite.c``), plus a tiny pure-numpy
per-pixel compositor used to cross-check the C code. TEST INFRASTRUCTURE ONLY - see
``oracle/__init__.py``.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_DIR, "_build", "liboracle.so")
_lib = None


def build() -> str:
    proc = subprocess.run(["make", "-C", _DIR], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("building the C oracle failed:\n" + proc.stdout)
    return _LIB_PATH


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _arr(a, dtype):
    if a is None:
        return None
    return np.ascontiguousarray(a, dtype=dtype)


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _real(dtype):
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        return np.float32, "f32", ctypes.c_float
    return np.float64, "f64", ctypes.c_double


def rasterize_to_pixels_fwd(means2d, conics, colors, opacities, pix_vels, rs_time, backgrounds, width,
                            height, tile_size, offsets, flatten_ids, dtype=np.float32, amb_tol=2e-5):
    """Returns dict(render_colors, render_alphas, last_ids, ambiguous, tested, contributing)."""
    rt, sfx, creal = _real(dtype)
    C, tile_h, tile_w = offsets.shape
    channels = colors.shape[-1]
    a = [_arr(x, rt) for x in (means2d, conics, colors, opacities, pix_vels, rs_time, backgrounds)]
    off = _arr(offsets, np.int32)
    flat = _arr(flatten_ids, np.int32)
    out_c = np.zeros((C, height, width, channels), rt)
    out_a = np.zeros((C, height, width, 1), rt)
    last = np.zeros((C, height, width), np.int32)
    amb = np.zeros((C, height, width), np.uint8)
    counters = np.zeros(2, np.int64)
    fn = getattr(load(), "rasterize_to_pixels_fwd_" + sfx)
    fn.restype = None
    fn(ctypes.c_int(C), ctypes.c_long(flat.size), _p(a[0]), _p(a[1]), _p(a[2]), ctypes.c_int(channels),
       _p(a[3]), _p(a[4]), _p(a[5]), _p(a[6]), ctypes.c_int(width), ctypes.c_int(height),
       ctypes.c_int(tile_size), ctypes.c_int(tile_w), ctypes.c_int(tile_h), _p(off), _p(flat), _p(out_c),
       _p(out_a), _p(last), _p(amb), creal(amb_tol), _p(counters))
    return dict(render_colors=out_c, render_alphas=out_a, last_ids=last, ambiguous=amb.astype(bool),
                tested=int(counters[0]), contributing=int(counters[1]))


def rasterize_to_points_fwd(means2d, conics, colors, opacities, pix_vels, depth_comps, backgrounds,
                            raster_pts, width, height, tile_width, tile_height, offsets, flatten_ids,
                            compute_alpha_sum, alpha_sum_threshold, depth_idx=None, dtype=np.float32,
                            amb_tol=2e-5):
    """Returns dict(render_colors, render_alphas, alpha_sum, last_ids, median_depths, ambiguous, ...)."""
    rt, sfx, creal = _real(dtype)
    C, grid_h, grid_w = offsets.shape
    channels = colors.shape[-1]
    if depth_idx is None:
        depth_idx = channels - 1
    a = [_arr(x, rt) for x in (means2d, conics, colors, opacities, pix_vels, depth_comps, backgrounds, raster_pts)]
    off = _arr(offsets, np.int32)
    flat = _arr(flatten_ids, np.int32)
    out_c = np.zeros((C, height, width, channels), rt)
    out_a = np.zeros((C, height, width, 1), rt)
    out_s = np.zeros((C, height, width, 1), rt)
    out_m = np.zeros((C, height, width, 1), rt)
    last = np.zeros((C, height, width), np.int32)
    amb = np.zeros((C, height, width), np.uint8)
    counters = np.zeros(2, np.int64)
    fn = getattr(load(), "rasterize_to_points_fwd_" + sfx)
    fn.restype = None
    fn(ctypes.c_int(C), ctypes.c_long(flat.size), _p(a[0]), _p(a[1]), _p(a[2]), ctypes.c_int(channels),
       _p(a[3]), _p(a[4]), _p(a[5]), _p(a[6]), _p(a[7]), ctypes.c_int(width), ctypes.c_int(height),
       ctypes.c_int(tile_width), ctypes.c_int(tile_height), ctypes.c_int(grid_w), ctypes.c_int(grid_h),
       ctypes.c_int(int(bool(compute_alpha_sum))), creal(alpha_sum_threshold), _p(off), _p(flat),
       ctypes.c_int(depth_idx), _p(out_c), _p(out_a), _p(out_s), _p(last), _p(out_m), _p(amb),
       creal(amb_tol), _p(counters))
    return dict(render_colors=out_c, render_alphas=out_a, alpha_sum=out_s if compute_alpha_sum else None,
                last_ids=last, median_depths=out_m, ambiguous=amb.astype(bool), tested=int(counters[0]),
                contributing=int(counters[1]))


def rasterize_to_pixels_bwd(means2d, conics, colors, opacities, pix_vels, rs_time, backgrounds, width,
                            height, tile_size, offsets, flatten_ids, render_alphas, last_ids,
                            v_render_colors, v_render_alphas, absgrad=False, dtype=np.float64):
    """Returns dict of float64 gradients: v_means2d, v_conics, v_colors, v_opacities, v_pix_vels
    (and v_means2d_abs)."""
    rt, sfx, _ = _real(dtype)
    C, tile_h, tile_w = offsets.shape
    channels = colors.shape[-1]
    a = [_arr(x, rt) for x in (means2d, conics, colors, opacities, pix_vels, rs_time, backgrounds,
                               render_alphas, v_render_colors, v_render_alphas)]
    off = _arr(offsets, np.int32)
    flat = _arr(flatten_ids, np.int32)
    last = _arr(last_ids, np.int32)
    g = dict(
        v_means2d_abs=np.zeros(means2d.shape, np.float64) if absgrad else None,
        v_means2d=np.zeros(means2d.shape, np.float64),
        v_conics=np.zeros(conics.shape, np.float64),
        v_colors=np.zeros(colors.shape, np.float64),
        v_opacities=np.zeros(opacities.shape, np.float64),
        v_pix_vels=np.zeros(pix_vels.shape, np.float64),
    )
    fn = getattr(load(), "rasterize_to_pixels_bwd_" + sfx)
    fn.restype = None
    fn(ctypes.c_int(C), ctypes.c_long(flat.size), _p(a[0]), _p(a[1]), _p(a[2]), ctypes.c_int(channels),
       _p(a[3]), _p(a[4]), _p(a[5]), _p(a[6]), ctypes.c_int(width), ctypes.c_int(height),
       ctypes.c_int(tile_size), ctypes.c_int(tile_w), ctypes.c_int(tile_h), _p(off), _p(flat), _p(a[7]),
       _p(last), _p(a[8]), _p(a[9]), _p(g["v_means2d_abs"]), _p(g["v_means2d"]), _p(g["v_conics"]),
       _p(g["v_colors"]), _p(g["v_opacities"]), _p(g["v_pix_vels"]))
    return g


def rasterize_to_points_bwd(means2d, conics, colors, opacities, pix_vels, depth_comps, backgrounds,
                            raster_pts, width, height, tile_width, tile_height, offsets, flatten_ids,
                            compute_alpha_sum, alpha_sum_threshold, render_alphas, last_ids,
                            v_render_colors, v_render_alphas, v_alpha_sum, depth_idx=None, absgrad=False,
                            dtype=np.float64):
    rt, sfx, creal = _real(dtype)
    C, grid_h, grid_w = offsets.shape
    channels = colors.shape[-1]
    if depth_idx is None:
        depth_idx = channels - 1
    a = [_arr(x, rt) for x in (means2d, conics, colors, opacities, pix_vels, depth_comps, backgrounds,
                               raster_pts, render_alphas, v_render_colors, v_render_alphas, v_alpha_sum)]
    off = _arr(offsets, np.int32)
    flat = _arr(flatten_ids, np.int32)
    last = _arr(last_ids, np.int32)
    g = dict(
        v_means2d_abs=np.zeros(means2d.shape, np.float64) if absgrad else None,
        v_means2d=np.zeros(means2d.shape, np.float64),
        v_conics=np.zeros(conics.shape, np.float64),
        v_colors=np.zeros(colors.shape, np.float64),
        v_opacities=np.zeros(opacities.shape, np.float64),
        v_pix_vels=np.zeros(pix_vels.shape, np.float64),
        v_depth_comps=np.zeros(depth_comps.shape, np.float64),
    )
    fn = getattr(load(), "rasterize_to_points_bwd_" + sfx)
    fn.restype = None
    fn(ctypes.c_int(C), ctypes.c_long(flat.size), _p(a[0]), _p(a[1]), _p(a[2]), ctypes.c_int(channels),
       _p(a[3]), _p(a[4]), _p(a[5]), _p(a[6]), _p(a[7]), ctypes.c_int(width), ctypes.c_int(height),
       ctypes.c_int(tile_width), ctypes.c_int(tile_height), ctypes.c_int(grid_w), ctypes.c_int(grid_h),
       ctypes.c_int(int(bool(compute_alpha_sum))), creal(alpha_sum_threshold), _p(off), _p(flat),
       ctypes.c_int(depth_idx), _p(a[8]), _p(last), _p(a[9]), _p(a[10]), _p(a[11]),
       _p(g["v_means2d_abs"]), _p(g["v_means2d"]), _p(g["v_conics"]), _p(g["v_colors"]),
       _p(g["v_opacities"]), _p(g["v_pix_vels"]), _p(g["v_depth_comps"]))
    return g


def _indices_in_range(lidar, range_start, range_end, transmittances, means2d, conics, opacities, pix_vels,
                      rs_time, raster_pts, width, height, tile_w, tile_h, offsets, flatten_ids, dtype, amb_tol):
    rt, sfx, creal = _real(dtype)
    C, grid_h, grid_w = offsets.shape
    N = opacities.shape[1]
    a = [_arr(x, rt) for x in (means2d, conics, opacities, pix_vels, rs_time, raster_pts, transmittances)]
    off = _arr(offsets, np.int32)
    flat = _arr(flatten_ids, np.int32)
    n_pix = C * height * width
    cnts = np.zeros(n_pix, np.int32)
    amb = np.zeros(n_pix, np.uint8)
    fn = getattr(load(), "rasterize_to_indices_in_range_" + sfx)
    fn.restype = None
    lim = 2 ** 32 - 1   # the reference's range arguments are uint32

    def call(starts, g_ids, p_ids):
        fn(ctypes.c_int(int(lidar)), ctypes.c_long(min(int(range_start), lim)),
           ctypes.c_long(min(int(range_end), lim)), ctypes.c_int(C), ctypes.c_long(N),
           ctypes.c_long(flat.size), _p(a[0]), _p(a[1]), _p(a[2]), _p(a[3]), _p(a[4]), _p(a[5]),
           ctypes.c_int(width), ctypes.c_int(height), ctypes.c_int(tile_w), ctypes.c_int(tile_h),
           ctypes.c_int(grid_w), ctypes.c_int(grid_h), _p(off), _p(flat), _p(a[6]), _p(starts), _p(cnts),
           _p(g_ids), _p(p_ids), _p(amb), creal(amb_tol))

    if flat.size:
        call(None, None, None)
    csum = np.cumsum(cnts, dtype=np.int64)
    total = int(csum[-1]) if n_pix else 0
    starts = np.ascontiguousarray(csum - cnts)
    g_ids = np.zeros(total, np.int64)
    p_ids = np.zeros(total, np.int64)
    if total:
        call(starts, g_ids, p_ids)
    hw = width * height
    return dict(gaussian_ids=g_ids, pixel_ids=p_ids % hw, camera_ids=p_ids // hw, counts=cnts.reshape(C, height, width),
                ambiguous=amb.astype(bool).reshape(C, height, width))


def rasterize_to_indices_in_range(range_start, range_end, transmittances, means2d, conics, opacities, pix_vels,
                                  width, height, tile_size, offsets, flatten_ids, rs_time=None,
                                  dtype=np.float32, amb_tol=2e-5):
    """gsplat/cuda/_wrapper.py:1115-1196. Returns dict(gaussian_ids, pixel_ids, camera_ids, counts,
    ambiguous)."""
    if rs_time is None:
        rs_time = np.zeros(offsets.shape[0])
    return _indices_in_range(False, range_start, range_end, transmittances, means2d, conics, opacities,
                             pix_vels, rs_time, None, width, height, tile_size, tile_size, offsets,
                             flatten_ids, dtype, amb_tol)


def rasterize_to_indices_in_range_lidar(range_start, range_end, transmittances, means2d, conics, opacities,
                                        pix_vels, raster_pts, width, height, tile_width, tile_height, offsets,
                                        flatten_ids, dtype=np.float32, amb_tol=2e-5):
    """gsplat/cuda/_wrapper.py:1198-1281."""
    return _indices_in_range(True, range_start, range_end, transmittances, means2d, conics, opacities,
                             pix_vels, None, raster_pts, width, height, tile_width, tile_height, offsets,
                             flatten_ids, dtype, amb_tol)


def _weights_along_rays(alphas, ray_ids, n_rays):
    """w_i = alpha_i * prod over earlier samples of the same ray of (1 - alpha_j); the samples of a ray
    are contiguous and in order (the two nerfacc helpers the reference's accumulate() calls)."""
    w = np.zeros_like(alphas)
    T = np.ones(n_rays, alphas.dtype)
    for k in range(alphas.size):
        r = ray_ids[k]
        w[k] = alphas[k] * T[r]
        T[r] *= 1 - alphas[k]
    return w


def accumulate(means2d, conics, opacities, colors, pix_vels, rs_time, gaussian_ids, pixel_ids, camera_ids,
               width, height, dtype=np.float64):
    """Compositing of explicit (Gaussian, pixel, camera) triples: gsplat/cuda/_torch_impl.py:610-700.
    Returns (renders [C,H,W,ch], alphas [C,H,W,1])."""
    f = lambda x: np.asarray(x, dtype)
    means2d, conics, opacities, colors, pix_vels, rs_time = map(f, (means2d, conics, opacities, colors, pix_vels, rs_time))
    C = means2d.shape[0]
    x, y = pixel_ids % width, pixel_ids // width
    roll = rs_time[camera_ids] * (y.astype(dtype) / (height - 1) - 0.5)
    coords = np.stack([x, y], -1).astype(dtype) + 0.5
    d = means2d[camera_ids, gaussian_ids] + roll[:, None] * pix_vels[camera_ids, gaussian_ids] - coords
    c = conics[camera_ids, gaussian_ids]
    sigma = 0.5 * (c[:, 0] * d[:, 0] ** 2 + c[:, 2] * d[:, 1] ** 2) + c[:, 1] * d[:, 0] * d[:, 1]
    alpha = np.minimum(opacities[camera_ids, gaussian_ids] * np.exp(-sigma), 0.999)
    rays = camera_ids * height * width + pixel_ids
    n_rays = C * height * width
    w = _weights_along_rays(alpha, rays, n_rays)
    renders = np.zeros((n_rays, colors.shape[-1]), dtype)
    np.add.at(renders, rays, w[:, None] * colors[camera_ids, gaussian_ids])
    acc = np.zeros(n_rays, dtype)
    np.add.at(acc, rays, w)
    return renders.reshape(C, height, width, -1), acc.reshape(C, height, width, 1)


def accumulate_lidar(means2d, conics, opacities, features, pix_vels, depth_comps, raster_pts, gaussian_ids,
                     pixel_ids, camera_ids, width, height, compute_alpha_sum, threshold, dtype=np.float64):
    """Lidar counterpart: gsplat/cuda/_torch_impl.py:702-820. Returns (renders, alphas, alpha_sum or None)."""
    f = lambda x: np.asarray(x, dtype)
    means2d, conics, opacities, features, pix_vels, depth_comps, raster_pts = map(
        f, (means2d, conics, opacities, features, pix_vels, depth_comps, raster_pts))
    C = means2d.shape[0]
    x, y = pixel_ids % width, pixel_ids // width
    pts = raster_pts[camera_ids, y, x]
    roll = pts[:, 3]
    d = np.mod(means2d[camera_ids, gaussian_ids] + roll[:, None] * pix_vels[camera_ids, gaussian_ids, :2]
               - pts[:, :2] + 180, 360) - 180
    d = np.where(d < -180, d + 360, d)
    c = conics[camera_ids, gaussian_ids]
    sigma = 0.5 * (c[:, 0] * d[:, 0] ** 2 + c[:, 2] * d[:, 1] ** 2) + c[:, 1] * d[:, 0] * d[:, 1]
    alpha = np.minimum(opacities[camera_ids, gaussian_ids] * np.exp(-sigma), 0.999)
    feats = features[camera_ids, gaussian_ids].copy()
    feats[:, -1] += (d * depth_comps[camera_ids, gaussian_ids]).sum(-1) + pix_vels[camera_ids, gaussian_ids, 2] * roll
    rays = camera_ids * height * width + pixel_ids
    n_rays = C * height * width
    asum = None
    if compute_alpha_sum:
        before = features[camera_ids, gaussian_ids, -1] < (pts[:, 2] - threshold)
        asum = np.zeros(n_rays, dtype)
        np.add.at(asum, rays, np.where(before, alpha, 0))
        asum = asum.reshape(C, height, width, 1)
    w = _weights_along_rays(alpha, rays, n_rays)
    renders = np.zeros((n_rays, feats.shape[-1]), dtype)
    np.add.at(renders, rays, w[:, None] * feats)
    acc = np.zeros(n_rays, dtype)
    np.add.at(acc, rays, w)
    return renders.reshape(C, height, width, -1), acc.reshape(C, height, width, 1), asum


# ---------------------------------------------------------------------------------------------
# Pure-python reference of one pixel / one lidar point (float64), used to validate the C code
# on tiny cases. Same rules as the C functions above.
# ---------------------------------------------------------------------------------------------
def composite_one(deltas, conics, opacities, features, extra_depth: Optional[np.ndarray] = None):
    """deltas [n,2], conics [n,3], opacities [n], features [n,D] in list order.
    Returns (out [D], alpha, last_index, weights [n])."""
    T = 1.0
    out = np.zeros(features.shape[1])
    last = 0
    w = np.zeros(len(deltas))
    for k in range(len(deltas)):
        dx, dy = deltas[k]
        a, b, c = conics[k]
        sigma = 0.5 * (a * dx * dx + c * dy * dy) + b * dx * dy
        alpha = min(0.999, opacities[k] * np.exp(-sigma))
        if sigma < 0 or alpha < 1.0 / 255.0:
            continue
        nT = T * (1 - alpha)
        if nT <= 1e-4:
            break
        vis = alpha * T
        out += features[k] * vis
        if extra_depth is not None:
            out[-1] += extra_depth[k] * vis
        w[k] = vis
        last = k
        T = nT
    return out, 1 - T, last, w
