"""CPU restatement (numpy, float32 / int64, vectorised) of tile intersection and offset
encoding. TEST INFRASTRUCTURE ONLY - see ``oracle/__init__.py``.

Follows
  isect_tiles          gsplat/cuda/csrc/rasterization.cu:15-90   (torch twin _torch_impl.py:422-488)
  isect_lidar_tiles    gsplat/cuda/csrc/rasterization.cu:287-395 (torch twin _torch_impl.py:492-581)
  isect_offset_encode  gsplat/cuda/csrc/rasterization.cu:218-262 (torch twin _torch_impl.py:585-607)
  sort                 cub::DeviceRadixSort::SortPairs is a stable sort of the 64-bit ids
                       (rasterization.cu:181-188, 494-501) = numpy stable argsort here.

One deliberate difference from the CUDA kernel, shared with the product: the azimuth tile index
is wrapped with a true modulo (always in [0, n_tiles_azim)), as the reference's torch twin does
(_torch_impl.py:566); the kernel's ``(j + n) % n`` goes negative when a Gaussian's azimuth
extent exceeds a full turn on the low side, which indexes out of bounds downstream.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np

f32 = np.float32


def _bit_length(v: int) -> int:
    return int(v).bit_length()


def cam_rects(means2d: np.ndarray, radii: np.ndarray, tile_size: int, tile_width: int, tile_height: int):
    """means2d [M,2] f32, radii [M,2] int32 -> x0, x1, y0, y1 int64 arrays (x1/y1 exclusive)."""
    ts = f32(tile_size)
    ex = radii[:, 0].astype(f32) / ts
    ey = radii[:, 1].astype(f32) / ts
    tx = means2d[:, 0].astype(f32) / ts
    ty = means2d[:, 1].astype(f32) / ts

    def clamp(v, hi):
        v = np.where(np.isnan(v), f32(0), v)
        return np.clip(v, 0, hi).astype(np.int64)

    x0 = clamp(np.floor(tx - ex), tile_width)
    y0 = clamp(np.floor(ty - ey), tile_height)
    x1 = clamp(np.ceil(tx + ex), tile_width)
    y1 = clamp(np.ceil(ty + ey), tile_height)
    return x0, x1, y0, y1


def lidar_rects(means2d: np.ndarray, radii: np.ndarray, elev_boundaries: np.ndarray,
                tile_azim_resolution: float, min_azim: float):
    """means2d [M,2] f32, radii [M,2] f32 -> x0, x1 (unwrapped azimuth tile range), y0, y1."""
    res = f32(tile_azim_resolution)
    n_az = int(math.ceil(f32(360.0) / res))
    n_el = len(elev_boundaries) - 1
    b = elev_boundaries.astype(f32)
    el = means2d[:, 1].astype(f32)
    el_lo = el - radii[:, 1].astype(f32)
    el_hi = el + radii[:, 1].astype(f32)
    azim = means2d[:, 0].astype(f32) - f32(min_azim)
    az_lo = azim - radii[:, 0].astype(f32)
    az_hi = azim + radii[:, 0].astype(f32)
    azim_max = f32(n_az) * res
    with np.errstate(invalid="ignore"):
        t_lo = np.where(az_lo >= 0, az_lo / res, (np.fmod(az_lo + f32(360), f32(360)) - azim_max) / res)
        t_hi = np.where(az_hi <= f32(360), az_hi / res, f32(n_az) + np.fmod(az_hi + f32(360), f32(360)) / res)
    x0 = np.floor(t_lo).astype(np.int64)
    x1 = np.ceil(t_hi).astype(np.int64)
    # i = number of boundaries strictly below the bound (boundaries are ascending)
    i_lo = np.searchsorted(b, el_lo, side="left")
    y0 = np.maximum(i_lo - 1, 0)
    i_hi = np.maximum(np.searchsorted(b, el_hi, side="left"), i_lo)
    y1 = np.minimum(i_hi, n_el)
    return x0, x1, y0.astype(np.int64), y1.astype(np.int64), n_az, n_el


def _emit_and_sort(visible, x0, x1, y0, y1, depths, cids, n_cameras, n_tiles, row_width, wrap, sort):
    cnt = np.where(visible, (y1 - y0) * (x1 - x0), 0).astype(np.int64)
    tiles_per_gauss = cnt.astype(np.int32)
    cnt_pos = np.maximum(cnt, 0)
    n_isects = int(cnt_pos.sum())
    tile_n_bits = _bit_length(n_tiles)
    cam_n_bits = _bit_length(n_cameras)
    if tile_n_bits + cam_n_bits > 32:
        raise RuntimeError("isect: tile bits + sensor bits exceed 32")
    src = np.repeat(np.arange(len(cnt), dtype=np.int64), cnt_pos)
    start = np.cumsum(cnt_pos) - cnt_pos
    k = np.arange(n_isects, dtype=np.int64) - start[src]
    w = np.maximum(x1 - x0, 1)[src]
    ty = y0[src] + k // w
    tx = x0[src] + k % w
    if wrap:
        tx = np.mod(tx, row_width)
    tile = ty * row_width + tx
    depth_bits = depths.astype(f32).view(np.int32).astype(np.int64)[src]
    isect_ids = (cids[src] << (32 + tile_n_bits)) | (tile << 32) | depth_bits
    flatten_ids = src.astype(np.int32)
    if sort:
        order = np.argsort(isect_ids, kind="stable")
        isect_ids = isect_ids[order]
        flatten_ids = flatten_ids[order]
    return tiles_per_gauss, isect_ids, flatten_ids


def isect_tiles(means2d, radii, depths, tile_size, tile_width, tile_height, sort=True,
                n_cameras: Optional[int] = None, camera_ids=None) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """[C,N,..] or packed [nnz,..] inputs -> (tiles_per_gauss, isect_ids int64, flatten_ids int32)."""
    packed = means2d.ndim == 2
    shape = depths.shape
    m2 = means2d.reshape(-1, 2)
    r = radii.reshape(-1, 2)
    d = depths.reshape(-1)
    if packed:
        cids = np.asarray(camera_ids, dtype=np.int64)
        C = int(n_cameras)
    else:
        C, N = shape
        cids = np.repeat(np.arange(C, dtype=np.int64), N)
    x0, x1, y0, y1 = cam_rects(m2, r, tile_size, tile_width, tile_height)
    tpg, ids, flat = _emit_and_sort(r[:, 0] > 0, x0, x1, y0, y1, d, cids, C, tile_width * tile_height,
                                    tile_width, False, sort)
    return tpg.reshape(shape), ids, flat


def camera_tile_counts(means2d, radii, tile_size, tile_width, tile_height) -> np.ndarray:
    """Tiles per (sensor, Gaussian) of :func:`isect_tiles` without emitting or sorting anything."""
    r = radii.reshape(-1, 2)
    x0, x1, y0, y1 = cam_rects(means2d.reshape(-1, 2), r, tile_size, tile_width, tile_height)
    cnt = np.where(r[:, 0] > 0, (y1 - y0) * (x1 - x0), 0)
    return cnt.astype(np.int32).reshape(radii.shape[:-1])


def isect_lidar_tiles(means2d, radii, depths, elev_boundaries, tile_azim_resolution, min_azim, sort=True,
                      n_cameras: Optional[int] = None, camera_ids=None):
    packed = means2d.ndim == 2
    shape = depths.shape
    m2 = means2d.reshape(-1, 2)
    r = radii.reshape(-1, 2)
    d = depths.reshape(-1)
    if packed:
        cids = np.asarray(camera_ids, dtype=np.int64)
        C = int(n_cameras)
    else:
        C, N = shape
        cids = np.repeat(np.arange(C, dtype=np.int64), N)
    x0, x1, y0, y1, n_az, n_el = lidar_rects(m2, r, np.asarray(elev_boundaries), tile_azim_resolution, min_azim)
    tpg, ids, flat = _emit_and_sort(r[:, 0] > 0, x0, x1, y0, y1, d, cids, C, n_az * n_el, n_az, True, sort)
    return tpg.reshape(shape), ids, flat


def isect_offset_encode(isect_ids: np.ndarray, n_cameras: int, tile_width: int, tile_height: int) -> np.ndarray:
    """Sorted isect ids -> offsets [C, tile_height, tile_width] int32 (start of every tile's list)."""
    n_tiles = tile_width * tile_height
    tile_n_bits = _bit_length(n_tiles)
    hi = isect_ids >> 32
    cid = hi >> tile_n_bits
    tid = hi & ((1 << tile_n_bits) - 1)
    flat = cid * n_tiles + tid
    targets = np.arange(n_cameras * n_tiles, dtype=np.int64)
    offsets = np.searchsorted(flat, targets, side="left")
    return offsets.astype(np.int32).reshape(n_cameras, tile_height, tile_width)


# ---------------------------------------------------------------------------------------------
# Lidar points -> tiles -> raster image (gsplat/cuda/csrc/rasterization.cu:531-833; the reference has
# no torch twin of these three, so this follows the CUDA kernels and is pinned by the properties the
# reference's own tests assert, tests/test_basic.py:787-890).
# ---------------------------------------------------------------------------------------------
def map_points_to_lidar_tiles(points2d, elev_boundaries, tile_azim_resolution, min_azim, sort=True,
                              n_cameras: Optional[int] = None, camera_ids=None):
    """points2d [C,N,2] or [nnz,2] float32 -> (tile_ids int64 = sensor << 32 | tile, flatten_ids int32).

    Kernel rasterization.cu:596-651: azimuth tile = int(azim / res) with azim = x - min_azim wrapped
    by fmodf(azim + 360, 360) outside [0, 360); elevation tile = (number of the first n_tiles_elev
    boundaries that are < y) - 1, at least 0. Sorted by tile id with a stable sort (the reference
    radix-sorts the 64-bit ids, rasterization.cu:705-742)."""
    p = np.asarray(points2d, dtype=np.float32)
    packed = p.ndim == 2
    pts = p.reshape(-1, 2)
    if packed:
        cids = np.asarray(camera_ids, dtype=np.int64)
    else:
        C, N = p.shape[:2]
        cids = np.repeat(np.arange(C, dtype=np.int64), N)
    eb = np.asarray(elev_boundaries, dtype=np.float32)
    res = np.float32(tile_azim_resolution)
    n_az = int(np.ceil(np.float32(360.0) / res))
    n_el = eb.shape[0] - 1
    azim = pts[:, 0] - np.float32(min_azim)
    inside = (azim >= 0) & (azim < np.float32(360.0))
    wrapped = np.fmod(azim + np.float32(360.0), np.float32(360.0))
    tile_azim = np.where(inside, azim, wrapped) / res
    tx = np.where(np.isnan(tile_azim), 0, np.trunc(tile_azim)).astype(np.int64)
    tx = np.clip(tx, 0, n_az - 1)
    below = (eb[None, :n_el] < pts[:, 1:2])          # NaN compares false, like the kernel's loop
    i = np.where(below.all(axis=1), n_el, np.argmin(below, axis=1))   # leading run of "below"
    ty = np.maximum(i - 1, 0).astype(np.int64)
    ids = (cids << 32) | (ty * n_az + tx)
    flat = np.arange(pts.shape[0], dtype=np.int32)
    if sort:
        order = np.argsort(ids, kind="stable")
        ids, flat = ids[order], flat[order]
    return ids, flat


def points_mapping_offset_encode(point_ids: np.ndarray, n_lidars: int, tile_width: int, tile_height: int):
    """Sorted point tile ids -> offsets [C, tile_height, tile_width] int32 (rasterization.cu:531-594)."""
    n_tiles = tile_width * tile_height
    ids = np.asarray(point_ids, dtype=np.int64)
    flat = (ids >> 32) * n_tiles + (ids & 0xFFFFFFFF)
    targets = np.arange(n_lidars * n_tiles, dtype=np.int64)
    return np.searchsorted(flat, targets, side="left").astype(np.int32).reshape(n_lidars, tile_height, tile_width)


def populate_image_from_points(points, image_width, image_height, tile_width, tile_height, tile_offsets,
                               flatten_ids):
    """[C,N,5] or [nnz,5] points -> image [C,H,W,5]: per tile, the k-th listed point lands on the
    tile's k-th pixel (row-major in the tile), at most tile_width * tile_height points per tile,
    pixels outside the image skipped (rasterization.cu:749-796)."""
    pts = np.asarray(points, dtype=np.float32).reshape(-1, 5)
    offs = np.asarray(tile_offsets)
    C, gh, gw = offs.shape
    flat_offs = offs.reshape(-1)
    n_points = len(flatten_ids)
    img = np.zeros((C, image_height, image_width, 5), np.float32)
    for b in range(C * gh * gw):
        cam, tile = divmod(b, gh * gw)
        by, bx = divmod(tile, gw)
        start = int(flat_offs[b])
        end = n_points if b + 1 == C * gh * gw else int(flat_offs[b + 1])
        end = min(end, start + tile_width * tile_height)
        for k in range(start, end):
            tr = k - start
            i, j = by * tile_height + tr // tile_width, bx * tile_width + tr % tile_width
            if i < image_height and j < image_width:
                img[cam, i, j] = pts[flatten_ids[k]]
    return img
