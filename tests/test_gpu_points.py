"""Parity of the point -> tile -> raster image ops (through the C ABI) against the oracle:
bit-exact ids / lists / offsets / images, on the sizes of the reference's own tests
(tests/test_basic.py:787-890) and on edge cases (azimuth wrap, out-of-range elevation, empty and
overfull tiles, packed layout, unsorted)."""

import math

import numpy as np
import pytest
import torch

from gpu_util import DEV, n, t

pytestmark = pytest.mark.gpu


def _points(C, N, seed, az=(-200.0, 400.0), el=(-50.0, 50.0)):
    g = torch.Generator().manual_seed(seed)
    p = torch.zeros(C, N, 5)
    p[..., 0] = torch.rand(C, N, generator=g) * (az[1] - az[0]) + az[0]
    p[..., 1] = torch.rand(C, N, generator=g) * (el[1] - el[0]) + el[0]
    p[..., 2:] = torch.rand(C, N, 3, generator=g) + 0.5
    return p


@pytest.mark.parametrize("C,N,sort", [(1, 1, True), (3, 100_000, True), (2, 30_000, False), (1, 1_000_000, True)])
def test_map_points_and_offsets_vs_oracle(C, N, sort):
    from oracle import isect
    from splatad_b200 import ops
    pts = _points(C, N, 10 + C)
    eb = torch.linspace(-45.0, 45.0, 17)
    res, min_az = 0.2 * 16, -180.0
    want_ids, want_flat = isect.map_points_to_lidar_tiles(n(pts[..., :2]), n(eb), res, min_az, sort=sort)
    ids, flat = ops.map_points_to_lidar_tiles(t(pts[..., :2]), t(eb), res, min_az, sort=sort)
    assert ids.dtype == torch.int64 and flat.dtype == torch.int32
    assert np.array_equal(n(ids), want_ids) and np.array_equal(n(flat), want_flat)
    if sort:
        n_az = math.ceil(360 / res)
        offs = ops.points_mapping_offset_encode(ids, C, n_az, 16)
        assert np.array_equal(n(offs), isect.points_mapping_offset_encode(want_ids, C, n_az, 16))


def test_map_points_packed_and_empty():
    from oracle import isect
    from splatad_b200 import ops
    g = torch.Generator().manual_seed(3)
    nnz, C = 50_000, 4
    cam = torch.sort(torch.randint(0, C, (nnz,), generator=g)).values
    pts = _points(1, nnz, 5)[0, :, :2]
    eb = torch.tensor([-30.0, -12.0, -3.0, 0.5, 4.0, 25.0])
    want = isect.map_points_to_lidar_tiles(n(pts), n(eb), 7.5, -90.0, n_cameras=C, camera_ids=n(cam))
    got = ops.map_points_to_lidar_tiles(t(pts), t(eb), 7.5, -90.0, packed=True, n_cameras=C, camera_ids=cam.to(DEV))
    assert np.array_equal(n(got[0]), want[0]) and np.array_equal(n(got[1]), want[1])
    ids, flat = ops.map_points_to_lidar_tiles(torch.zeros(2, 0, 2, device=DEV), t(eb), 7.5, -90.0)
    assert ids.numel() == 0 and flat.numel() == 0
    offs = ops.points_mapping_offset_encode(ids, 2, 48, 5)
    assert offs.shape == (2, 5, 48) and int(offs.abs().sum()) == 0


@pytest.mark.parametrize("C,N,tw,th,W,H", [(3, 200_000, 32, 8, None, 32), (1, 5_000, 8, 4, 700, 14), (2, 0, 8, 4, 64, 8)])
def test_populate_image_vs_oracle(C, N, tw, th, W, H):
    """Full tiles (every pixel set, as the reference test requires), sparse tiles with an image that
    cuts the last tile column / row, and no points at all."""
    from oracle import isect
    from splatad_b200 import ops
    res = 0.5 * tw
    n_az, n_el = math.ceil(360 / res), math.ceil(H / th)
    W = n_az * tw if W is None else W
    eb = torch.linspace(-20 - 1e-2, 20 + 1e-2, n_el + 1)
    pts = _points(C, N, 21, az=(-180.0, 180.0), el=(-20.0, 20.0))
    ids, flat = ops.map_points_to_lidar_tiles(t(pts[..., :2]), t(eb), res, -180.0)
    offs = ops.points_mapping_offset_encode(ids, C, n_az, n_el)
    img = ops.populate_image_from_points(t(pts), W, H, tw, th, offs, flat)
    want = isect.populate_image_from_points(n(pts), W, H, tw, th, n(offs), n(flat))
    assert img.shape == (C, H, W, 5) and np.array_equal(n(img), want)
    if N >= 200_000:
        assert bool((img[..., 2] > 0).all())
