"""Pins of the oracle's point -> tile -> raster image functions. The reference has no torch twin of
these three ops; its tests assert properties of the CUDA results (tests/test_basic.py:787-890),
restated here on the oracle at a smaller size, plus a hand-worked example."""

import math

import numpy as np

from oracle import isect


def test_map_points_properties_like_the_reference_test():
    rng = np.random.default_rng(42)
    C, N = 3, 100_000   # as in the reference test: the last tile is half as wide as the others
    width, height, min_azimuth = 360.0, 90.0, -180
    tile_azim_resolution = 0.2 * 16
    n_azim_tiles = math.ceil(360 / tile_azim_resolution)
    n_elev_tiles = 16
    eb = np.linspace(-height / 2.0, height / 2.0, n_elev_tiles + 1).astype(np.float32)
    p = np.zeros((C, N, 2), np.float32)
    p[..., 0] = rng.random((C, N)) * width - width / 2
    p[..., 1] = rng.random((C, N)) * height - height / 2
    ids, flat = isect.map_points_to_lidar_tiles(p, eb, tile_azim_resolution, min_azimuth)
    offs = isect.points_mapping_offset_encode(ids, C, n_azim_tiles, n_elev_tiles)
    cam, tile = ids >> 32, ids & 0xFFFFFFFF
    assert cam.shape[0] == C * N and len(np.unique(cam)) == C
    for i in range(C):
        assert np.unique(cam[i * N:(i + 1) * N])[0] == i
        t = tile[i * N:(i + 1) * N]
        assert (t[:-1] <= t[1:]).all() and t.max() < n_azim_tiles * n_elev_tiles
        last = p.reshape(-1, 2)[flat[i * N:(i + 1) * N][-10:]]
        assert (last[:, 0] <= width / 2).all() and (last[:, 0] >= width / 2 - tile_azim_resolution).all()
        assert (last[:, 1] <= eb[-1]).all() and (last[:, 1] >= eb[-2]).all()
        o = offs[i].reshape(-1)
        assert (o[1:] >= o[:-1]).all()
    assert offs.shape == (C, n_elev_tiles, n_azim_tiles)
    # stable: inside a tile the points keep their order
    same = ids[1:] == ids[:-1]
    assert (flat[1:][same] > flat[:-1][same]).all()


def test_known_answer():
    # two elevation tiles (boundaries -10, 0, 10), azimuth tiles of 90 degrees from -180
    eb = np.array([-10.0, 0.0, 10.0], np.float32)
    pts = np.array([[[-170.0, 5.0], [100.0, -5.0], [-170.0, -20.0], [190.0, 5.0], [-180.0, 0.0], [179.0, 9.0]]],
                   np.float32)
    ids, flat = isect.map_points_to_lidar_tiles(pts, eb, 90.0, -180.0, sort=False)
    # azimuth tiles: -170 -> 0, 100 -> 3, 190 wraps to 10 deg from the start -> 0, -180 -> 0, 179 -> 3
    # elevation tiles: 5 -> 1 (two boundaries below), -5 -> 0, -20 -> 0 (none below, clamped), 0 -> 0
    # (only -10 is strictly below)
    assert ids.tolist() == [4 + 0, 0 + 3, 0 + 0, 4 + 0, 0 + 0, 4 + 3] and flat.tolist() == [0, 1, 2, 3, 4, 5]
    ids, flat = isect.map_points_to_lidar_tiles(pts, eb, 90.0, -180.0)
    assert ids.tolist() == [0, 0, 3, 4, 4, 7] and flat.tolist() == [2, 4, 1, 0, 3, 5]
    offs = isect.points_mapping_offset_encode(ids, 1, 4, 2)
    assert offs.reshape(-1).tolist() == [0, 2, 2, 2, 3, 5, 5, 5]
    vals = np.arange(30, dtype=np.float32).reshape(1, 6, 5)
    img = isect.populate_image_from_points(vals, 8, 2, 2, 1, offs, flat)
    # tiles are 2 pixels wide and 1 high: tile (0,0) takes points 2 and 4, tile (0,3) point 1, ...
    assert img.shape == (1, 2, 8, 5)
    assert img[0, 0, 0].tolist() == vals[0, 2].tolist() and img[0, 0, 1].tolist() == vals[0, 4].tolist()
    assert img[0, 0, 6].tolist() == vals[0, 1].tolist() and float(np.abs(img[0, 0, 2:6]).sum()) == 0.0
    assert img[0, 1, 0].tolist() == vals[0, 0].tolist() and img[0, 1, 1].tolist() == vals[0, 3].tolist()
    assert img[0, 1, 6].tolist() == vals[0, 5].tolist()


def test_populate_fills_every_pixel_when_tiles_are_full():
    rng = np.random.default_rng(1)
    C, N, tw, th, n_chan = 2, 40_000, 8, 4, 16
    res = 0.5 * tw
    n_az, n_el = math.ceil(360 / res), n_chan // th
    eb = np.linspace(-20 - 1e-2, 20 + 1e-2, n_el + 1).astype(np.float32)
    pts = np.zeros((C, N, 5), np.float32)
    pts[..., 0] = rng.random((C, N)) * 360 - 180
    pts[..., 1] = rng.random((C, N)) * 40 - 20
    pts[..., 2:] = rng.random((C, N, 3)) + 0.5
    ids, flat = isect.map_points_to_lidar_tiles(pts[..., :2], eb, res, -180.0)
    offs = isect.points_mapping_offset_encode(ids, C, n_az, n_el)
    img = isect.populate_image_from_points(pts, n_az * tw, n_chan, tw, th, offs, flat)
    assert img.shape == (C, n_chan, n_az * tw, 5) and (img[..., 2] > 0).all()
