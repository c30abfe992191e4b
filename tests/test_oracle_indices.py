"""Pins of the oracle's rasterize_to_indices_in_range[_lidar] and accumulate[_lidar].

The reference has no CPU twin of the two index kernels; it tests them through its torch
compositor (gsplat/cuda/_torch_impl.py:822-1005: indices of a batch range -> accumulate -> add to
the running render), compared with the fused kernels in tests/test_basic.py. The same chain is
checked here on the oracle: (1) on the fixtures made with the reference's accumulate() the index
functions return exactly the pair lists the fixtures were generated from, and the restated
accumulate() reproduces the reference's renders; (2) the batched loop reproduces the oracle's
fused compositing, whose arithmetic is pinned separately.
"""

import math

import numpy as np
import torch

from oracle import composite, pipeline
from splatad_b200 import scenes


def _all_pairs_lists(C, N):
    offsets = (np.arange(C, dtype=np.int32) * N).reshape(C, 1, 1)
    return offsets, np.arange(C * N, dtype=np.int32)


def test_indices_and_accumulate_on_the_reference_fixture_pixels(golden):
    g = golden("accumulate_pixels")
    C, N = g["opacities"].shape
    W, H = int(g["width"]), int(g["height"])
    offsets, flat = _all_pairs_lists(C, N)
    T = np.ones((C, H, W), np.float32)
    for dtype, tol in ((np.float32, 2e-5), (np.float64, 2e-6)):
        out = composite.rasterize_to_indices_in_range(0, 10 ** 10, T, g["means2d"], g["conics"], g["opacities"],
                                                      g["pix_vels"], W, H, 8, offsets, flat, rs_time=g["rs"],
                                                      dtype=dtype)
        # the pair lists the fixture was generated from: every Gaussian for every pixel, pixel-major
        assert out["camera_ids"].tolist() == np.repeat(np.arange(C), W * H * N).tolist()
        assert out["pixel_ids"].tolist() == np.tile(np.repeat(np.arange(W * H), N), C).tolist()
        assert out["gaussian_ids"].tolist() == np.tile(np.arange(N), C * W * H).tolist()
        renders, alphas = composite.accumulate(g["means2d"], g["conics"], g["opacities"], g["colors"],
                                               g["pix_vels"], g["rs"], out["gaussian_ids"], out["pixel_ids"],
                                               out["camera_ids"], W, H, dtype=dtype)
        np.testing.assert_allclose(renders, g["renders"], rtol=tol, atol=tol)
        np.testing.assert_allclose(alphas, g["alphas"], rtol=tol, atol=tol)


def test_indices_and_accumulate_on_the_reference_fixture_points(golden):
    g = golden("accumulate_points")
    C, N = g["opacities"].shape
    W, H = int(g["width"]), int(g["height"])
    offsets, flat = _all_pairs_lists(C, N)
    T = np.ones((C, H, W), np.float32)
    for dtype, tol in ((np.float32, 5e-5), (np.float64, 5e-6)):
        out = composite.rasterize_to_indices_in_range_lidar(0, 1, T, g["means2d"], g["conics"], g["opacities"],
                                                            g["pix_vels"], g["raster_pts"], W, H, 8, 4, offsets,
                                                            flat, dtype=dtype)
        assert out["pixel_ids"].tolist() == np.tile(np.repeat(np.arange(W * H), N), C).tolist()
        assert out["gaussian_ids"].tolist() == np.tile(np.arange(N), C * W * H).tolist()
        renders, alphas, asum = composite.accumulate_lidar(
            g["means2d"], g["conics"], g["opacities"], g["features"], g["pix_vels"], g["depth_compensations"],
            g["raster_pts"], out["gaussian_ids"], out["pixel_ids"], out["camera_ids"], W, H, True,
            float(g["threshold"]), dtype=dtype)
        np.testing.assert_allclose(renders, g["renders"], rtol=tol, atol=tol * 10)
        np.testing.assert_allclose(alphas, g["alphas"], rtol=tol, atol=tol)
        np.testing.assert_allclose(asum, g["alpha_sum"], rtol=tol, atol=tol)


def _max_batches(offsets, n_isects, block):
    fl = np.concatenate([offsets.reshape(-1), [n_isects]])
    return int(math.ceil((fl[1:] - fl[:-1]).max() / block))


def test_batched_loop_reproduces_the_fused_pixels():
    kw = scenes.config1(N=4000, seed=11)
    kw.update(width=96, height=64, tile_size=8, sh_degree=None, render_mode="RGB",
              colors=torch.rand(4000, 3, generator=torch.Generator().manual_seed(5)))
    kw["Ks"] = torch.tensor([[[60.0, 0.0, 48.0], [0.0, 60.0, 32.0], [0.0, 0.0, 1.0]]])
    kw["scales"] = kw["scales"] * 2.0
    packed = kw.pop("packed")
    assert packed
    render, alphas, meta = pipeline.rasterization(**kw, dtype=np.float64)
    W, H, ts = 96, 64, 8
    offsets, flat = meta["isect_offsets"], meta["flatten_ids"]
    nb = _max_batches(offsets, flat.size, ts * ts)
    assert nb >= 3, nb   # the loop below really iterates
    rs = kw["rolling_shutter_time"].numpy()
    ok = ~meta["ambiguous"]
    assert ok.mean() > 0.99
    for per_iter in (nb, 1, 2):
        colors = np.zeros_like(render)
        acc = np.zeros_like(alphas)
        counts = np.zeros(alphas.shape[:3], np.int64)
        for step in range(0, nb, per_iter):
            T = 1.0 - acc[..., 0]
            out = composite.rasterize_to_indices_in_range(step, step + per_iter, T, meta["means2d"], meta["conics"],
                                                          meta["opacities"], meta["pix_vels"], W, H, ts, offsets,
                                                          flat, rs_time=rs, dtype=np.float64)
            if out["gaussian_ids"].size == 0:
                break
            counts += out["counts"]
            # sorted by (camera, pixel), like the cumulative-sum layout of the reference
            ray = out["camera_ids"] * W * H + out["pixel_ids"]
            assert (np.diff(ray) >= 0).all()
            r, a = composite.accumulate(meta["means2d"], meta["conics"], meta["opacities"], meta["colors"],
                                        meta["pix_vels"], rs, out["gaussian_ids"], out["pixel_ids"],
                                        out["camera_ids"], W, H)
            colors = colors + r * T[..., None]
            acc = acc + a * T[..., None]
        if per_iter == nb:
            # one call over the whole lists is the fused compositing, pair for pair
            assert counts.sum() == meta["contributing"]
            whole = counts
            sel = ok
        else:
            # a call does not know that a pixel stopped (T * (1 - alpha) <= 1e-4) in an earlier call:
            # such a pixel resumes with the transmittance it had before the stopping Gaussian. That is
            # the reference's behaviour too (its kernel keeps no such state); those pixels are set aside.
            sel = ok & (counts == whole)
            assert sel.mean() > 0.9 and (counts >= whole).all()
        np.testing.assert_allclose(colors[sel], render[sel], rtol=1e-9, atol=1e-10)
        np.testing.assert_allclose(acc[sel], alphas[sel], rtol=1e-9, atol=1e-10)


def test_batched_loop_reproduces_the_fused_points():
    kw = scenes.config0(N=6000, seed=12)
    feats, alphas, asum, meta = pipeline.lidar_rasterization(**kw, dtype=np.float64)
    H, W = kw["raster_pts"].shape[1:3]
    tw, th = kw["tile_width"], kw["tile_height"]
    offsets, flat = meta["isect_offsets"], meta["flatten_ids"]
    nb = _max_batches(offsets, flat.size, tw * th)
    assert nb >= 2, nb
    pts = kw["raster_pts"].numpy()
    lf = np.concatenate([kw["lidar_features"].numpy().astype(np.float64), meta["depths"][..., None]], axis=-1)
    ok = ~meta["ambiguous"]
    thr = 0.2
    for per_iter in (nb, 1):
        render = np.zeros_like(feats)
        acc = np.zeros_like(alphas)
        sums = np.zeros_like(alphas)
        counts = np.zeros(alphas.shape[:3], np.int64)
        for step in range(0, nb, per_iter):
            T = 1.0 - acc[..., 0]
            out = composite.rasterize_to_indices_in_range_lidar(step, step + per_iter, T, meta["means2d"],
                                                                meta["conics"], meta["opacities"], meta["pix_vels"],
                                                                pts, W, H, tw, th, offsets, flat, dtype=np.float64)
            if out["gaussian_ids"].size == 0:
                break
            counts += out["counts"]
            r, a, s = composite.accumulate_lidar(meta["means2d"], meta["conics"], meta["opacities"], lf,
                                                 meta["pix_vels"], meta["depth_compensations"], pts,
                                                 out["gaussian_ids"], out["pixel_ids"], out["camera_ids"], W, H,
                                                 True, thr)
            render = render + r * T[..., None]
            acc = acc + a * T[..., None]
            sums = sums + s
        if per_iter == nb:
            assert counts.sum() == meta["contributing"]
            whole = counts
            sel = ok
        else:
            sel = ok & (counts == whole)   # pixels that did not resume after a stop, see the camera test
            assert sel.mean() > 0.9 and (counts >= whole).all()
        np.testing.assert_allclose(render[sel], feats[sel], rtol=1e-9, atol=1e-9)
        np.testing.assert_allclose(acc[sel], alphas[sel], rtol=1e-9, atol=1e-10)
        np.testing.assert_allclose(sums[sel], asum[sel], rtol=1e-9, atol=1e-10)


def test_edge_cases():
    # no intersections at all; a range past every list; points that are not rendered (range <= 0)
    C, N, W, H = 1, 4, 8, 8
    z = np.zeros
    out = composite.rasterize_to_indices_in_range(0, 5, np.ones((C, H, W)), z((C, N, 2)), z((C, N, 3)), z((C, N)),
                                                  z((C, N, 2)), W, H, 4, z((C, 2, 2), np.int32), z(0, np.int32))
    assert out["gaussian_ids"].size == 0 and out["pixel_ids"].size == 0
    means2d = np.full((C, N, 2), 4.0)
    conics = np.tile(np.array([0.05, 0.0, 0.05]), (C, N, 1))
    opac = np.full((C, N), 0.5)
    offsets = np.array([[[0, 4], [8, 12]]], np.int32)
    flat = np.tile(np.arange(4, dtype=np.int32), 4)
    args = (means2d, conics, opac, z((C, N, 2)), W, H, 4, offsets, flat)
    full = composite.rasterize_to_indices_in_range(0, 1, np.ones((C, H, W)), *args)
    assert full["gaussian_ids"].size == W * H * N
    assert composite.rasterize_to_indices_in_range(1, 2, np.ones((C, H, W)), *args)["gaussian_ids"].size == 0
    # a pixel that is already opaque stops at its first Gaussian and contributes nothing
    T = np.ones((C, H, W))
    T[0, 3, 3] = 1e-4
    part = composite.rasterize_to_indices_in_range(0, 1, T, *args)
    assert part["counts"][0, 3, 3] == 0 and part["gaussian_ids"].size == (W * H - 1) * N
    pts = z((C, H, W, 4))
    pts[..., 0] = 4.0
    pts[..., 1] = 4.0
    pts[..., 2] = 10.0
    pts[0, 0, 0, 2] = 0.0
    lid = composite.rasterize_to_indices_in_range_lidar(0, 1, np.ones((C, H, W)), means2d, conics, opac,
                                                        z((C, N, 3)), pts, W, H, 4, 4, offsets, flat)
    assert lid["counts"][0, 0, 0] == 0 and lid["gaussian_ids"].size == (W * H - 1) * N
