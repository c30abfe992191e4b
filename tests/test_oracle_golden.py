"""The CPU oracle against the golden vectors produced by the reference's own PyTorch code
(tests/golden/make_golden.py). These pin the oracle; the GPU tests then compare the CUDA
library with the oracle (and with the same fixtures)."""

import numpy as np
import torch

from oracle import composite, isect, projection


def t(a, dtype=torch.float32):
    return torch.from_numpy(np.asarray(a)).to(dtype)


def test_quat_scale_to_covar(golden):
    g = golden("quat_scale_to_covar")
    cov = projection.quat_scale_to_covar(t(g["quats"]), t(g["scales"]))
    np.testing.assert_allclose(cov.numpy(), g["covars"], rtol=1e-5, atol=1e-6)


def test_lidar_projection(golden):
    g = golden("lidar_projection")
    out = projection.fully_fused_lidar_projection(
        t(g["means"]), None, t(g["quats"]), t(g["scales"]), t(g["velocities"]), t(g["viewmats"]),
        t(g["lin"]), t(g["ang"]), t(g["rs"]), float(g["min_elevation"]), float(g["max_elevation"]),
        float(g["min_azimuth"]), float(g["max_azimuth"]), float(g["eps2d"]), float(g["near_plane"]),
        float(g["far_plane"]), 0.0, True)
    radii, means2d, depths, conics, comps, pix_vels, dcomp = [o.numpy() for o in out]
    vis_ref = g["radii"][..., 0] > 0
    vis = radii[..., 0] > 0
    assert (vis == vis_ref).mean() > 0.999  # culling decisions (identical up to rounding at a border)
    m = vis & vis_ref
    assert m.sum() > 300
    np.testing.assert_allclose(radii[m], g["radii"][m], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(means2d[m], g["means2d"][m], rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(depths[m], g["depths"][m], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(conics[m], g["conics"][m], rtol=2e-3, atol=1e-5)
    np.testing.assert_allclose(comps[m], g["compensations"][m], rtol=1e-3, atol=1e-5)
    np.testing.assert_allclose(pix_vels[m], g["pix_vels"][m], rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(dcomp[m], g["depth_compensations"][m], rtol=5e-3, atol=1e-4)


def test_camera_projection(golden):
    g = golden("camera_projection")
    out = projection.fully_fused_projection(
        t(g["means"]), None, t(g["quats"]), t(g["scales"]), t(g["velocities"]), t(g["viewmats"]),
        t(g["Ks"]), int(g["width"]), int(g["height"]), t(g["lin"]), t(g["ang"]), t(g["rs"]),
        float(g["eps2d"]), float(g["near_plane"]), float(g["far_plane"]), 0.0, True)
    radii, means2d, depths, conics, comps, pix_vels = [o.numpy() for o in out]
    vis_ref = g["radii"][..., 0] > 0
    vis = radii[..., 0] > 0
    assert (vis == vis_ref).mean() > 0.999
    m = vis & vis_ref
    assert m.sum() > 100
    assert np.abs(radii[m].astype(np.int64) - g["radii"][m]).max() <= 1  # int truncation at a rounding edge
    assert (radii[m] == g["radii"][m]).mean() > 0.995
    np.testing.assert_allclose(means2d[m], g["means2d"][m], rtol=1e-4, atol=1e-3)
    np.testing.assert_allclose(depths[m], g["depths"][m], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(conics[m], g["conics"][m], rtol=2e-3, atol=1e-6)
    np.testing.assert_allclose(comps[m], g["compensations"][m], rtol=1e-3, atol=1e-5)
    np.testing.assert_allclose(pix_vels[m], g["pix_vels"][m], rtol=1e-3, atol=1e-2)


def test_isect_tiles_bit_exact(golden):
    g = golden("isect_tiles")
    tpg, ids, flat = isect.isect_tiles(g["means2d"], g["radii"], g["depths"], int(g["tile_size"]),
                                       int(g["tile_width"]), int(g["tile_height"]))
    offs = isect.isect_offset_encode(ids, g["means2d"].shape[0], int(g["tile_width"]), int(g["tile_height"]))
    assert np.array_equal(tpg, g["tiles_per_gauss"])
    assert np.array_equal(ids, g["isect_ids"])
    assert np.array_equal(flat, g["flatten_ids"])
    assert np.array_equal(offs, g["isect_offsets"])


def _check_lidar(g):
    tpg, ids, flat = isect.isect_lidar_tiles(g["means2d"], g["radii"], g["depths"], g["elev_boundaries"],
                                             float(g["tile_azim_resolution"]), float(g["min_azimuth"]))
    offs = isect.isect_offset_encode(ids, g["means2d"].shape[0], int(g["n_azim_tiles"]), int(g["n_elev_tiles"]))
    assert np.array_equal(tpg, g["tiles_per_gauss"])
    assert np.array_equal(ids, g["isect_ids"])
    assert np.array_equal(flat, g["flatten_ids"])
    assert np.array_equal(offs, g["isect_offsets"])


def test_isect_lidar_tiles_bit_exact(golden):
    _check_lidar(golden("isect_lidar_tiles"))


def test_isect_lidar_tiles_wrap_bit_exact(golden):
    _check_lidar(golden("isect_lidar_tiles_wrap"))


def test_spherical_harmonics(golden):
    g = golden("spherical_harmonics")
    for d in range(5):
        out = projection.spherical_harmonics(d, t(g["dirs"]), t(g["coeffs"]))
        np.testing.assert_allclose(out.numpy(), g[f"colors_deg{d}"], rtol=1e-4, atol=1e-5)


def _all_pairs_lists(C, n_pix, N):
    """Every tile = one sensor's whole image, every Gaussian listed once per sensor in index order."""
    offsets = (np.arange(C, dtype=np.int32) * N).reshape(C, 1, 1)
    flatten_ids = np.arange(C * N, dtype=np.int32)
    return offsets, flatten_ids


def test_composite_pixels_against_reference_accumulate(golden):
    g = golden("accumulate_pixels")
    C, N = g["opacities"].shape
    W, H = int(g["width"]), int(g["height"])
    offsets, flat = _all_pairs_lists(C, W * H, N)
    for dtype, tol in ((np.float32, 2e-5), (np.float64, 2e-6)):
        # one tile of size >= max(W, H) covers the image
        out = composite.rasterize_to_pixels_fwd(g["means2d"], g["conics"], g["colors"], g["opacities"],
                                                g["pix_vels"], g["rs"], None, W, H, 8, offsets, flat, dtype=dtype)
        np.testing.assert_allclose(out["render_colors"], g["renders"], rtol=tol, atol=tol)
        np.testing.assert_allclose(out["render_alphas"], g["alphas"], rtol=tol, atol=tol)
        assert out["contributing"] == C * W * H * N  # nothing was thresholded away in this fixture


def test_composite_points_against_reference_accumulate(golden):
    g = golden("accumulate_points")
    C, N = g["opacities"].shape
    W, H = int(g["width"]), int(g["height"])
    offsets, flat = _all_pairs_lists(C, W * H, N)
    for dtype, tol in ((np.float32, 5e-5), (np.float64, 5e-6)):
        out = composite.rasterize_to_points_fwd(
            g["means2d"], g["conics"], g["features"], g["opacities"], g["pix_vels"],
            g["depth_compensations"], None, g["raster_pts"], W, H, 8, 4, offsets, flat, True,
            float(g["threshold"]), dtype=dtype)
        np.testing.assert_allclose(out["render_colors"], g["renders"], rtol=tol, atol=tol * 10)
        np.testing.assert_allclose(out["render_alphas"], g["alphas"], rtol=tol, atol=tol)
        np.testing.assert_allclose(out["alpha_sum"], g["alpha_sum"], rtol=tol, atol=tol)
        assert out["contributing"] == C * W * H * N
