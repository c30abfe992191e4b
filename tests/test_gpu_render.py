"""End-to-end parity of ``lidar_rasterization`` / ``rasterization`` against the CPU oracle
pipeline on the benchmark configurations at sizes the oracle finishes in seconds.

Bars: tile counts, tile offsets and sorted Gaussian id lists bit-exact; rendered features / RGB /
alpha within 1e-4 relative + 1e-5 absolute, range within 1 mm, on all pixels whose threshold
decisions are not flagged ambiguous by the oracle. A Gaussian whose tile rectangle differs
between the two projections (a one-ulp difference at a tile border) would break bit-exactness;
the count of such Gaussians is reported and must be zero for the seeded scenes used here.
"""

import numpy as np
import pytest
import torch

from gpu_util import DEV, assert_close, n

pytestmark = pytest.mark.gpu


def _to_gpu(cfg):
    return {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in cfg.items()}


def _lidar_stagewise_reference(cfg, m, **kw):
    """Oracle isect + compositing run on the PRODUCT's projection outputs (identical stage
    inputs), plus the number of Gaussians whose tile count differs from the one obtained with
    the oracle's own projection."""
    from oracle import pipeline
    from splatad_b200 import ops
    C = cfg["viewmats"].shape[0]
    g = _to_gpu(cfg)
    lin = g.get("linear_velocity", torch.zeros(C, 3, device=DEV))
    ang = g.get("angular_velocity", torch.zeros(C, 3, device=DEV))
    rs = g.get("rolling_shutter_time", torch.zeros(C, device=DEV))
    proj = ops.fully_fused_lidar_projection(
        g["means"], None, g["quats"], g["scales"], g["velocities"], g["viewmats"], lin, ang, rs,
        min_elevation=cfg["min_elevation"], max_elevation=cfg["max_elevation"], min_azimuth=cfg["min_azimuth"],
        max_azimuth=cfg["max_azimuth"], eps2d=cfg["eps2d"],
        calc_compensations=kw.get("rasterize_mode") == "antialiased")
    radii, means2d, depths, conics, comps, pix_vels, dcomp = proj
    assert torch.equal(radii, m["radii"]) and torch.equal(means2d, m["means2d"])
    if not kw.get("use_depth_compensation", True):
        dcomp = dcomp * 0
    asum = kw.get("compute_alpha_sum_until_points", True)
    ref = pipeline.lidar_from_projection(
        n(radii), n(means2d), n(depths), n(conics), n(m["opacities"]), n(pix_vels), n(dcomp),
        n(cfg["lidar_features"]), n(cfg["raster_pts"]), n(cfg["tile_elevation_boundaries"]),
        min_azimuth=cfg["min_azimuth"], max_azimuth=cfg["max_azimuth"],
        n_elevation_channels=cfg["n_elevation_channels"], azimuth_resolution=cfg["azimuth_resolution"],
        tile_width=cfg["tile_width"], tile_height=cfg["tile_height"], compute_alpha_sum_until_points=asum)
    tpg = ref["tiles_per_gauss"]
    # rectangles from the oracle's own projection of the same Gaussians
    _, _, _, ometa = pipeline.lidar_rasterization(**cfg, **kw)
    rect_diff = int((ometa["tiles_per_gauss"] != tpg).sum())
    ref.update(rect_diff=rect_diff, oracle_meta=ometa)
    return ref


def _check_lists(m, ref, label):
    assert np.array_equal(n(m["tiles_per_gauss"]), ref["tiles_per_gauss"]), f"{label}: tile counts differ"
    assert np.array_equal(n(m["isect_offsets"]), ref["isect_offsets"]), f"{label}: tile offsets differ"
    assert np.array_equal(n(m["flatten_ids"]), ref["flatten_ids"]), f"{label}: sorted Gaussian id lists differ"
    assert np.array_equal(n(m["isect_ids"]), ref["isect_ids"]), f"{label}: isect ids differ"
    total = ref["tiles_per_gauss"].size
    print(f"{label}: {ref['rect_diff']} of {total} (sensor, Gaussian) pairs get a different tile count from the "
          f"oracle's own float32 projection")
    assert ref["rect_diff"] <= max(2, total // 2000), f"{label}: {ref['rect_diff']} tile rectangles differ"


def _check_lidar_render(label, out_c, out_a, out_s, m, ref):
    o = ref["out"]
    ok = ~o["ambiguous"][..., None]
    assert o["ambiguous"].mean() < 0.01
    assert_close(label + " features+range", n(out_c), o["render_colors"], 1e-4, 1e-5, mask=ok)
    assert_close(label + " alpha", n(out_a), o["render_alphas"], 1e-4, 1e-5, mask=ok)
    if out_s is not None:
        assert_close(label + " alpha sum", n(out_s), o["alpha_sum"], 1e-4, 1e-5, mask=ok)
    d = np.abs(n(out_c)[..., -1] - o["render_colors"][..., -1])[~o["ambiguous"]]
    lim = 1e-3 + 1e-4 * np.abs(o["render_colors"][..., -1])[~o["ambiguous"]]
    assert (d <= lim).all(), f"{label}: range differs by {d.max()} m"


def test_config0_lidar():
    import splatad_b200
    from splatad_b200 import scenes
    cfg = scenes.config0()
    out_c, out_a, out_s, m = splatad_b200.lidar_rasterization(**_to_gpu(cfg))
    assert out_c.shape == (1, 32, 512, 5) and out_a.shape == (1, 32, 512, 1) and out_s.shape == (1, 32, 512, 1)
    for key in ("camera_ids", "gaussian_ids", "radii", "means2d", "depths", "conics", "opacities", "pix_vels",
                "tile_grid_width", "tile_grid_height", "tiles_per_gauss", "isect_ids", "flatten_ids",
                "isect_offsets", "width", "height", "tile_width", "tile_height", "n_cameras", "median_depths"):
        assert key in m, key
    ref = _lidar_stagewise_reference(cfg, m)
    _check_lists(m, ref, "config0")
    _check_lidar_render("config0", out_c, out_a, out_s, m, ref)
    ok = ~ref["out"]["ambiguous"][..., None]
    assert_close("config0 median", n(m["median_depths"]), ref["out"]["median_depths"], 1e-4, 1e-3, mask=ok)
    # and against the fully independent oracle pipeline (own projection), away from flagged pixels
    # and from pixels touched by a differing rectangle
    if ref["rect_diff"] == 0:
        from oracle import pipeline
        ref_c, ref_a, ref_s, meta = pipeline.lidar_rasterization(**cfg)
        ok2 = ~meta["ambiguous"][..., None]
        assert_close("config0 vs independent oracle", n(out_c), ref_c, 2e-4, 2e-4, mask=ok2, max_bad_frac=1e-3)


def test_config2_lidar_reduced():
    """Config 2's sensor (128 x 1800, rolling shutter) on 60k Gaussians."""
    import splatad_b200
    from splatad_b200 import scenes
    cfg = scenes.config2(N=60_000)
    out_c, out_a, out_s, m = splatad_b200.lidar_rasterization(**_to_gpu(cfg))
    assert out_c.shape == (1, 128, 1800, 17)
    ref = _lidar_stagewise_reference(cfg, m)
    _check_lists(m, ref, "config2/60k")
    _check_lidar_render("config2/60k", out_c, out_a, out_s, m, ref)


def test_lidar_channel_chunking_and_options():
    """40 features (> 32 -> chunks of 31 + range), antialiased mode, depth compensation off,
    alpha sum off, two sensors."""
    import splatad_b200
    from oracle import pipeline
    from splatad_b200 import scenes
    cfg = scenes.config0(N=6000)
    g = torch.Generator().manual_seed(5)
    cfg["lidar_features"] = torch.randn(2, 6000, 40, generator=g)
    cfg["viewmats"] = cfg["viewmats"].repeat(2, 1, 1)
    cfg["viewmats"][1, 0, 3] = 1.5
    cfg["raster_pts"] = cfg["raster_pts"].repeat(2, 1, 1, 1)
    kw = dict(rasterize_mode="antialiased", use_depth_compensation=False, compute_alpha_sum_until_points=False)
    ref_c, ref_a, ref_s, meta = pipeline.lidar_rasterization(**cfg, **kw)
    out_c, out_a, out_s, m = splatad_b200.lidar_rasterization(**_to_gpu(cfg), **kw)
    assert out_s is None and out_c.shape == (2, 32, 512, 41)
    assert m["median_depths"].shape == (2, 32, 512, 2)
    assert int((n(m["tiles_per_gauss"]) != meta["tiles_per_gauss"]).sum()) <= 2
    ok = ~meta["ambiguous"][..., None]
    # independent oracle (own projection): projection rounding differences show up at 1e-4 level
    assert_close("chunked features", n(out_c), ref_c, 3e-4, 3e-4, mask=ok, max_bad_frac=1e-3)
    assert_close("chunked alpha", n(out_a), ref_a, 3e-4, 1e-4, mask=ok, max_bad_frac=1e-3)
    # chunks agree with each other: the range channel of a one-chunk render of the first 31 features
    cfg31 = dict(cfg, lidar_features=cfg["lidar_features"][..., :31].contiguous())
    c31, a31, _, _ = splatad_b200.lidar_rasterization(**_to_gpu(cfg31), **kw)
    # (same decisions and products; the range is accumulated from its own array in one case and as
    # the last feature column in the other, which the compiler may contract differently)
    assert torch.equal(c31[..., :31], out_c[..., :31]) and torch.equal(a31, out_a)
    assert_close("range of chunked vs single render", n(c31[..., -1]), n(out_c[..., -1]), 1e-6, 1e-7)


@pytest.mark.parametrize("packed", [True, False])
def test_config1_camera_reduced(packed):
    """Config 1's camera (1920 x 1080, rolling shutter, SH degree 3, RGB+D) on 30k Gaussians.
    Lists are bit-exact against the oracle's isect run on the product's projection outputs; the
    image is compared with the fully independent oracle pipeline."""
    import math
    import splatad_b200
    from oracle import isect, pipeline
    from splatad_b200 import scenes
    cfg = scenes.config1(N=30_000, packed=packed)
    out_c, out_a, m = splatad_b200.rasterization(**_to_gpu(cfg))
    assert out_c.shape == (1, 1080, 1920, 4) and out_a.shape == (1, 1080, 1920, 1)
    for key in ("camera_ids", "gaussian_ids", "radii", "means2d", "depths", "conics", "opacities", "pix_vels",
                "tile_width", "tile_height", "tiles_per_gauss", "isect_ids", "flatten_ids", "isect_offsets",
                "width", "height", "tile_size", "n_cameras"):
        assert key in m, key
    tw, th = math.ceil(1920 / 16), math.ceil(1080 / 16)
    cam_ids = n(m["camera_ids"]) if packed else None
    tpg, ids, flat = isect.isect_tiles(n(m["means2d"]), n(m["radii"]), n(m["depths"]), 16, tw, th, n_cameras=1,
                                       camera_ids=cam_ids)
    offs = isect.isect_offset_encode(ids, 1, tw, th)
    assert np.array_equal(n(m["tiles_per_gauss"]), tpg), "tile counts differ"
    assert np.array_equal(n(m["isect_ids"]), ids), "isect ids differ"
    assert np.array_equal(n(m["flatten_ids"]), flat), "sorted Gaussian id lists differ"
    assert np.array_equal(n(m["isect_offsets"]), offs), "tile offsets differ"

    ref_c, ref_a, meta = pipeline.rasterization(**cfg)
    got_tpg = n(m["tiles_per_gauss"])
    if packed:
        dense = np.zeros(30_000, np.int32)
        dense[n(m["gaussian_ids"])] = got_tpg
        got_tpg = dense[None]
    rect_diff = int((got_tpg != meta["tiles_per_gauss"]).sum())
    print(f"config1/30k packed={packed}: {rect_diff} Gaussians get a different tile count from the oracle's "
          f"own float32 projection")
    assert rect_diff <= 15
    ok = ~meta["ambiguous"][..., None]
    assert meta["ambiguous"].mean() < 0.01
    # independent projection: rounding differences of the projected means / conics reach the image
    assert_close("config1 RGB+D", n(out_c), ref_c, 5e-4, 5e-4, mask=ok, max_bad_frac=2e-3)
    assert_close("config1 alpha", n(out_a), ref_a, 5e-4, 1e-4, mask=ok, max_bad_frac=2e-3)


@pytest.mark.parametrize("mode", ["RGB", "D", "ED", "RGB+ED"])
def test_camera_render_modes_and_backgrounds(mode):
    import splatad_b200
    from oracle import pipeline
    from splatad_b200 import scenes
    cfg = scenes.config1(N=4000, packed=False)
    cfg.update(width=320, height=200, render_mode=mode, sh_degree=None)
    cfg["Ks"] = torch.tensor([[[250.0, 0.0, 160.0], [0.0, 250.0, 100.0], [0.0, 0.0, 1.0]]])
    g = torch.Generator().manual_seed(3)
    cfg["colors"] = torch.rand(4000, 3, generator=g)
    cfg["backgrounds"] = torch.rand(1, 3, generator=g)
    ref_c, ref_a, meta = pipeline.rasterization(**cfg)
    out_c, out_a, m = splatad_b200.rasterization(**_to_gpu(cfg))
    assert out_c.shape == ref_c.shape
    ok = ~meta["ambiguous"][..., None]
    assert_close(f"mode {mode}", n(out_c), ref_c, 5e-4, 5e-4, mask=ok, max_bad_frac=2e-3)
    assert_close(f"mode {mode} alpha", n(out_a), ref_a, 5e-4, 1e-4, mask=ok, max_bad_frac=2e-3)


def test_lidar_training_step_gradients_flow():
    """Forward + backward through the whole lidar path: gradients reach every Gaussian parameter,
    ``meta["means2d"]`` receives its gradient and, with ``absgrad``, the sum of absolute
    contributions, which bounds it. The values of the gradients are compared with an independent
    float64 chain in ``test_gpu_gradients.py``."""
    import splatad_b200
    from splatad_b200 import scenes
    cfg = _to_gpu(scenes.config0(N=3000))
    names = ("means", "quats", "scales", "opacities", "lidar_features")
    for k in names:
        cfg[k] = cfg[k].clone().requires_grad_(True)
    out_c, out_a, out_s, m = splatad_b200.lidar_rasterization(**cfg, absgrad=True)
    m["means2d"].retain_grad()
    g = torch.Generator().manual_seed(1)
    w_c = torch.randn(out_c.shape, generator=g).to(DEV)
    w_a = torch.randn(out_a.shape, generator=g).to(DEV)
    ((out_c * w_c).sum() + (out_a * w_a).sum()).backward()
    for k in names:
        assert cfg[k].grad is not None and torch.isfinite(cfg[k].grad).all(), k
        assert float(cfg[k].grad.abs().sum()) > 0, k
    assert m["means2d"].grad is not None and hasattr(m["means2d"], "absgrad")
    assert torch.all(m["means2d"].absgrad + 1e-6 >= m["means2d"].grad.abs())


def test_repeated_frames_skip_the_count_round_trip():
    """From the second frame of a shape on, plan and fill are enqueued with a capacity guessed from
    the previous count. Results must not depend on that: same lists, same render, same gradients;
    and a frame whose count outgrows the guess is redone the two-step way."""
    import splatad_b200
    from splatad_b200 import ops, scenes
    cfg = scenes.config2(N=40_000)
    g = _to_gpu(cfg)
    ops._isect_count_hint.clear()
    first = splatad_b200.lidar_rasterization(**g)            # no hint yet: two-step protocol
    assert len(ops._isect_count_hint) == 1
    second = splatad_b200.lidar_rasterization(**g)           # hinted
    for a, b in zip(first[:3], second[:3]):
        assert torch.equal(a, b)
    for key in ("tiles_per_gauss", "isect_ids", "flatten_ids", "isect_offsets", "median_depths"):
        assert torch.equal(first[3][key], second[3][key]), key
    assert second[3]["isect_ids"].numel() == first[3]["isect_ids"].numel()
    # three times the scale -> far more intersections than the hint allows for
    big = dict(g, scales=g["scales"] * 3.0)
    key = next(iter(ops._isect_count_hint))
    hinted = ops._isect_count_hint[key]
    third = splatad_b200.lidar_rasterization(**big)
    assert third[3]["isect_ids"].numel() > hinted + hinted // 8 + 65536
    ops._isect_count_hint.clear()
    want = splatad_b200.lidar_rasterization(**big)           # two-step protocol again
    for a, b in zip(third[:3], want[:3]):
        assert torch.equal(a, b)
    assert torch.equal(third[3]["isect_ids"], want[3]["isect_ids"])
    assert torch.equal(third[3]["flatten_ids"], want[3]["flatten_ids"])
    # gradients through a hinted frame equal those of a two-step frame
    grads = []
    for _ in range(2):
        leaves = {k: g[k].clone().requires_grad_(True) for k in ("means", "quats", "scales", "opacities")}
        out = splatad_b200.lidar_rasterization(**dict(big, **leaves))
        (out[0].square().mean() + out[1].mean()).backward()
        grads.append({k: v.grad.clone() for k, v in leaves.items()})
    for k in grads[0]:
        assert_close(f"hinted grad {k}", n(grads[1][k]), n(grads[0][k]), 1e-4, 1e-7, max_bad_frac=1e-3)


def test_depth_range_carried_over_between_lidar_frames():
    """From the third frame of a shape on, the depth buckets span the previous frame's depth range
    (widened) and the rectangle count fills them. Whatever that range is, the lists and the render are
    those of a first frame; a range so wrong that an end bucket overflows is dropped, not mistaken for
    crowded depths."""
    import struct
    import splatad_b200
    from splatad_b200 import ops, scenes
    bits = lambda v: struct.unpack("<I", struct.pack("<f", v))[0]   # noqa: E731
    g = _to_gpu(scenes.config2(N=150_001))    # a shape of its own
    ops._isect_count_hint.clear()
    ops._depth_range_hint.clear()
    first = splatad_b200.lidar_rasterization(**g)      # two-step protocol
    second = splatad_b200.lidar_rasterization(**g)     # one call per frame; reports its depth range
    assert len(ops._depth_range_hint) == 1
    key = next(iter(ops._depth_range_hint))
    lo, hi = ops._depth_range_hint[key]
    depths = first[3]["depths"][first[3]["radii"][..., 0] > 0]
    assert (lo, hi) == (bits(float(depths.min())), bits(float(depths.max())))

    def same(frame):
        for a, b in zip(first[:3], frame[:3]):
            assert torch.equal(a, b)
        for name in ("tiles_per_gauss", "isect_ids", "flatten_ids", "isect_offsets", "median_depths"):
            assert torch.equal(first[3][name], frame[3][name]), name

    same(second)
    same(splatad_b200.lidar_rasterization(**g))        # buckets over the carried range
    # a range that covers only the near fifth of the depths: everything else lands in the last bucket
    ops._depth_range_hint[key] = (lo, bits(float(depths.min()) + 0.2 * float(depths.max() - depths.min())))
    same(splatad_b200.lidar_rasterization(**g))
    assert ops._depth_sort_mode.get(key, 1) == 1       # not taken for crowded depths
    # the frame above dropped the range; the next one reports it again
    assert key not in ops._depth_range_hint
    same(splatad_b200.lidar_rasterization(**g))
    assert ops._depth_range_hint[key] == (lo, hi)
    # a range far beyond the scene: all depths share a few buckets at the low end
    ops._depth_range_hint[key] = (bits(0.0), bits(1.0e6))
    same(splatad_b200.lidar_rasterization(**g))
    assert ops._depth_sort_mode.get(key, 1) == 1


def test_many_frames_over_eight_sensor_poses_reproduce_their_first_frame():
    """A sensor that changes its pose every frame (yaw 0, 45 .. 315 degrees in turn, as the benchmark
    does) goes through every fast path at once - hinted capacity, early count, carried depth range,
    pipelined projection: 800 frames later every pose still renders exactly what it rendered in a
    first frame, and no bulk copy ever ran into its wait limit."""
    import ctypes
    import math
    import splatad_b200
    from splatad_b200 import _lib, ops, scenes
    g = _to_gpu(scenes.config2(N=120_003))    # a shape of its own, with a ragged last slab
    poses = []
    for k in range(8):
        c, s_ = math.cos(math.radians(45.0 * k)), math.sin(math.radians(45.0 * k))
        vm = g["viewmats"].clone()
        vm[0, :3, :3] = torch.tensor([[c, s_, 0.0], [-s_, c, 0.0], [0.0, 0.0, 1.0]], device=vm.device)
        poses.append(vm)
    first = []
    for vm in poses:
        ops._isect_count_hint.clear()
        ops._depth_range_hint.clear()
        out = splatad_b200.lidar_rasterization(**dict(g, viewmats=vm))
        first.append((out[0].clone(), out[1].clone(), out[3]["flatten_ids"].clone(), out[3]["isect_offsets"].clone()))
    for i in range(800):
        out = splatad_b200.lidar_rasterization(**dict(g, viewmats=poses[i % 8]))
        if i % 37 == 0 or i >= 792:
            want = first[i % 8]
            assert torch.equal(out[0], want[0]) and torch.equal(out[1], want[1]), i
            assert torch.equal(out[3]["flatten_ids"], want[2]) and torch.equal(out[3]["isect_offsets"], want[3]), i
    torch.cuda.synchronize()
    count = ctypes.c_int64(-1)
    _lib.check(_lib.load().splatad_async_copy_timeouts(ctypes.addressof(count)))
    assert count.value == 0


def test_repeated_camera_frames():
    import splatad_b200
    from splatad_b200 import ops, scenes
    cfg = scenes.config1(N=30_000)
    g = _to_gpu(cfg)
    ops._isect_count_hint.clear()
    first = splatad_b200.rasterization(**g)
    second = splatad_b200.rasterization(**g)
    assert torch.equal(first[0], second[0]) and torch.equal(first[1], second[1])
    for key in ("isect_ids", "flatten_ids", "isect_offsets", "tiles_per_gauss"):
        assert torch.equal(first[2][key], second[2][key]), key


def test_repeated_packed_camera_frames_do_not_wait_for_the_row_count():
    """From the second frame of a shape on, a packed camera frame is enqueued on padded rows and cut
    to length before compositing; a frame whose rows outgrow the room is redone. Renders, meta and
    gradients must be those of the first (two-step) frame."""
    import splatad_b200
    from splatad_b200 import ops, scenes
    cfg = scenes.config1(N=200_001)         # a shape of its own: the first call is a first frame
    cfg.update(absgrad=True, rasterize_mode="antialiased")
    g = _to_gpu(cfg)
    leaves = ("means", "quats", "scales", "opacities", "colors")

    def frame(scale=1.0):
        kw = dict(g)
        for k in leaves:
            kw[k] = g[k].clone().requires_grad_(True)
        m_in = kw["means"]
        kw["means"] = m_in * torch.tensor([scale, scale, 1.0], device=DEV)
        colors, alphas, meta = splatad_b200.rasterization(**kw)
        meta["means2d"].retain_grad()
        (colors.square().mean() + alphas.mean()).backward()
        grads = {k: kw[k].grad if k != "means" else m_in.grad for k in leaves}
        return colors, alphas, meta, grads

    for key in [k for k in ops._packed_nnz_hint if k[:2] == (1, 200_001)]:
        del ops._packed_nnz_hint[key]
    first = frame()
    second = frame()                         # padded rows, cut to length
    nnz = first[2]["camera_ids"].numel()
    assert 100_000 < nnz < 200_001   # more rows than the 64 Ki granule of the room
    assert torch.equal(first[0], second[0]) and torch.equal(first[1], second[1])
    for key in ("camera_ids", "gaussian_ids", "radii", "means2d", "depths", "conics", "opacities", "pix_vels",
                "isect_ids", "flatten_ids", "isect_offsets", "tiles_per_gauss"):
        a, b = first[2][key], second[2][key]
        assert a.shape == b.shape and torch.equal(a, b), key
    for key in ("means2d",):
        assert second[2][key].grad is not None and second[2][key].absgrad is not None
        assert_close("packed d/d" + key, n(second[2][key].grad), n(first[2][key].grad), 1e-4, 1e-9)
        assert_close("packed absgrad", n(second[2][key].absgrad), n(first[2][key].absgrad), 1e-4, 1e-9)
    for k in leaves:
        ga, gb = n(first[3][k]), n(second[3][k])
        assert_close("packed d/d" + k, gb, ga, 1e-3, 1e-3 * float(np.sqrt((ga ** 2).mean())), max_bad_frac=1e-3)
    # a frame that sees far fewer Gaussians, then the full one again: the second outgrows its room
    few = frame(scale=40.0)
    assert few[2]["camera_ids"].numel() < nnz // 2
    third = frame()
    assert torch.equal(first[0], third[0])
    assert torch.equal(first[2]["flatten_ids"], third[2]["flatten_ids"])


def test_config2_full_size_properties():
    """The headline frame (1 M Gaussians, 15.3 M intersections) through properties that do not depend
    on size (the comparison with the CPU oracle at this size is ``test_gpu_full_size.py``) - and by
    building its tile lists twice,
    with the two independent implementations the library has (row / column split for small tile
    grids, radix split otherwise), which must agree bit for bit."""
    import splatad_b200
    from splatad_b200 import ops, scenes
    cfg = scenes.config2()
    g = _to_gpu(cfg)
    feats, alphas, asum, m = splatad_b200.lidar_rasterization(**g)
    ids, flat, tpg, offs = m["isect_ids"], m["flatten_ids"], m["tiles_per_gauss"], m["isect_offsets"]
    n_isects = ids.numel()
    assert n_isects > 15_000_000 and flat.numel() == n_isects
    # counts, order, offsets
    assert int(tpg.sum()) == n_isects
    assert bool((ids[1:] >= ids[:-1]).all()), "isect ids are not sorted"
    assert torch.equal(offs, ops.isect_offset_encode(ids.clone(), 1, m["tile_grid_width"], m["tile_grid_height"]))
    # every Gaussian appears once per tile it touches
    assert torch.equal(torch.bincount(flat.long(), minlength=tpg.numel()), tpg.reshape(-1).long())
    # depth bits of the ids are the Gaussians' depths; the tile of an id is the tile whose range holds it
    assert torch.equal((ids & 0xFFFFFFFF).to(torch.int32), m["depths"].reshape(-1)[flat.long()].view(torch.int32))
    tile_of = torch.bucketize(torch.arange(n_isects, device=DEV), offs.reshape(-1).long(), right=True) - 1
    assert torch.equal(ids >> 32, tile_of)
    # the same lists from the radix split: the packed layout with 64 (empty but one) sensors is
    # outside the row / column split's reach, and sensor 0 leaves the ids unchanged
    N = cfg["means"].shape[0]
    zeros = torch.zeros(N, dtype=torch.int64, device=DEV)
    _, ids2, flat2 = ops.isect_lidar_tiles(
        m["means2d"][0], m["radii"][0], m["depths"][0], g["tile_elevation_boundaries"],
        cfg["azimuth_resolution"] * cfg["tile_width"], cfg["min_azimuth"], packed=True, n_cameras=64,
        camera_ids=zeros, gaussian_ids=torch.arange(N, device=DEV))
    assert torch.equal(ids2, ids) and torch.equal(flat2, flat)
    # render: repeatable, alphas in range
    again = splatad_b200.lidar_rasterization(**g)
    assert torch.equal(again[0], feats) and torch.equal(again[1], alphas) and torch.equal(again[2], asum)
    assert float(alphas.min()) >= 0.0 and float(alphas.max()) <= 1.0 and bool(torch.isfinite(feats).all())


def _camera_lists_match_oracle(m, C, label):
    """Tile lists of a (packed) camera render against the oracle's isect on the same projection."""
    import math
    from oracle import isect
    tw, th = math.ceil(m["width"] / m["tile_size"]), math.ceil(m["height"] / m["tile_size"])
    cam_ids = n(m["camera_ids"]) if m["camera_ids"] is not None else None
    tpg, ids, flat = isect.isect_tiles(n(m["means2d"]), n(m["radii"]), n(m["depths"]), m["tile_size"], tw, th,
                                       n_cameras=C, camera_ids=cam_ids)
    assert np.array_equal(n(m["tiles_per_gauss"]), tpg), f"{label}: tile counts differ"
    assert np.array_equal(n(m["isect_ids"]), ids), f"{label}: isect ids differ"
    assert np.array_equal(n(m["flatten_ids"]), flat), f"{label}: sorted Gaussian id lists differ"
    assert np.array_equal(n(m["isect_offsets"]), isect.isect_offset_encode(ids, C, tw, th)), f"{label}: offsets"


def test_config3_six_cameras_and_lidar_reduced():
    """Config 3's rig (six 1920 x 1080 cameras yawed 60 degrees apart + the 128-beam lidar) on 20k
    Gaussians: 48960 camera tiles go through the radix split, the lidar through the row / column
    split; both against the oracle."""
    import splatad_b200
    from oracle import pipeline
    from splatad_b200 import scenes
    cfg = scenes.config3(N=20_000)
    cam, lid = cfg["camera"], cfg["lidar"]
    out_c, out_a, m = splatad_b200.rasterization(**_to_gpu(cam))
    assert out_c.shape == (6, 1080, 1920, 4)
    _camera_lists_match_oracle(m, 6, "config3 cameras")
    ref_c, ref_a, meta = pipeline.rasterization(**cam)
    ok = ~meta["ambiguous"][..., None]
    assert meta["ambiguous"].mean() < 0.01
    assert_close("config3 RGB+D", n(out_c), ref_c, 5e-4, 5e-4, mask=ok, max_bad_frac=2e-3)
    assert_close("config3 alpha", n(out_a), ref_a, 5e-4, 1e-4, mask=ok, max_bad_frac=2e-3)
    lo_c, lo_a, lo_s, lm = splatad_b200.lidar_rasterization(**_to_gpu(lid))
    ref = _lidar_stagewise_reference(lid, lm)
    _check_lists(lm, ref, "config3 lidar")
    _check_lidar_render("config3 lidar", lo_c, lo_a, lo_s, lm, ref)


def test_config4_training_step_reduced():
    """Config 4's rig (eight cameras, two lidars) on 20k Gaussians, forward + backward with fixed
    seeded cotangents: forward against the oracle, gradients of the packed and the [C, N] camera
    layouts (two different backward code paths) against each other, all parameters reached."""
    import splatad_b200
    from splatad_b200 import scenes
    cfg = scenes.config4(N=20_000)
    cam, lid = _to_gpu(cfg["camera"]), _to_gpu(cfg["lidar"])
    names = ("means", "quats", "scales", "opacities")
    g = torch.Generator().manual_seed(44)
    # two lidars
    leaves = {k: lid[k].clone().requires_grad_(True) for k in names + ("lidar_features",)}
    lo_c, lo_a, lo_s, lm = splatad_b200.lidar_rasterization(**dict(lid, **leaves))
    assert lo_c.shape == (2, 128, 1800, 17)
    ref = _lidar_stagewise_reference(cfg["lidar"], lm)
    _check_lists(lm, ref, "config4 lidars")
    _check_lidar_render("config4 lidars", lo_c, lo_a, lo_s, lm, ref)
    w_c = torch.randn(lo_c.shape, generator=g).to(DEV)
    w_a = torch.randn(lo_a.shape, generator=g).to(DEV)
    ((lo_c * w_c).sum() + (lo_a * w_a).sum()).backward()
    for k, v in leaves.items():
        assert v.grad is not None and bool(torch.isfinite(v.grad).all()) and float(v.grad.abs().sum()) > 0, k
    # eight cameras, packed and unpacked
    w_img = torch.randn(8, 1080, 1920, 4, generator=g).to(DEV)
    grads = {}
    for packed in (True, False):
        leaves = {k: cam[k].clone().requires_grad_(True) for k in names + ("colors",)}
        out_c, out_a, m = splatad_b200.rasterization(**dict(cam, packed=packed, **leaves))
        if packed:
            _camera_lists_match_oracle(m, 8, "config4 cameras")
        ((out_c * w_img).sum() + out_a.sum()).backward()
        grads[packed] = {k: v.grad.clone() for k, v in leaves.items()}
    for k in grads[True]:
        a, b = grads[True][k], grads[False][k]
        assert float(b.abs().sum()) > 0, k
        err = float((a - b).norm() / b.norm())
        assert err < 1e-4, f"config4 camera grad {k}: packed vs [C,N] relative L2 {err:.2e}"
