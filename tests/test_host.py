"""CPU-only checks of the host side: the C-ABI library loads and exports every declared symbol,
the Python ops refuse CPU tensors (no fallback), scene generators and sharding helpers."""

import ctypes
import os

import pytest
import torch


def test_header_symbols_are_exported():
    from splatad_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        _lib.build()
    decls = _lib.parse_header()
    assert len(decls) >= 24
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in decls:
        assert hasattr(lib, name), f"{name} is declared in include/splatad_b200.h but not exported"
    loaded = _lib.load()
    assert loaded.splatad_version() == 100
    # workspace queries are pure host functions
    assert loaded.splatad_isect_plan_workspace_bytes(1000) > 4 * 4 * 1000
    assert loaded.splatad_isect_fill_workspace_bytes(1000) >= 4 * 4 * 1000


def test_error_mapping():
    from splatad_b200 import _lib
    lib = _lib.load()
    # null output pointer is rejected before any CUDA call
    rc = lib.splatad_isect_offset_encode(None, 0, 1, 4, 4, None, None)
    assert rc == _lib.ERR_BAD_ARG
    with pytest.raises(ValueError):
        _lib.check(rc)
    assert "isect_offset_encode" in _lib.last_error()
    rc = lib.splatad_rasterize_to_pixels_fwd(1, 0, None, None, None, 100, None, None, None, None, 8, 8, 16, 1, 1,
                                             None, None, None, None, None, None)
    assert rc == _lib.ERR_CHANNELS


def test_projection_entries_refuse_null_sensor_motion():
    """Every projection entry point that reads the sensors' motion refuses NULL for it with
    SPLATAD_ERR_BAD_ARG before anything is launched (a C caller may pass NULL for ``velocities``, not
    for these)."""
    from splatad_b200 import _lib
    lib = _lib.load()
    x = ctypes.c_void_p(256)   # never dereferenced: the argument check comes first
    geom = (x, None, x, x, None, x, x, 640, 480)            # means, covars, quats, scales, velocities, viewmats, Ks, w, h
    for missing in range(3):
        motion = [x, x, x]
        motion[missing] = None
        tail = (*motion, 0.3, 0.01, 1e10, 0.0)
        assert lib.splatad_projection_packed_count(1, 8, *geom, *tail, x, 1 << 20, x, x, None) == _lib.ERR_BAD_ARG
        assert "projection_packed_count" in _lib.last_error()
        assert lib.splatad_projection_packed_fill(1, 8, *geom, *tail, x, -1, x, x, x, x, x, x, None, x,
                                                  None) == _lib.ERR_BAD_ARG
        assert lib.splatad_projection_packed_bwd(1, 8, 4, *geom, *motion, 0.3, x, x, x, None, x, x, x, None, x, 0,
                                                 x, None, x, x, None, None, None) == _lib.ERR_BAD_ARG
        assert lib.splatad_projection_bwd(1, 8, *geom, *motion, 0.3, x, x, None, x, x, x, None, x, x, None, x, x,
                                          None, None, None) == _lib.ERR_BAD_ARG
        assert lib.splatad_lidar_projection_bwd(1, 8, x, None, x, x, None, x, *motion, 0.017, x, x, None, x, x, x,
                                                None, x, x, x, None, x, x, None, None, None) == _lib.ERR_BAD_ARG


def test_arguments_from_two_devices_are_refused_before_any_launch():
    """The call wrapper makes the tensors' GPU current for the launch and raises when the arguments of
    one call come from different GPUs (no GPU needed: the check is on the recorded device indices)."""
    from splatad_b200 import _lib
    a, b = _lib.DevPtr(256, 0), _lib.DevPtr(512, 1)
    with pytest.raises(ValueError, match="cuda:0 and cuda:1"):
        _lib.call("splatad_sh_fwd", 1, 1, 0, a, b, None, a, _lib.DevPtr(0, 0))


def test_ops_refuse_cpu_tensors():
    import splatad_b200
    N = 8
    with pytest.raises(RuntimeError, match="CUDA"):
        splatad_b200.fully_fused_lidar_projection(
            torch.rand(N, 3), None, torch.rand(N, 4), torch.rand(N, 3), None, torch.eye(4)[None],
            torch.zeros(1, 3), torch.zeros(1, 3), torch.zeros(1))


def test_api_signatures_match_reference_names():
    import inspect

    import splatad_b200
    sig = inspect.signature(splatad_b200.lidar_rasterization)
    assert list(sig.parameters)[:9] == ["means", "quats", "scales", "opacities", "lidar_features", "velocities",
                                        "viewmats", "raster_pts", "tile_elevation_boundaries"]
    assert sig.parameters["eps2d"].default == 0.017 and sig.parameters["tile_width"].default == 32
    sig = inspect.signature(splatad_b200.rasterization)
    assert list(sig.parameters)[:10] == ["means", "quats", "scales", "opacities", "colors", "velocities",
                                         "viewmats", "Ks", "width", "height"]
    assert sig.parameters["packed"].default is True and sig.parameters["eps2d"].default == 0.3


def test_scene_generators_are_seeded_and_shaped():
    from splatad_b200 import scenes
    a, b = scenes.config0(), scenes.config0()
    assert torch.equal(a["means"], b["means"]) and torch.equal(a["raster_pts"], b["raster_pts"])
    assert a["raster_pts"].shape == (1, 32, 512, 4) and a["lidar_features"].shape == (1, 20000, 4)
    assert a["tile_elevation_boundaries"].shape == (5,)
    e = scenes.beams_128()
    assert e.numel() == 128 and float(e[0]) == -25.0 and abs(float(e[-1]) - 15.0) < 1e-5
    assert abs(float(e[60] - e[59]) - 0.1) < 1e-4
    c2 = scenes.config2(N=1000)
    assert c2["raster_pts"].shape == (1, 128, 1800, 4) and c2["tile_elevation_boundaries"].shape == (17,)
    assert float(c2["raster_pts"][0, 0, 0, 3]) == pytest.approx(-0.05) and c2["azimuth_resolution"] == pytest.approx(0.2)
    c1 = scenes.config1(N=1000)
    assert c1["colors"].shape == (1000, 16, 3) and c1["width"] == 1920
    moving = (c1["velocities"].abs().sum(-1) > 0).float().mean()
    assert 0.05 < float(moving) < 0.16
    vm = scenes.yawed_camera_viewmats([0, 60, 120])
    for R in vm[:, :3, :3]:
        assert torch.allclose(R @ R.T, torch.eye(3), atol=1e-6) and float(torch.det(R)) == pytest.approx(1.0)


def test_wait_for_count_polls_the_early_triple_and_falls_back_to_the_event():
    """The host side of the early intersection count: the triple {count, sequence, status} that a
    kernel stores into slot[4:7] is taken as soon as the sequence number matches; a stale sequence
    number (the kernel never wrote) ends in the plan's own counters after the event."""
    from splatad_b200 import _lib

    class Event:
        def __init__(self):
            self.waited = 0

        def synchronize(self):
            self.waited += 1

    slot = torch.zeros(8, dtype=torch.int64)
    slot[0], slot[2] = 111, 1            # what the plan copies at its end
    slot[4], slot[5], slot[6] = 222, 7, 4
    ev = Event()
    assert _lib.wait_for_count(slot, 7, ev) == (222, 4) and ev.waited == 0
    assert _lib.wait_for_count(slot, 8, ev, patience_s=0.01) == (111, 1) and ev.waited == 1
    assert _lib.wait_for_count(slot, 0, ev) == (111, 1) and ev.waited == 2     # no early request armed
    a, b = _lib.next_sequence(), _lib.next_sequence()
    assert b == a + 1 and a > 0


def test_early_depth_range_is_read_only_with_a_matching_sequence():
    """slot[7] holds dmin bits | dmax bits << 32 of the frame's listed depths, valid once slot[5]
    carries the frame's sequence number; 0 means the reporting kernel did not know the range."""
    from splatad_b200 import _lib
    slot = torch.zeros(8, dtype=torch.int64)
    lo, hi = 0x3E99999A, 0x42E20000                    # 0.3 and 113.0 as float bit patterns
    slot[5], slot[7] = 9, lo | (hi << 32)
    assert _lib.early_depth_range(slot, 9) == (lo, hi)
    assert _lib.early_depth_range(slot, 10) is None    # another frame's words
    assert _lib.early_depth_range(slot, 0) is None     # nothing was armed
    slot[7] = 0
    assert _lib.early_depth_range(slot, 9) is None


def test_gradient_accumulators_share_one_zeroed_buffer():
    """The backward passes take all their zero-initialised accumulators as views of one buffer: the
    shapes are those asked for, None stays None, every view starts a multiple of 256 bytes behind the
    buffer's start (itself 512-byte aligned when it comes from the CUDA allocator) and the views do
    not overlap."""
    from splatad_b200 import ops
    a, b, c = torch.empty(5, 2), torch.empty(7), torch.empty(0, 3)
    va, none, vb, vc = ops._zeros_like_many(a, None, b, c)
    assert none is None and va.shape == a.shape and vb.shape == b.shape and vc.shape == c.shape
    assert float(va.abs().sum() + vb.abs().sum()) == 0.0
    assert (vb.data_ptr() - va.data_ptr()) % 256 == 0     # (an empty view may report no address at all)
    va.fill_(1.0)
    assert float(vb.abs().sum()) == 0.0 and vb.data_ptr() >= va.data_ptr() + va.numel() * 4
    assert ops._zeros_like_many(None, None) == [None, None]
