"""Bit-exact parity of tile intersection (tiles per Gaussian, sorted isect ids, flatten ids,
offsets) between the CUDA library and the CPU oracle / the reference's golden vectors."""

import math

import numpy as np
import pytest
import torch

from gpu_util import DEV, n, t

pytestmark = pytest.mark.gpu


def _check(got, want, label):
    for name, a, b in zip(("tiles_per_gauss", "isect_ids", "flatten_ids", "isect_offsets"), got, want):
        a = n(a)
        assert a.shape == b.shape, f"{label} {name}: shape {a.shape} vs {b.shape}"
        if not np.array_equal(a, b):
            bad = np.nonzero(a.reshape(-1) != b.reshape(-1))[0]
            raise AssertionError(f"{label} {name}: {bad.size} of {a.size} entries differ, first at {bad[0]}: "
                                 f"got {a.reshape(-1)[bad[0]]} want {b.reshape(-1)[bad[0]]}")


def _run_cam(means2d, radii, depths, ts, tw, th, **kw):
    from splatad_b200 import ops
    C = kw.get("n_cameras") or means2d.shape[0]
    tpg, ids, flat = ops.isect_tiles(t(means2d), t(radii, torch.int32), t(depths), ts, tw, th, **kw)
    offs = ops.isect_offset_encode(ids, C, tw, th)
    # the offsets handed over by the fill equal the ones recomputed from the ids alone
    assert torch.equal(offs, ops.isect_offset_encode(ids.clone(), C, tw, th))
    return tpg, ids, flat, offs


def _run_lidar(means2d, radii, depths, eb, res, min_az, **kw):
    from splatad_b200 import ops
    C = kw.get("n_cameras") or means2d.shape[0]
    tpg, ids, flat = ops.isect_lidar_tiles(t(means2d), t(radii), t(depths), t(eb), res, min_az, **kw)
    n_az = math.ceil(360 / res)
    offs = ops.isect_offset_encode(ids, C, n_az, len(eb) - 1)
    assert torch.equal(offs, ops.isect_offset_encode(ids.clone(), C, n_az, len(eb) - 1))
    return tpg, ids, flat, offs


def test_isect_tiles_golden(golden):
    g = golden("isect_tiles")
    got = _run_cam(g["means2d"], g["radii"], g["depths"], int(g["tile_size"]), int(g["tile_width"]), int(g["tile_height"]))
    _check(got, [g[k] for k in ("tiles_per_gauss", "isect_ids", "flatten_ids", "isect_offsets")], "golden camera")


@pytest.mark.parametrize("name", ["isect_lidar_tiles", "isect_lidar_tiles_wrap"])
def test_isect_lidar_tiles_golden(golden, name):
    g = golden(name)
    got = _run_lidar(g["means2d"], g["radii"], g["depths"], g["elev_boundaries"], float(g["tile_azim_resolution"]),
                     float(g["min_azimuth"]))
    _check(got, [g[k] for k in ("tiles_per_gauss", "isect_ids", "flatten_ids", "isect_offsets")], name)


@pytest.mark.parametrize("C,N,W,H,ts", [(1, 1, 64, 64, 16), (2, 5000, 640, 480, 16), (3, 70000, 1920, 1080, 16),
                                         (1, 3000, 100, 60, 7), (1, 6000, 1100, 200, 16), (2, 9000, 300, 250, 16)])
def test_isect_tiles_vs_oracle(C, N, W, H, ts):
    from oracle import isect
    g = torch.Generator().manual_seed(C * 1000 + N)
    means2d = (torch.rand(C, N, 2, generator=g) * 1.4 - 0.2) * torch.tensor([W, H])
    radii = torch.randint(0, 60, (C, N, 2), generator=g, dtype=torch.int32)
    radii[:, ::9, 0] = 0
    depths = torch.rand(C, N, generator=g) * 50
    depths[:, 1::4] = depths[:, 0::4][:, : depths[:, 1::4].shape[1]]  # equal depths: ties keep flatten order
    tw, th = math.ceil(W / ts), math.ceil(H / ts)
    want = list(isect.isect_tiles(n(means2d), n(radii), n(depths), ts, tw, th))
    want.append(isect.isect_offset_encode(want[1], C, tw, th))
    got = _run_cam(means2d, radii, depths, ts, tw, th)
    _check(got, want, f"camera C={C} N={N}")
    # unsorted variant: emission in flatten order
    from splatad_b200 import ops
    tpg, ids, flat = ops.isect_tiles(t(means2d), t(radii, torch.int32), t(depths), ts, tw, th, sort=False)
    w = isect.isect_tiles(n(means2d), n(radii), n(depths), ts, tw, th, sort=False)
    _check((tpg, ids, flat), w, f"camera unsorted C={C} N={N}")


def test_isect_tiles_packed():
    from oracle import isect
    C, N, W, H, ts = 3, 20000, 640, 480, 16
    g = torch.Generator().manual_seed(77)
    nnz = 30000
    cam = torch.sort(torch.randint(0, C, (nnz,), generator=g)).values
    gau = torch.randint(0, N, (nnz,), generator=g)
    means2d = (torch.rand(nnz, 2, generator=g) * 1.2 - 0.1) * torch.tensor([W, H])
    radii = torch.randint(1, 40, (nnz, 2), generator=g, dtype=torch.int32)
    depths = torch.rand(nnz, generator=g) * 50
    tw, th = math.ceil(W / ts), math.ceil(H / ts)
    want = list(isect.isect_tiles(n(means2d), n(radii), n(depths), ts, tw, th, n_cameras=C, camera_ids=n(cam)))
    want.append(isect.isect_offset_encode(want[1], C, tw, th))
    got = _run_cam(means2d, radii, depths, ts, tw, th, packed=True, n_cameras=C, camera_ids=cam.to(DEV),
                   gaussian_ids=gau.to(DEV))
    _check(got, want, "camera packed")


@pytest.mark.parametrize("C,N", [(1, 1), (1, 4000), (2, 60000)])
def test_isect_lidar_tiles_vs_oracle(C, N):
    from oracle import isect
    from splatad_b200 import scenes
    g = torch.Generator().manual_seed(C * 100 + N)
    elev = scenes.beams_128()
    eb = scenes.elevation_boundaries(elev, 8)
    means2d = torch.stack([torch.rand(C, N, generator=g) * 360 - 180, torch.rand(C, N, generator=g) * 44 - 27], -1)
    radii = torch.rand(C, N, 2, generator=g) * torch.tensor([12.0, 4.0])
    radii[:, ::50, 0] = 200.0 + torch.rand(C, len(range(0, N, 50)), generator=g) * 300  # more than a full turn
    radii[:, ::11, 0] = 0
    depths = torch.rand(C, N, generator=g) * 80
    depths[:, 1::4] = depths[:, 0::4][:, : depths[:, 1::4].shape[1]]
    res = 0.2 * 32
    want = list(isect.isect_lidar_tiles(n(means2d), n(radii), n(depths), n(eb), res, -180.0))
    n_az = math.ceil(360 / res)
    want.append(isect.isect_offset_encode(want[1], C, n_az, len(eb) - 1))
    got = _run_lidar(means2d, radii, depths, eb, res, -180.0)
    _check(got, want, f"lidar C={C} N={N}")


def test_isect_empty_and_invisible():
    from splatad_b200 import ops
    z2 = torch.zeros(2, 0, 2, device=DEV)
    tpg, ids, flat = ops.isect_tiles(z2, z2.int(), torch.zeros(2, 0, device=DEV), 16, 4, 4)
    assert tpg.shape == (2, 0) and ids.numel() == 0 and flat.numel() == 0
    offs = ops.isect_offset_encode(ids, 2, 4, 4)
    assert offs.shape == (2, 4, 4) and int(offs.abs().sum()) == 0
    # all Gaussians culled
    m = torch.rand(1, 100, 2, device=DEV) * 64
    tpg, ids, flat = ops.isect_tiles(m, torch.zeros(1, 100, 2, dtype=torch.int32, device=DEV),
                                     torch.rand(1, 100, device=DEV), 16, 4, 4)
    assert int(tpg.sum()) == 0 and ids.numel() == 0


def test_isect_key_bits_error():
    from splatad_b200 import ops
    m = torch.rand(1, 10, 2, device=DEV)
    with pytest.raises(RuntimeError):
        ops.isect_tiles(m, torch.ones(1, 10, 2, dtype=torch.int32, device=DEV), torch.rand(1, 10, device=DEV),
                        1, 1 << 16, 1 << 16)


def test_two_deferred_intersections_outstanding():
    """Two deferred tile intersections alive at once - a camera call and a lidar call of different
    sizes, resolved in the opposite order: each reads ITS count (own pinned slot), so lengths, lists
    and offsets equal those of the two-step calls. A second pair runs on another stream, which has
    workspaces and capacity hints of its own."""
    from splatad_b200 import ops, scenes
    g = torch.Generator().manual_seed(5)
    C, N, W, H, ts = 2, 30_000, 640, 480, 16
    means2d = ((torch.rand(C, N, 2, generator=g) * 1.2 - 0.1) * torch.tensor([W, H])).to(DEV)
    radii = torch.randint(1, 40, (C, N, 2), generator=g, dtype=torch.int32).to(DEV)
    depths = (torch.rand(C, N, generator=g) * 50).to(DEV)
    tw, th = math.ceil(W / ts), math.ceil(H / ts)
    eb = scenes.elevation_boundaries(scenes.beams_128(), 8).to(DEV)
    M = 50_000
    l_means = torch.stack([torch.rand(1, M, generator=g) * 360 - 180, torch.rand(1, M, generator=g) * 44 - 27], -1).to(DEV)
    l_radii = (torch.rand(1, M, 2, generator=g) * torch.tensor([12.0, 4.0])).to(DEV)
    l_depths = (torch.rand(1, M, generator=g) * 80).to(DEV)
    res, n_az = 0.2 * 32, math.ceil(360 / (0.2 * 32))

    def cam():
        return ops.isect_tiles_deferred(means2d, radii, depths, ts, tw, th)

    def lid():
        return ops.isect_lidar_tiles_deferred(l_means, l_radii, l_depths, eb, res, -180.0)

    want_cam = ops.isect_tiles(means2d, radii, depths, ts, tw, th)
    want_lid = ops.isect_lidar_tiles(l_means, l_radii, l_depths, eb, res, -180.0)
    assert want_cam[1].numel() != want_lid[1].numel()

    def check_pair():
        cam().resolve(), lid().resolve()          # first frames of the two shapes: they leave the hints
        d_cam, d_lid = cam(), lid()               # both enqueued ahead of their counts, both outstanding
        assert d_cam._resolved is None and d_lid._resolved is None
        offs_lid, offs_cam = d_lid.offsets(16, n_az).clone(), d_cam.offsets(th, tw).clone()
        ids_l, flat_l = d_lid.resolve()           # opposite order
        ids_c, flat_c = d_cam.resolve()
        assert torch.equal(ids_c, want_cam[1]) and torch.equal(flat_c, want_cam[2])
        assert torch.equal(ids_l, want_lid[1]) and torch.equal(flat_l, want_lid[2])
        assert torch.equal(offs_cam, ops.isect_offset_encode(want_cam[1].clone(), C, tw, th))
        assert torch.equal(offs_lid, ops.isect_offset_encode(want_lid[1].clone(), 1, n_az, 16))
        assert torch.equal(d_cam.tiles_per_gauss, want_cam[0]) and torch.equal(d_lid.tiles_per_gauss, want_lid[0])

    check_pair()
    side = torch.cuda.Stream(DEV)
    side.wait_stream(torch.cuda.current_stream(DEV))
    with torch.cuda.stream(side):
        check_pair()
    side.synchronize()


@pytest.mark.parametrize("distinct", [1, 7, 150, 3000])
def test_depth_order_with_crowded_depths(distinct):
    """Depth order of the visible Gaussians when many depths coincide: with `distinct` different
    depths among 40,000 Gaussians a depth bucket holds from a dozen elements (ranked by counting) over
    a few hundred (bitonic network in shared memory) to thousands (beyond what the bucket sort
    orders: the plan says so and the lists come from the radix passes). All give the reference's
    order - ties by flatten index - bit for bit, for the two-step call, for a second, hinted frame of
    the same shape, and for the camera path."""
    from oracle import isect
    from splatad_b200 import ops, scenes
    C, N = 2, 20_000
    g = torch.Generator().manual_seed(100 + distinct)
    eb = scenes.elevation_boundaries(scenes.beams_128(), 8)
    means2d = torch.stack([torch.rand(C, N, generator=g) * 360 - 180, torch.rand(C, N, generator=g) * 44 - 27], -1)
    radii = torch.rand(C, N, 2, generator=g) * torch.tensor([9.0, 3.0])
    radii[:, ::13, 0] = 0
    levels = torch.rand(distinct, generator=g) * 80 + 0.5
    depths = levels[torch.randint(0, distinct, (C, N), generator=g)]
    res, n_az = 0.2 * 32, math.ceil(360 / (0.2 * 32))
    want = list(isect.isect_lidar_tiles(n(means2d), n(radii), n(depths), n(eb), res, -180.0))
    want.append(isect.isect_offset_encode(want[1], C, n_az, len(eb) - 1))
    ops._depth_sort_mode.clear()
    _check(_run_lidar(means2d, radii, depths, eb, res, -180.0), want, f"lidar, {distinct} depths")
    for _ in range(2):   # first deferred call leaves the hint, the second is enqueued ahead of its count
        d = ops.isect_lidar_tiles_deferred(t(means2d), t(radii), t(depths), t(eb), res, -180.0)
        got = d.resolve()
        if got is None:
            d = d.redo()
            got = d.resolve()
        _check((d.tiles_per_gauss, got[0], got[1]), want[:3], f"lidar deferred, {distinct} depths")
    crowded = 2 * N * 12 // 13 / distinct > 1024
    assert (2 in ops._depth_sort_mode.values()) == crowded
    # camera rectangles (one 640 x 480 camera: the row / column split; packed: three cameras)
    W, H, ts = 640, 480, 16
    m2 = (torch.rand(1, N, 2, generator=g) * 1.2 - 0.1) * torch.tensor([W, H])
    r2 = torch.randint(0, 40, (1, N, 2), generator=g, dtype=torch.int32)
    d2 = depths[:1]
    tw, th = math.ceil(W / ts), math.ceil(H / ts)
    want = list(isect.isect_tiles(n(m2), n(r2), n(d2), ts, tw, th))
    want.append(isect.isect_offset_encode(want[1], 1, tw, th))
    _check(_run_cam(m2, r2, d2, ts, tw, th), want, f"camera, {distinct} depths")


@pytest.mark.parametrize("lo,hi", [(0.0, 80.0), (10.0, 30.0), (0.0, 1.0e7), (79.0, 200.0)])
def test_depth_range_hint_never_changes_the_lists(lo, hi):
    """`splatad_isect_set_depth_range_hint` makes the depth buckets of the next plan span the given
    range instead of the measured one (and lets the rectangle count fill them): a range that fits, one
    that covers a slice of the depths, one far too wide and one that starts where the depths end all
    give the oracle's lists bit for bit - or, when an end bucket overflows, the status bit that sends
    the caller back to a plan without a hint."""
    import struct
    from oracle import isect
    from splatad_b200 import _lib, ops, scenes
    bits = lambda v: struct.unpack("<I", struct.pack("<f", v))[0]   # noqa: E731
    C, N = 1, 30_000
    g = torch.Generator().manual_seed(7)
    eb = scenes.elevation_boundaries(scenes.beams_128(), 8)
    means2d = torch.stack([torch.rand(C, N, generator=g) * 360 - 180, torch.rand(C, N, generator=g) * 44 - 27], -1)
    radii = torch.rand(C, N, 2, generator=g) * torch.tensor([9.0, 3.0])
    radii[:, ::7, 0] = 0
    depths = torch.rand(C, N, generator=g) * 80
    res, n_az = 0.2 * 32, math.ceil(360 / (0.2 * 32))
    want = list(isect.isect_lidar_tiles(n(means2d), n(radii), n(depths), n(eb), res, -180.0))
    want.append(isect.isect_offset_encode(want[1], C, n_az, len(eb) - 1))
    ops._depth_sort_mode.clear()
    _lib.load().splatad_isect_set_depth_range_hint(bits(lo), bits(hi))
    got = _run_lidar(means2d, radii, depths, eb, res, -180.0)   # an overflowing end bucket makes ops repeat the plan
    _check(got, want, f"lidar, depth range hint [{lo}, {hi}]")
    # a hint is consumed by one plan: the next call measures its own range again
    _check(_run_lidar(means2d, radii, depths, eb, res, -180.0), want, "lidar, after the hint")
    ops._depth_sort_mode.clear()   # an overflow above made this shape take the radix passes: not for other tests
