"""Parity of the compositing kernels (rasterize_to_pixels / rasterize_to_points, forward and
backward, through the C ABI) against the C oracle.

Forward tolerance: 1e-4 relative + 1e-5 absolute on every pixel whose threshold decisions are
not within 2e-5 (relative) of flipping; the oracle flags those (a different but equally valid
floating-point evaluation order may include or exclude one more Gaussian there) and their
fraction is asserted to be small. Ranges (depth) are also checked to 1 mm.
Backward tolerance: 1e-3 relative against the float64 oracle.
"""

import math

import numpy as np
import pytest
import torch

from gpu_util import DEV, assert_close, n, rel_l2, t

pytestmark = pytest.mark.gpu


def _camera_case(C, N, W, H, ts, channels, seed, rs_time=0.03, sigma_px=(2.0, 14.0)):
    from oracle import isect
    g = torch.Generator().manual_seed(seed)
    means2d = (torch.rand(C, N, 2, generator=g) * 1.1 - 0.05) * torch.tensor([W, H])
    sig = torch.rand(C, N, 2, generator=g) * (sigma_px[1] - sigma_px[0]) + sigma_px[0]
    rho = torch.rand(C, N, generator=g) * 1.2 - 0.6
    cov = torch.stack([sig[..., 0] ** 2, rho * sig[..., 0] * sig[..., 1], rho * sig[..., 0] * sig[..., 1],
                       sig[..., 1] ** 2], -1).reshape(C, N, 2, 2)
    inv = torch.linalg.inv(cov)
    conics = torch.stack([inv[..., 0, 0], inv[..., 0, 1], inv[..., 1, 1]], -1).contiguous()
    opac = torch.rand(C, N, generator=g) * 0.95 + 0.04
    opac[:, ::13] = 1.0  # exercises the 0.999 cap
    colors = torch.randn(C, N, channels, generator=g)
    pix_vels = torch.randn(C, N, 2, generator=g) * 40
    depths = torch.rand(C, N, generator=g) * 50 + 0.5
    rs = torch.full((C,), rs_time)
    radii = (3 * sig + pix_vels.abs() * 0.5 * rs_time).to(torch.int32)
    tw, th = math.ceil(W / ts), math.ceil(H / ts)
    _, ids, flat = isect.isect_tiles(n(means2d), n(radii), n(depths), ts, tw, th)
    offs = isect.isect_offset_encode(ids, C, tw, th)
    return dict(means2d=means2d, conics=conics, colors=colors, opacities=opac, pix_vels=pix_vels, rs=rs,
                offsets=offs, flatten_ids=flat, W=W, H=H, ts=ts)


def _check_fwd(label, got_c, got_a, ref, depth_channel=None):
    amb = ref["ambiguous"]
    frac = amb.mean()
    assert frac < 0.02, f"{label}: {frac:.3%} of the pixels are within tolerance of a threshold"
    ok = ~amb
    assert_close(label + " colors", got_c, ref["render_colors"], 1e-4, 1e-5, mask=ok[..., None])
    assert_close(label + " alphas", got_a, ref["render_alphas"], 1e-4, 1e-5, mask=ok[..., None])
    if depth_channel is not None:
        d = np.abs(got_c[..., depth_channel] - ref["render_colors"][..., depth_channel])[ok]
        lim = 1e-3 + 1e-4 * np.abs(ref["render_colors"][..., depth_channel])[ok]
        assert (d <= lim).all(), f"{label}: range off by {d.max()} m"


@pytest.mark.parametrize("channels", [1, 3, 4, 5, 17, 32])
@pytest.mark.parametrize("with_bg", [False, True])
def test_rasterize_to_pixels_fwd(channels, with_bg):
    from oracle import composite
    from splatad_b200 import ops
    c = _camera_case(2, 3000, 200, 136, 16, channels, 100 + channels)
    bg = torch.rand(2, channels) if with_bg else None
    ref = composite.rasterize_to_pixels_fwd(n(c["means2d"]), n(c["conics"]), n(c["colors"]), n(c["opacities"]),
                                            n(c["pix_vels"]), n(c["rs"]), n(bg), c["W"], c["H"], c["ts"],
                                            c["offsets"], c["flatten_ids"])
    out_c, out_a = ops.rasterize_to_pixels(t(c["means2d"]), t(c["conics"]), t(c["colors"]), t(c["opacities"]),
                                           t(c["pix_vels"]), c["W"], c["H"], c["ts"],
                                           t(c["offsets"], torch.int32), t(c["flatten_ids"], torch.int32),
                                           t(c["rs"]), backgrounds=t(bg))
    assert ref["contributing"] > 10 * c["W"] * c["H"]
    _check_fwd(f"pixels ch={channels} bg={with_bg}", n(out_c), n(out_a), ref)


def test_rasterize_to_pixels_many_channels_and_odd_tile():
    """> 32 channels are rendered in chunks; tile sizes whose square is not a warp multiple work."""
    from oracle import composite
    from splatad_b200 import ops
    c = _camera_case(1, 800, 70, 50, 6, 40, 7)
    ref = composite.rasterize_to_pixels_fwd(n(c["means2d"]), n(c["conics"]), n(c["colors"]), n(c["opacities"]),
                                            n(c["pix_vels"]), n(c["rs"]), None, c["W"], c["H"], c["ts"],
                                            c["offsets"], c["flatten_ids"])
    out_c, out_a = ops.rasterize_to_pixels(t(c["means2d"]), t(c["conics"]), t(c["colors"]), t(c["opacities"]),
                                           t(c["pix_vels"]), c["W"], c["H"], c["ts"],
                                           t(c["offsets"], torch.int32), t(c["flatten_ids"], torch.int32), t(c["rs"]))
    _check_fwd("pixels 40 channels tile 6", n(out_c), n(out_a), ref)


@pytest.mark.parametrize("channels", [3, 20])
def test_rasterize_to_pixels_largest_tile(channels):
    """32 x 32 tiles are blocks of 1024 threads: the forward kernels run at any channel count, the
    backward kernels while their registers allow it and say so otherwise."""
    from oracle import composite
    from splatad_b200 import ops
    c = _camera_case(1, 1500, 100, 70, 32, channels, 70 + channels)
    ref = composite.rasterize_to_pixels_fwd(n(c["means2d"]), n(c["conics"]), n(c["colors"]), n(c["opacities"]),
                                            n(c["pix_vels"]), n(c["rs"]), None, c["W"], c["H"], c["ts"],
                                            c["offsets"], c["flatten_ids"])
    leaves = {k: t(c[k]).requires_grad_(True) for k in ("means2d", "conics", "colors", "opacities", "pix_vels")}
    out_c, out_a = ops.rasterize_to_pixels(leaves["means2d"], leaves["conics"], leaves["colors"], leaves["opacities"],
                                           leaves["pix_vels"], c["W"], c["H"], c["ts"],
                                           t(c["offsets"], torch.int32), t(c["flatten_ids"], torch.int32), t(c["rs"]))
    _check_fwd(f"pixels tile 32 ch={channels}", n(out_c), n(out_a), ref)
    loss = out_c.sum() + out_a.sum()
    if channels == 3:
        loss.backward()
        assert float(leaves["colors"].grad.abs().sum()) > 0
    else:
        with pytest.raises(ValueError, match="1024 threads"):
            loss.backward()


def _grad_check(label, got, want, rel=1e-3):
    got, want = n(got).astype(np.float64), np.asarray(want, dtype=np.float64)
    rms = float(np.sqrt(np.mean(want ** 2)))
    e = rel_l2(got, want)
    assert e < rel, f"{label}: relative L2 error {e:.3e}"
    assert_close(label, got, want, rel, 2 * rel * rms, max_bad_frac=2e-3)


@pytest.mark.parametrize("channels,with_bg,absgrad", [(3, False, True), (4, True, False), (17, False, False)])
def test_rasterize_to_pixels_bwd(channels, with_bg, absgrad):
    from oracle import composite
    from splatad_b200 import ops
    c = _camera_case(2, 2000, 160, 120, 16, channels, 200 + channels)
    bg = torch.rand(2, channels) if with_bg else None
    g = torch.Generator().manual_seed(3)
    v_c = torch.randn(2, c["H"], c["W"], channels, generator=g)
    v_a = torch.randn(2, c["H"], c["W"], 1, generator=g)
    leaves = {k: t(c[k]).requires_grad_(True) for k in ("means2d", "conics", "colors", "opacities", "pix_vels")}
    bg_g = t(bg).requires_grad_(True) if with_bg else None
    ref_f = composite.rasterize_to_pixels_fwd(n(c["means2d"]), n(c["conics"]), n(c["colors"]), n(c["opacities"]),
                                              n(c["pix_vels"]), n(c["rs"]), n(bg), c["W"], c["H"], c["ts"],
                                              c["offsets"], c["flatten_ids"], dtype=np.float64)
    # only pixels whose include/exclude decisions are unambiguous take part in the comparison
    f32 = composite.rasterize_to_pixels_fwd(n(c["means2d"]), n(c["conics"]), n(c["colors"]), n(c["opacities"]),
                                            n(c["pix_vels"]), n(c["rs"]), n(bg), c["W"], c["H"], c["ts"],
                                            c["offsets"], c["flatten_ids"], amb_tol=1e-4)
    same = (f32["last_ids"] == ref_f["last_ids"]) & ~f32["ambiguous"]
    assert same.mean() > 0.97
    mask = t(same[..., None].astype(np.float32))
    out_c, out_a = ops.rasterize_to_pixels(leaves["means2d"], leaves["conics"], leaves["colors"],
                                           leaves["opacities"], leaves["pix_vels"], c["W"], c["H"], c["ts"],
                                           t(c["offsets"], torch.int32), t(c["flatten_ids"], torch.int32),
                                           t(c["rs"]), backgrounds=bg_g, absgrad=absgrad)
    ((out_c * t(v_c) * mask).sum() + (out_a * t(v_a) * mask).sum()).backward()
    mk = same[..., None].astype(np.float64)
    ref = composite.rasterize_to_pixels_bwd(n(c["means2d"]), n(c["conics"]), n(c["colors"]), n(c["opacities"]),
                                            n(c["pix_vels"]), n(c["rs"]), n(bg), c["W"], c["H"], c["ts"],
                                            c["offsets"], c["flatten_ids"], ref_f["render_alphas"],
                                            ref_f["last_ids"], n(v_c) * mk, n(v_a) * mk, absgrad=absgrad)
    _grad_check("pixels v_means2d", leaves["means2d"].grad, ref["v_means2d"])
    _grad_check("pixels v_conics", leaves["conics"].grad, ref["v_conics"])
    _grad_check("pixels v_colors", leaves["colors"].grad, ref["v_colors"])
    _grad_check("pixels v_opacities", leaves["opacities"].grad, ref["v_opacities"])
    _grad_check("pixels v_pix_vels", leaves["pix_vels"].grad, ref["v_pix_vels"])
    if absgrad:
        _grad_check("pixels absgrad", leaves["means2d"].absgrad, ref["v_means2d_abs"])
    if with_bg:
        want_bg = (n(v_c) * mk * (1.0 - ref_f["render_alphas"])).sum(axis=(1, 2))
        _grad_check("pixels v_backgrounds", bg_g.grad, want_bg)


def _lidar_case(C, N, H, W, tw, th, channels, seed, sweep=0.1):
    from oracle import isect
    from splatad_b200 import scenes
    g = torch.Generator().manual_seed(seed)
    elev = torch.linspace(-20.0, 12.0, H)
    az_res = 360.0 / W
    pts = torch.cat([scenes.lidar_sensor(elev, W, g, sweep_time=sweep) for _ in range(C)], 0)
    pts[..., :2] += torch.randn(C, H, W, 2, generator=g) * 0.01
    pts[..., 2] = pts[..., 2] * (torch.rand(C, H, W, generator=g) > 0.1)  # ~10 % of the points have no return
    means2d = torch.stack([torch.rand(C, N, generator=g) * 360 - 180, torch.rand(C, N, generator=g) * 36 - 22], -1)
    sig = torch.rand(C, N, 2, generator=g) * torch.tensor([4.0, 2.0]) + torch.tensor([0.5, 0.3])
    rho = torch.rand(C, N, generator=g) * 1.2 - 0.6
    cov = torch.stack([sig[..., 0] ** 2, rho * sig[..., 0] * sig[..., 1], rho * sig[..., 0] * sig[..., 1],
                       sig[..., 1] ** 2], -1).reshape(C, N, 2, 2)
    inv = torch.linalg.inv(cov)
    conics = torch.stack([inv[..., 0, 0], inv[..., 0, 1], inv[..., 1, 1]], -1).contiguous()
    opac = torch.rand(C, N, generator=g) * 0.95 + 0.04
    opac[:, ::13] = 1.0
    depths = torch.rand(C, N, generator=g) * 80 + 1
    feats = torch.randn(C, N, channels, generator=g)
    feats[..., -1] = depths
    pix_vels = torch.randn(C, N, 3, generator=g) * torch.tensor([20.0, 5.0, 3.0])
    dcomp = torch.randn(C, N, 2, generator=g) * 0.05
    radii = 3 * sig + pix_vels[..., :2].abs() * 0.5 * sweep
    eb = scenes.elevation_boundaries(elev, th)
    res = az_res * tw
    _, ids, flat = isect.isect_lidar_tiles(n(means2d), n(radii), n(depths), n(eb), res, -180.0)
    n_az = math.ceil(360 / res)
    offs = isect.isect_offset_encode(ids, C, n_az, len(eb) - 1)
    return dict(means2d=means2d, conics=conics, feats=feats, opacities=opac, pix_vels=pix_vels, dcomp=dcomp,
                pts=pts, offsets=offs, flatten_ids=flat, W=W, H=H, tw=tw, th=th)


@pytest.mark.parametrize("channels", [2, 5, 17, 32])
@pytest.mark.parametrize("asum", [False, True])
def test_rasterize_to_points_fwd(channels, asum):
    from oracle import composite
    from splatad_b200 import ops
    c = _lidar_case(2, 4000, 32, 512, 32, 8, channels, 300 + channels)
    ref = composite.rasterize_to_points_fwd(n(c["means2d"]), n(c["conics"]), n(c["feats"]), n(c["opacities"]),
                                            n(c["pix_vels"]), n(c["dcomp"]), None, n(c["pts"]), c["W"], c["H"],
                                            c["tw"], c["th"], c["offsets"], c["flatten_ids"], asum, 0.5)
    out_c, out_a, out_s, out_m = ops.rasterize_to_points(
        t(c["means2d"]), t(c["conics"]), t(c["feats"]), t(c["opacities"]), t(c["pix_vels"]), t(c["dcomp"]),
        t(c["pts"]), c["W"], c["H"], c["tw"], c["th"], t(c["offsets"], torch.int32),
        t(c["flatten_ids"], torch.int32), asum, 0.5)
    assert ref["contributing"] > 5 * c["W"] * c["H"]
    label = f"points ch={channels} asum={asum}"
    _check_fwd(label, n(out_c), n(out_a), ref, depth_channel=channels - 1)
    ok = ~ref["ambiguous"][..., None]
    assert_close(label + " median", n(out_m), ref["median_depths"], 1e-4, 1e-3, mask=ok)
    if asum:
        assert_close(label + " alpha_sum", n(out_s), ref["alpha_sum"], 1e-4, 1e-5, mask=ok)
    else:
        assert out_s is None
    # points without a return render nothing
    dead = n(c["pts"])[..., 2] <= 0
    assert dead.any() and np.all(n(out_c)[dead] == 0) and np.all(n(out_a)[dead] == 0)


@pytest.mark.parametrize("channels,asum,absgrad", [(5, True, True), (17, False, False), (4, True, False)])
def test_rasterize_to_points_bwd(channels, asum, absgrad):
    from oracle import composite
    from splatad_b200 import ops
    c = _lidar_case(2, 3000, 32, 256, 32, 8, channels, 400 + channels)
    g = torch.Generator().manual_seed(4)
    C, H, W = 2, c["H"], c["W"]
    v_c = torch.randn(C, H, W, channels, generator=g)
    v_a = torch.randn(C, H, W, 1, generator=g)
    v_s = torch.randn(C, H, W, 1, generator=g)
    keys = ("means2d", "conics", "feats", "opacities", "pix_vels", "dcomp")
    args64 = [n(c[k]) for k in keys]
    ref_f = composite.rasterize_to_points_fwd(*args64, None, n(c["pts"]), W, H, c["tw"], c["th"], c["offsets"],
                                              c["flatten_ids"], asum, 0.5, dtype=np.float64)
    f32 = composite.rasterize_to_points_fwd(*args64, None, n(c["pts"]), W, H, c["tw"], c["th"], c["offsets"],
                                            c["flatten_ids"], asum, 0.5, amb_tol=1e-4)
    same = (f32["last_ids"] == ref_f["last_ids"]) & ~f32["ambiguous"]
    assert same.mean() > 0.97
    mk = same[..., None].astype(np.float64)
    mask = t(mk)
    leaves = {k: t(c[k]).requires_grad_(True) for k in keys}
    out_c, out_a, out_s, _ = ops.rasterize_to_points(
        leaves["means2d"], leaves["conics"], leaves["feats"], leaves["opacities"], leaves["pix_vels"],
        leaves["dcomp"], t(c["pts"]), W, H, c["tw"], c["th"], t(c["offsets"], torch.int32),
        t(c["flatten_ids"], torch.int32), asum, 0.5, absgrad=absgrad)
    loss = (out_c * t(v_c) * mask).sum() + (out_a * t(v_a) * mask).sum()
    if asum:
        loss = loss + (out_s * t(v_s) * mask).sum()
    loss.backward()
    ref = composite.rasterize_to_points_bwd(*args64, None, n(c["pts"]), W, H, c["tw"], c["th"], c["offsets"],
                                            c["flatten_ids"], asum, 0.5, ref_f["render_alphas"], ref_f["last_ids"],
                                            n(v_c) * mk, n(v_a) * mk, (n(v_s) * mk) if asum else None,
                                            absgrad=absgrad)
    _grad_check("points v_means2d", leaves["means2d"].grad, ref["v_means2d"])
    _grad_check("points v_conics", leaves["conics"].grad, ref["v_conics"])
    _grad_check("points v_features", leaves["feats"].grad, ref["v_colors"])
    _grad_check("points v_opacities", leaves["opacities"].grad, ref["v_opacities"])
    _grad_check("points v_pix_vels", leaves["pix_vels"].grad, ref["v_pix_vels"])
    _grad_check("points v_depth_comps", leaves["dcomp"].grad, ref["v_depth_comps"])
    if absgrad:
        _grad_check("points absgrad", leaves["means2d"].absgrad, ref["v_means2d_abs"])


def test_accumulate_until_points_known_answer():
    """Ten Gaussians stacked on one lidar point at ranges 20..120 m, the point at 85 m, threshold
    0.5 m (the hand-built case of the reference's tests/test_basic.py:1257-1281): the alpha sum
    counts exactly the Gaussians nearer than 84.5 m, and every output has a closed form."""
    from splatad_b200 import ops
    from oracle import isect
    H, W, tw, th = 32, 1800, 64, 4
    elev = torch.linspace(-30.0, 30.0, H)
    az = torch.linspace(-180 + 0.1, 180 - 0.1, W)
    pts = torch.zeros(1, H, W, 4)
    pts[0, :, :, 0] = az[None, :]
    pts[0, :, :, 1] = elev[:, None]
    pi, pj = 16, 900
    pts[0, pi, pj, 2] = 85.0
    N = 10
    means2d = (pts[0, pi, pj, :2] + 0.1).repeat(N, 1)[None]
    conics = torch.tensor([1.0, 0.0, 1.0]).repeat(N, 1)[None]
    depths = torch.linspace(20.0, 120.0, N)[None]
    g = torch.Generator().manual_seed(9)
    opac = torch.rand(1, N, generator=g)
    feats = torch.cat([torch.randn(1, N, 5, generator=g), depths[..., None]], -1)
    radii = torch.ones(1, N, 2)
    eb = torch.linspace(-30.0 - 1e-2, 30.0 + 1e-2, H // th + 1)
    res = 0.2 * tw
    _, ids, flat = isect.isect_lidar_tiles(n(means2d), n(radii), n(depths), n(eb), res, -180.0)
    offs = isect.isect_offset_encode(ids, 1, math.ceil(360 / res), H // th)
    out_c, out_a, out_s, out_m = ops.rasterize_to_points(
        t(means2d), t(conics), t(feats), t(opac), torch.zeros(1, N, 3, device=DEV),
        torch.zeros(1, N, 2, device=DEV), t(pts), W, H, tw, th, t(offs, torch.int32), t(flat, torch.int32),
        True, 0.5)
    # closed form
    alpha = np.minimum(0.999, n(opac)[0].astype(np.float64) * math.exp(-0.5 * (0.1 ** 2 + 0.1 ** 2)))
    T, want_c, want_s, median = 1.0, np.zeros(6), 0.0, 0.0
    for k in range(N):
        if alpha[k] < 1 / 255:
            continue
        nT = T * (1 - alpha[k])
        if nT <= 1e-4:
            break
        want_c += n(feats)[0, k] * alpha[k] * T
        if T > 0.5 >= nT:
            median = float(depths[0, k])
        if float(depths[0, k]) < 85.0 - 0.5:
            want_s += alpha[k]
        T = nT
    assert_close("known answer features", n(out_c)[0, pi, pj], want_c, 1e-4, 1e-5)
    assert_close("known answer alpha", n(out_a)[0, pi, pj, 0], 1 - T, 1e-4, 1e-5)
    assert_close("known answer alpha sum", n(out_s)[0, pi, pj, 0], want_s, 1e-4, 1e-5)
    assert_close("known answer median", n(out_m)[0, pi, pj, 0], median, 1e-5, 1e-5)
    # every other point has range 0: nothing rendered
    others = np.ones((H, W), bool)
    others[pi, pj] = False
    assert np.all(n(out_a)[0, others] == 0) and np.all(n(out_c)[0, others] == 0)


@pytest.mark.parametrize("channels", [1, 5, 32])
def test_rasterize_to_points_split_ranges(channels):
    """Ranges passed as their own array give the same render and the same gradients as ranges
    concatenated to the features as last channel (the reference's layout, gsplat/rendering.py:779)."""
    from splatad_b200 import ops
    c = _lidar_case(2, 3000, 32, 256, 32, 8, channels, 500 + channels)
    g = torch.Generator().manual_seed(5)
    C, H, W = 2, c["H"], c["W"]
    v = [t(torch.randn(C, H, W, k, generator=g)) for k in (channels, 1, 1)]
    common = lambda L: (L["opacities"], L["pix_vels"], L["dcomp"], t(c["pts"]), W, H, c["tw"], c["th"],
                        t(c["offsets"], torch.int32), t(c["flatten_ids"], torch.int32), True, 0.5)
    keys = ("means2d", "conics", "feats", "opacities", "pix_vels", "dcomp")
    A = {k: t(c[k]).requires_grad_(True) for k in keys}
    outs_a = ops.rasterize_to_points(A["means2d"], A["conics"], A["feats"], *common(A))
    B = {k: t(c[k]).requires_grad_(True) for k in keys if k != "feats"}
    B["f"] = t(c["feats"][..., :-1].contiguous()).requires_grad_(True)
    B["r"] = t(c["feats"][..., -1].contiguous()).requires_grad_(True)
    outs_b = ops.rasterize_to_points_split(B["means2d"], B["conics"], B["f"], B["r"], *common(B))
    # same decisions, same arithmetic; the compiler may contract the range accumulation differently
    assert_close("split render", n(outs_b[0]), n(outs_a[0]), 1e-6, 1e-7)
    for a, b in zip(outs_a[1:], outs_b[1:]):
        assert torch.equal(a, b)
    for outs in (outs_a, outs_b):
        (outs[0] * v[0]).sum().add((outs[1] * v[1]).sum()).add((outs[2] * v[2]).sum()).backward()
    for k in ("means2d", "conics", "opacities", "pix_vels", "dcomp"):
        _grad_check(f"split {k}", B[k].grad, n(A[k].grad), rel=1e-5)
    if channels > 1:
        _grad_check("split features", B["f"].grad, n(A["feats"].grad[..., :-1]), rel=1e-5)
    _grad_check("split ranges", B["r"].grad, n(A["feats"].grad[..., -1]), rel=1e-5)
