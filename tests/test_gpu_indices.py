"""Parity of rasterize_to_indices_in_range / rasterize_to_indices_in_range_lidar (through the C
ABI) against the oracle: the same triples in the same order, bit-exact, for every pixel whose
threshold decisions are not within 2e-5 (relative) of flipping (the oracle flags those; a pixel
that is flagged may list one Gaussian more or fewer and everything behind it may differ).
Plus the reference's own use of the op (gsplat/cuda/_torch_impl.py:822-903): batched loop ->
accumulate -> image, compared with the fused compositing of this library.
"""

import numpy as np
import pytest
import torch

from gpu_util import DEV, assert_close, n, t
from test_gpu_composite import _camera_case, _lidar_case

pytestmark = pytest.mark.gpu


def _check_triples(label, got, ref, C, H, W):
    g_ids, p_ids, c_ids = (n(x) for x in got)
    for x in got:
        assert x.dtype == torch.int64 and x.is_cuda and x.dim() == 1
    assert g_ids.shape == p_ids.shape == c_ids.shape
    ray = c_ids * H * W + p_ids
    assert (np.diff(ray) >= 0).all(), f"{label}: not ordered by camera / pixel"
    assert ((p_ids >= 0) & (p_ids < H * W) & (c_ids >= 0) & (c_ids < C)).all()
    ok = ~ref["ambiguous"].reshape(-1)
    assert ok.mean() > 0.98, f"{label}: {1 - ok.mean():.3%} of the pixels sit on a threshold"
    counts = np.bincount(ray, minlength=C * H * W)
    want = ref["counts"].reshape(-1)
    assert (counts[ok] == want[ok]).all(), f"{label}: {(counts[ok] != want[ok]).sum()} pixel counts differ"
    ref_ray = ref["camera_ids"] * H * W + ref["pixel_ids"]
    keep, ref_keep = ok[ray], ok[ref_ray]
    assert np.array_equal(ray[keep], ref_ray[ref_keep])
    assert np.array_equal(g_ids[keep], ref["gaussian_ids"][ref_keep]), f"{label}: Gaussian lists differ"
    return int(keep.sum())


def _transmittances(C, H, W, seed):
    g = torch.Generator().manual_seed(seed)
    T = torch.rand(C, H, W, generator=g)
    T[torch.rand(C, H, W, generator=g) < 0.1] = 0.0       # opaque already
    T[torch.rand(C, H, W, generator=g) < 0.1] = 1.0
    return T


@pytest.mark.parametrize("ts,W,H", [(16, 200, 120), (8, 96, 70), (5, 61, 33)])
def test_indices_in_range_pixels(ts, W, H):
    from oracle import composite
    from splatad_b200 import ops
    C, N = 2, 3000
    c = _camera_case(C, N, W, H, ts, 3, 900 + ts)
    args_ref = (n(c["means2d"]), n(c["conics"]), n(c["opacities"]), n(c["pix_vels"]), W, H, ts, c["offsets"],
                c["flatten_ids"])
    args = (t(c["means2d"]), t(c["conics"]), t(c["opacities"]), t(c["pix_vels"]), W, H, ts,
            t(c["offsets"], torch.int32), t(c["flatten_ids"], torch.int32))
    fl = np.concatenate([c["offsets"].reshape(-1), [c["flatten_ids"].size]])
    nb = int(np.ceil((fl[1:] - fl[:-1]).max() / (ts * ts)))
    assert nb >= 2
    listed = 0
    for (lo, hi, T) in [(0, 10 ** 10, torch.ones(C, H, W)), (0, 1, _transmittances(C, H, W, 1)),
                        (1, 3, _transmittances(C, H, W, 2)), (nb - 1, nb, torch.ones(C, H, W)),
                        (nb, nb + 5, torch.ones(C, H, W))]:
        ref = composite.rasterize_to_indices_in_range(lo, hi, n(T), *args_ref, rs_time=n(c["rs"]))
        got = ops.rasterize_to_indices_in_range(lo, hi, t(T), *args, rolling_shutter_time=t(c["rs"]))
        listed += _check_triples(f"pixels ts={ts} range=({lo},{hi})", got, ref, C, H, W)
        if lo >= nb:
            assert got[0].numel() == 0
    assert listed > 10 * W * H
    # no rolling shutter argument = zeros
    ref = composite.rasterize_to_indices_in_range(0, 2, np.ones((C, H, W), np.float32), *args_ref)
    got = ops.rasterize_to_indices_in_range(0, 2, torch.ones(C, H, W, device=DEV), *args)
    _check_triples("pixels no rolling shutter", got, ref, C, H, W)


@pytest.mark.parametrize("tw,th,W,H,N", [(32, 8, 512, 32, 16000), (16, 4, 250, 30, 4000)])
def test_indices_in_range_points(tw, th, W, H, N):
    from oracle import composite
    from splatad_b200 import ops
    C = 2
    c = _lidar_case(C, N, H, W, tw, th, 2, 950 + tw)
    args_ref = (n(c["means2d"]), n(c["conics"]), n(c["opacities"]), n(c["pix_vels"]), n(c["pts"]), W, H, tw, th,
                c["offsets"], c["flatten_ids"])
    args = (t(c["means2d"]), t(c["conics"]), t(c["opacities"]), t(c["pix_vels"]), t(c["pts"]), W, H, tw, th,
            t(c["offsets"], torch.int32), t(c["flatten_ids"], torch.int32))
    fl = np.concatenate([c["offsets"].reshape(-1), [c["flatten_ids"].size]])
    nb = int(np.ceil((fl[1:] - fl[:-1]).max() / (tw * th)))
    assert nb >= 2
    listed = 0
    for (lo, hi, T) in [(0, 10 ** 10, torch.ones(C, H, W)), (0, 1, _transmittances(C, H, W, 3)),
                        (1, 2, _transmittances(C, H, W, 4)), (nb, nb + 1, torch.ones(C, H, W))]:
        ref = composite.rasterize_to_indices_in_range_lidar(lo, hi, n(T), *args_ref)
        got = ops.rasterize_to_indices_in_range_lidar(lo, hi, t(T), *args)
        listed += _check_triples(f"points tile={tw}x{th} range=({lo},{hi})", got, ref, C, H, W)
    assert listed > 5 * W * H
    # points without a return list nothing
    dead = (n(c["pts"])[..., 2] <= 0).reshape(-1)
    got = ops.rasterize_to_indices_in_range_lidar(0, 10 ** 10, torch.ones(C, H, W, device=DEV), *args)
    ray = n(got[2]) * H * W + n(got[1])
    assert dead.any() and not dead[ray].any()


def test_indices_edge_cases():
    from splatad_b200 import ops
    C, N, W, H, ts = 1, 5, 40, 24, 8
    z = lambda *s: torch.zeros(*s, device=DEV)
    offs = torch.zeros(C, 3, 5, dtype=torch.int32, device=DEV)
    empty = torch.zeros(0, dtype=torch.int32, device=DEV)
    got = ops.rasterize_to_indices_in_range(0, 4, torch.ones(C, H, W, device=DEV), z(C, N, 2), z(C, N, 3), z(C, N),
                                            z(C, N, 2), W, H, ts, offs, empty)
    assert all(x.numel() == 0 and x.dtype == torch.int64 for x in got)
    with pytest.raises(AssertionError):   # the tile grid must cover the image, as in the reference
        ops.rasterize_to_indices_in_range(0, 4, torch.ones(C, H, W, device=DEV), z(C, N, 2), z(C, N, 3), z(C, N),
                                          z(C, N, 2), W, H, 4, offs, empty)
    # one Gaussian over the whole image, listed once per pixel; every pixel of the tile grid's
    # ragged last row/column outside the image is ignored
    means2d = torch.tensor([[[20.0, 12.0]]], device=DEV)
    conics = torch.tensor([[[1e-4, 0.0, 1e-4]]], device=DEV)
    opac = torch.tensor([[0.5]], device=DEV)
    offs = torch.arange(15, dtype=torch.int32, device=DEV).reshape(1, 3, 5)
    flat = torch.zeros(15, dtype=torch.int32, device=DEV)
    g_ids, p_ids, c_ids = ops.rasterize_to_indices_in_range(0, 1, torch.ones(1, H, W, device=DEV), means2d, conics,
                                                            opac, z(1, 1, 2), W, H, ts, offs, flat)
    assert g_ids.numel() == W * H and (g_ids == 0).all() and (c_ids == 0).all()
    assert torch.equal(p_ids, torch.arange(W * H, device=DEV))


def _accumulate_torch(means2d, conics, opacities, colors, pix_vels, rs, g_ids, p_ids, c_ids, W, H):
    """gsplat/cuda/_torch_impl.py:610-700 in float64 torch ops on the device, the two nerfacc helpers
    as a segmented exclusive product (log-space cumulative sum)."""
    C = means2d.shape[0]
    f = lambda x: x.double()
    x, y = p_ids % W, p_ids // W
    roll = f(rs)[c_ids] * (y.double() / (H - 1) - 0.5)
    coords = torch.stack([x, y], -1).double() + 0.5
    d = f(means2d)[c_ids, g_ids] + roll[:, None] * f(pix_vels)[c_ids, g_ids] - coords
    cn = f(conics)[c_ids, g_ids]
    sigma = 0.5 * (cn[:, 0] * d[:, 0] ** 2 + cn[:, 2] * d[:, 1] ** 2) + cn[:, 1] * d[:, 0] * d[:, 1]
    alpha = torch.clamp_max(f(opacities)[c_ids, g_ids] * torch.exp(-sigma), 0.999)
    ray = c_ids * H * W + p_ids
    n_rays = C * H * W
    lg = torch.log1p(-alpha)
    cs = torch.cumsum(lg, 0)
    excl = cs - lg
    first = torch.ones_like(ray, dtype=torch.bool)
    first[1:] = ray[1:] != ray[:-1]
    seg_base = torch.zeros(n_rays, dtype=torch.float64, device=ray.device)
    seg_base[ray[first]] = excl[first]
    w = alpha * torch.exp(excl - seg_base[ray])
    out = torch.zeros(n_rays, colors.shape[-1], dtype=torch.float64, device=ray.device)
    out.index_add_(0, ray, w[:, None] * f(colors)[c_ids, g_ids])
    acc = torch.zeros(n_rays, dtype=torch.float64, device=ray.device)
    acc.index_add_(0, ray, w)
    return out.reshape(C, H, W, -1), acc.reshape(C, H, W, 1)


def test_batched_loop_reproduces_the_fused_render():
    """The reference's torch compositor on this library's ops, at a mid-size camera frame: the
    lists come from rasterization()'s own meta (device-built offsets, packed off)."""
    import splatad_b200 as sp
    from splatad_b200 import scenes
    kw = scenes.config1(device=DEV, N=60_000, seed=21, packed=False)
    kw.update(width=640, height=360, sh_degree=None, render_mode="RGB",
              colors=torch.rand(60_000, 3, device=DEV))
    kw["Ks"] = torch.tensor([[[400.0, 0.0, 320.0], [0.0, 400.0, 180.0], [0.0, 0.0, 1.0]]], device=DEV)
    render, alphas, meta = sp.rasterization(**kw)
    W, H, ts = 640, 360, kw["tile_size"]
    C = 1
    offs, flat = meta["isect_offsets"], meta["flatten_ids"]
    fl = torch.cat([offs.flatten()[: C * offs.shape[1] * offs.shape[2]].long(),
                    torch.tensor([flat.numel()], device=DEV)])
    nb = int(((fl[1:] - fl[:-1]).max().item() + ts * ts - 1) // (ts * ts))
    assert nb >= 2
    colors = kw["colors"][None].expand(C, -1, -1)
    rs = kw["rolling_shutter_time"]
    for per_iter in (nb, 1):
        img = torch.zeros(C, H, W, 3, dtype=torch.float64, device=DEV)
        acc = torch.zeros(C, H, W, 1, dtype=torch.float64, device=DEV)
        cnt = torch.zeros(C * H * W, dtype=torch.int64, device=DEV)
        for step in range(0, nb, per_iter):
            T = 1.0 - acc[..., 0]
            g_ids, p_ids, c_ids = sp.rasterize_to_indices_in_range(
                step, step + per_iter, T.float(), meta["means2d"], meta["conics"], meta["opacities"],
                meta["pix_vels"], W, H, ts, offs, flat, rolling_shutter_time=rs)
            if g_ids.numel() == 0:
                break
            cnt += torch.bincount(c_ids * H * W + p_ids, minlength=C * H * W)
            r, a = _accumulate_torch(meta["means2d"], meta["conics"], meta["opacities"], colors, meta["pix_vels"],
                                     rs, g_ids, p_ids, c_ids, W, H)
            img = img + r * T[..., None]
            acc = acc + a * T[..., None]
        if per_iter == nb:
            whole, sel = cnt, np.ones((C, H, W, 1), bool)
            assert cnt.sum().item() > 20 * W * H
        else:
            # pixels that stopped in an earlier call resume (the op keeps no such state, neither does
            # the reference's): they are set aside
            sel = n(cnt == whole).reshape(C, H, W, 1)
            assert sel.mean() > 0.5
        # float32 fused render against a float64 accumulation of the same pairs; a pair whose alpha
        # sits on 1/255 may be in one and not the other: 1e-3 of the pixels may differ
        assert_close(f"loop({per_iter}) colors", n(img), n(render), 1e-4, 2e-5, mask=sel, max_bad_frac=1e-3)
        assert_close(f"loop({per_iter}) alphas", n(acc), n(alphas), 1e-4, 2e-5, mask=sel, max_bad_frac=1e-3)


def test_count_composited_pairs_against_the_oracle_counters():
    """The pair counts behind the compositing flop model: the GPU count of evaluated and blended
    (point, Gaussian) pairs of a frame equals the oracle's counters, up to the handful of pairs whose
    threshold decision is within float32 rounding of flipping."""
    import splatad_b200
    from oracle import pipeline
    from splatad_b200 import ops, scenes
    cfg = scenes.config0(N=8000)
    g = {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in cfg.items()}
    _, _, _, m = splatad_b200.lidar_rasterization(**g)
    tested, contributing = ops.count_composited_pairs(
        m["means2d"], m["conics"], m["opacities"], m["pix_vels"], m["isect_offsets"], m["flatten_ids"],
        m["width"], m["height"], m["tile_width"], m["tile_height"], raster_pts=g["raster_pts"])
    _, _, _, meta = pipeline.lidar_rasterization(**cfg)
    assert contributing > 10_000 and tested >= contributing
    assert abs(tested - meta["tested"]) <= 2e-3 * meta["tested"], (tested, meta["tested"])
    assert abs(contributing - meta["contributing"]) <= 2e-3 * meta["contributing"], (contributing, meta["contributing"])
    cam = scenes.config1(N=5000)
    cam.update(width=320, height=200)
    cam["Ks"] = torch.tensor([[[250.0, 0.0, 160.0], [0.0, 250.0, 100.0], [0.0, 0.0, 1.0]]])
    gc = {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in cam.items()}
    _, _, m = splatad_b200.rasterization(**gc)
    tested, contributing = ops.count_composited_pairs(
        m["means2d"], m["conics"], m["opacities"], m["pix_vels"], m["isect_offsets"], m["flatten_ids"],
        m["width"], m["height"], m["tile_size"], m["tile_size"], rolling_shutter_time=gc["rolling_shutter_time"])
    _, _, meta = pipeline.rasterization(**cam)
    assert abs(tested - meta["tested"]) <= 2e-3 * meta["tested"], (tested, meta["tested"])
    assert abs(contributing - meta["contributing"]) <= 2e-3 * meta["contributing"], (contributing, meta["contributing"])
