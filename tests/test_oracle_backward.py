"""The analytic backward of the C compositing oracle against torch.autograd through a plain
float64 per-pixel compositor written here (camera and lidar), and the projection oracle's
autograd against finite differences. Pins the arbiter used by the GPU gradient tests."""

import math

import numpy as np
import torch

from oracle import composite, isect, projection

# the thresholds are float32 constants in the kernels and in the C oracle
A_MAX = float(np.float32(0.999))
A_MIN = float(np.float32(1.0) / np.float32(255.0))
T_STOP = float(np.float32(1e-4))


def _torch_composite_pixels(means2d, conics, colors, opac, pix_vels, rs, offsets, flat, W, H, ts, bg=None):
    C, th, tw = offsets.shape
    n_isects = len(flat)
    offs = np.concatenate([offsets.reshape(-1), [n_isects]])
    out_c = torch.zeros(C, H, W, colors.shape[-1], dtype=torch.float64)
    out_a = torch.zeros(C, H, W, 1, dtype=torch.float64)
    m2, cn, cl, op, pv = (x.reshape(-1, x.shape[-1]) if x.dim() == 3 else x.reshape(-1)
                          for x in (means2d, conics, colors, opac, pix_vels))
    for cam in range(C):
        for i in range(H):
            for j in range(W):
                tile = cam * th * tw + (i // ts) * tw + (j // ts)
                px, py = j + 0.5, i + 0.5
                roll = rs[cam] * ((py - 0.5) / (H - 1) - 0.5)
                T = torch.ones((), dtype=torch.float64)
                acc = torch.zeros(colors.shape[-1], dtype=torch.float64)
                for idx in range(offs[tile], offs[tile + 1]):
                    g = int(flat[idx])
                    dx = m2[g, 0] + roll * pv[g, 0] - px
                    dy = m2[g, 1] + roll * pv[g, 1] - py
                    sigma = 0.5 * (cn[g, 0] * dx * dx + cn[g, 2] * dy * dy) + cn[g, 1] * dx * dy
                    alpha = torch.clamp_max(op[g] * torch.exp(-sigma), A_MAX)
                    if float(sigma) < 0 or float(alpha) < A_MIN:
                        continue
                    nT = T * (1 - alpha)
                    if float(nT) <= T_STOP:
                        break
                    acc = acc + cl[g] * alpha * T
                    T = nT
                if bg is not None:
                    acc = acc + T * bg[cam]
                out_c[cam, i, j] = acc
                out_a[cam, i, j, 0] = 1 - T
    return out_c, out_a


def test_pixels_backward_matches_autograd():
    g = torch.Generator().manual_seed(0)
    C, N, W, H, ts, ch = 2, 40, 12, 8, 4, 3
    means2d = (torch.rand(C, N, 2, generator=g, dtype=torch.float64) * 1.2 - 0.1) * torch.tensor([W, H])
    sig = torch.rand(C, N, 2, generator=g, dtype=torch.float64) * 2 + 0.8
    conics = torch.stack([1 / sig[..., 0] ** 2, torch.zeros(C, N, dtype=torch.float64) + 0.02, 1 / sig[..., 1] ** 2], -1)
    opac = torch.rand(C, N, generator=g, dtype=torch.float64) * 0.9 + 0.05
    opac[:, ::7] = 1.0
    colors = torch.randn(C, N, ch, generator=g, dtype=torch.float64)
    pix_vels = torch.randn(C, N, 2, generator=g, dtype=torch.float64) * 10
    rs = torch.tensor([0.05, 0.0], dtype=torch.float64)
    bg = torch.rand(C, ch, generator=g, dtype=torch.float64)
    depths = torch.rand(C, N, generator=g)
    radii = (3 * sig + 1).to(torch.int32)
    tw, th = math.ceil(W / ts), math.ceil(H / ts)
    _, ids, flat = isect.isect_tiles(means2d.float().numpy(), radii.numpy(), depths.numpy(), ts, tw, th)
    offs = isect.isect_offset_encode(ids, C, tw, th)
    leaves = [x.clone().requires_grad_(True) for x in (means2d, conics, colors, opac, pix_vels)]
    out_c, out_a = _torch_composite_pixels(*leaves, rs, offs, flat, W, H, ts, bg)
    v_c = torch.randn(out_c.shape, generator=g, dtype=torch.float64)
    v_a = torch.randn(out_a.shape, generator=g, dtype=torch.float64)
    grads = torch.autograd.grad((out_c * v_c).sum() + (out_a * v_a).sum(), leaves)
    a = [x.numpy() for x in (means2d, conics, colors, opac, pix_vels)]
    fwd = composite.rasterize_to_pixels_fwd(*a, rs.numpy(), bg.numpy(), W, H, ts, offs, flat, dtype=np.float64)
    np.testing.assert_allclose(fwd["render_colors"], out_c.detach().numpy(), rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(fwd["render_alphas"], out_a.detach().numpy(), rtol=1e-10, atol=1e-12)
    assert fwd["contributing"] > 500
    bwd = composite.rasterize_to_pixels_bwd(*a, rs.numpy(), bg.numpy(), W, H, ts, offs, flat, fwd["render_alphas"],
                                            fwd["last_ids"], v_c.numpy(), v_a.numpy(), absgrad=True)
    for name, want in zip(("v_means2d", "v_conics", "v_colors", "v_opacities", "v_pix_vels"), grads):
        np.testing.assert_allclose(bwd[name], want.numpy(), rtol=1e-7, atol=1e-9, err_msg=name)
    assert np.all(bwd["v_means2d_abs"] >= np.abs(bwd["v_means2d"]) - 1e-12)


def _wrap(d):
    d = torch.fmod(d + 180.0, 360.0) - 180.0
    return torch.where(d < -180.0, d + 360.0, d)


def test_points_backward_matches_autograd_without_alpha_cap():
    """With every alpha below the 0.999 cap the reference's analytic lidar backward is the true
    gradient (under the cap it also drops the depth-compensation terms, which autograd keeps)."""
    g = torch.Generator().manual_seed(1)
    C, N, W, H, tw_, th_, ch = 1, 30, 16, 4, 8, 2, 4
    az = torch.linspace(-179.0, 179.0, W, dtype=torch.float64)
    el = torch.linspace(-6.0, 6.0, H, dtype=torch.float64)
    pts = torch.zeros(C, H, W, 4, dtype=torch.float64)
    pts[..., 0] = az[None, None, :]
    pts[..., 1] = el[None, :, None]
    pts[..., 2] = torch.rand(C, H, W, generator=g, dtype=torch.float64) * 40 + 5
    pts[..., 3] = (torch.rand(C, H, W, generator=g, dtype=torch.float64) - 0.5) * 0.1
    means2d = torch.stack([torch.rand(C, N, generator=g, dtype=torch.float64) * 360 - 180,
                           torch.rand(C, N, generator=g, dtype=torch.float64) * 12 - 6], -1)
    sig = torch.stack([torch.rand(C, N, generator=g, dtype=torch.float64) * 30 + 20,
                       torch.rand(C, N, generator=g, dtype=torch.float64) * 4 + 3], -1)
    conics = torch.stack([1 / sig[..., 0] ** 2, torch.full((C, N), 1e-3, dtype=torch.float64), 1 / sig[..., 1] ** 2], -1)
    opac = torch.rand(C, N, generator=g, dtype=torch.float64) * 0.8 + 0.1
    feats = torch.randn(C, N, ch, generator=g, dtype=torch.float64)
    feats[..., -1] = torch.rand(C, N, generator=g, dtype=torch.float64) * 50
    pix_vels = torch.randn(C, N, 3, generator=g, dtype=torch.float64) * 3
    dcomp = torch.randn(C, N, 2, generator=g, dtype=torch.float64) * 0.05
    eb = torch.tensor([-7.0, 0.0, 7.0])
    radii = (3 * sig).float()
    res = (360.0 / W) * tw_
    _, ids, flat = isect.isect_lidar_tiles(means2d.float().numpy(), radii.numpy(), feats[..., -1].float().numpy(),
                                           eb.numpy(), res, -180.0)
    n_az = math.ceil(360 / res)
    offs = isect.isect_offset_encode(ids, C, n_az, 2)
    offs_flat = np.concatenate([offs.reshape(-1), [len(flat)]])
    leaves = [x.clone().requires_grad_(True) for x in (means2d, conics, feats, opac, pix_vels, dcomp)]
    m2, cn, ft, op, pv, dc = leaves
    thr = 0.5
    out_c = torch.zeros(C, H, W, ch, dtype=torch.float64)
    out_a = torch.zeros(C, H, W, 1, dtype=torch.float64)
    out_s = torch.zeros(C, H, W, 1, dtype=torch.float64)
    for i in range(H):
        for j in range(W):
            tile = (i // th_) * n_az + (j // tw_)
            px, py, pz, roll = pts[0, i, j]
            T = torch.ones((), dtype=torch.float64)
            acc = torch.zeros(ch, dtype=torch.float64)
            s = torch.zeros((), dtype=torch.float64)
            for idx in range(offs_flat[tile], offs_flat[tile + 1]):
                k = int(flat[idx])
                dx = _wrap(m2[0, k, 0] + roll * pv[0, k, 0] - px)
                dy = _wrap(m2[0, k, 1] + roll * pv[0, k, 1] - py)
                sigma = 0.5 * (cn[0, k, 0] * dx * dx + cn[0, k, 2] * dy * dy) + cn[0, k, 1] * dx * dy
                alpha = torch.clamp_max(op[0, k] * torch.exp(-sigma), A_MAX)
                if float(sigma) < 0 or float(alpha) < A_MIN:
                    continue
                nT = T * (1 - alpha)
                if float(nT) <= T_STOP:
                    break
                w = alpha * T
                extra = dc[0, k, 0] * dx + dc[0, k, 1] * dy + pv[0, k, 2] * roll
                acc = acc + ft[0, k] * w + torch.nn.functional.one_hot(torch.tensor(ch - 1), ch) * extra * w
                if float(ft[0, k, -1]) < float(pz) - thr:
                    s = s + alpha
                T = nT
            out_c[0, i, j] = acc
            out_a[0, i, j, 0] = 1 - T
            out_s[0, i, j, 0] = s
    v_c = torch.randn(out_c.shape, generator=g, dtype=torch.float64)
    v_a = torch.randn(out_a.shape, generator=g, dtype=torch.float64)
    v_s = torch.randn(out_s.shape, generator=g, dtype=torch.float64)
    grads = torch.autograd.grad((out_c * v_c).sum() + (out_a * v_a).sum() + (out_s * v_s).sum(), leaves)
    a = [x.numpy() for x in (means2d, conics, feats, opac, pix_vels, dcomp)]
    fwd = composite.rasterize_to_points_fwd(*a, None, pts.numpy(), W, H, tw_, th_, offs, flat, True, thr, dtype=np.float64)
    np.testing.assert_allclose(fwd["render_colors"], out_c.detach().numpy(), rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(fwd["render_alphas"], out_a.detach().numpy(), rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(fwd["alpha_sum"], out_s.detach().numpy(), rtol=1e-9, atol=1e-11)
    assert fwd["contributing"] > 300
    bwd = composite.rasterize_to_points_bwd(*a, None, pts.numpy(), W, H, tw_, th_, offs, flat, True, thr,
                                            fwd["render_alphas"], fwd["last_ids"], v_c.numpy(), v_a.numpy(),
                                            v_s.numpy())
    # the depth channel's own gradient: autograd sees the range both as a feature and in the
    # (non-differentiated) alpha-sum comparison, like the analytic formula
    for name, want in zip(("v_means2d", "v_conics", "v_colors", "v_opacities", "v_pix_vels", "v_depth_comps"), grads):
        np.testing.assert_allclose(bwd[name], want.numpy(), rtol=1e-7, atol=1e-9, err_msg=name)


def test_projection_oracle_autograd_vs_finite_differences():
    g = torch.Generator().manual_seed(2)
    N = 6
    means = torch.randn(N, 3, generator=g, dtype=torch.float64) * 5 + torch.tensor([12.0, 3.0, 0.5])
    quats = torch.randn(N, 4, generator=g, dtype=torch.float64)
    scales = torch.rand(N, 3, generator=g, dtype=torch.float64) * 0.4 + 0.1
    vel = torch.randn(N, 3, generator=g, dtype=torch.float64)
    vm = torch.eye(4, dtype=torch.float64)[None]
    lin = torch.tensor([[5.0, 1.0, 0.0]], dtype=torch.float64)
    ang = torch.tensor([[0.0, 0.02, 0.1]], dtype=torch.float64)
    rs = torch.tensor([0.1], dtype=torch.float64)

    def f(m, q, s, v):
        out = projection.fully_fused_lidar_projection(m, None, q, s, v, vm, lin, ang, rs, eps2d=0.017)
        return out[1].sum() + (out[3] * 0.01).sum() + out[5].sum() + (out[6] * 3).sum() + out[2].sum()

    assert torch.autograd.gradcheck(f, [x.clone().requires_grad_(True) for x in (means, quats, scales, vel)],
                                    eps=1e-6, atol=1e-5, rtol=1e-4)
