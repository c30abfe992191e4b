"""End-to-end gradient parity: a training step through the WHOLE ``lidar_rasterization()`` /
``rasterization()`` call (projection -> colours -> tile lists -> compositing and back, packed
gathers and fused colour kernels included) against an independent float64 chain - the oracle's
differentiable projection and SH (torch autograd) feeding the analytic compositing backward of the
C oracle - on the product's own (bit-exact, separately tested) tile lists.

Bar: relative L2 error below 1e-3 for the gradient of every Gaussian parameter (means, quats,
scales, opacities, SH coefficients / features, and velocities under ``ops.velocity_grads()``), and
elementwise 1e-3 relative with an absolute floor of 2e-3 of the gradient's RMS. The loss only
counts pixels / points whose include / skip / stop decisions are the same in float32 and float64
(the oracle flags the others), and the scenes drop the few Gaussians that one projection culls
and the other keeps (a float32 rounding at a culling plane), so both sides differentiate the same
function.
"""

import numpy as np
import pytest
import torch

from gpu_util import DEV, assert_close, n, rel_l2

pytestmark = pytest.mark.gpu

GAUSS = ("means", "quats", "scales", "opacities", "velocities")


def _to_gpu(cfg):
    return {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in cfg.items()}


def _grad_check(label, got, want, rel=1e-3):
    got, want = n(got).astype(np.float64), n(want).astype(np.float64)
    rms = float(np.sqrt(np.mean(want ** 2)))
    assert rms > 0, f"{label}: the reference gradient is zero"
    e = rel_l2(got, want)
    print(f"{label}: relative L2 error {e:.2e}")
    assert e < rel, f"{label}: relative L2 error {e:.3e}"
    assert_close(label, got, want, rel, 2 * rel * rms, max_bad_frac=2e-3)


def _subset(cfg, keep, per_gaussian):
    out = dict(cfg)
    for k in per_gaussian:
        v = cfg.get(k)
        if v is None:
            continue
        out[k] = (v[:, keep] if (k == "lidar_features" or (k == "colors" and v.dim() == 4)) else v[keep]).contiguous()
    return out


def _drop_disputed_lidar(cfg):
    """Removes the Gaussians that the float32 product and the float64 oracle do not cull alike."""
    from oracle import projection as op
    from splatad_b200 import ops
    C = cfg["viewmats"].shape[0]
    z = lambda *s: torch.zeros(*s)  # noqa: E731
    lin, ang, rs = (cfg.get("linear_velocity", z(C, 3)), cfg.get("angular_velocity", z(C, 3)),
                    cfg.get("rolling_shutter_time", z(C)))
    kw = dict(min_elevation=cfg["min_elevation"], max_elevation=cfg["max_elevation"], min_azimuth=cfg["min_azimuth"],
              max_azimuth=cfg["max_azimuth"], eps2d=cfg["eps2d"])
    d = lambda x: None if x is None else x.double()  # noqa: E731
    g = lambda x: None if x is None else x.to(DEV)  # noqa: E731
    with torch.no_grad():
        want = op.fully_fused_lidar_projection(d(cfg["means"]), None, d(cfg["quats"]), d(cfg["scales"]),
                                               d(cfg["velocities"]), d(cfg["viewmats"]), d(lin), d(ang), d(rs), **kw)
        got = ops.fully_fused_lidar_projection(g(cfg["means"]), None, g(cfg["quats"]), g(cfg["scales"]),
                                               g(cfg["velocities"]), g(cfg["viewmats"]), g(lin), g(ang), g(rs), **kw)
    keep = ((got[0][..., 0] > 0).cpu() == (want[0][..., 0] > 0)).all(0)
    print(f"dropping {int((~keep).sum())} of {keep.numel()} Gaussians culled differently in float32 and float64")
    assert keep.float().mean() > 0.99
    return _subset(cfg, keep, GAUSS + ("lidar_features",))


def _drop_disputed_camera(cfg):
    from oracle import projection as op
    from splatad_b200 import ops
    C = cfg["viewmats"].shape[0]
    z = lambda *s: torch.zeros(*s)  # noqa: E731
    lin, ang, rs = (cfg.get("linear_velocity", z(C, 3)), cfg.get("angular_velocity", z(C, 3)),
                    cfg.get("rolling_shutter_time", z(C)))
    d = lambda x: None if x is None else x.double()  # noqa: E731
    g = lambda x: None if x is None else x.to(DEV)  # noqa: E731
    with torch.no_grad():
        want = op.fully_fused_projection(d(cfg["means"]), None, d(cfg["quats"]), d(cfg["scales"]),
                                         d(cfg["velocities"]), d(cfg["viewmats"]), d(cfg["Ks"]), cfg["width"],
                                         cfg["height"], d(lin), d(ang), d(rs))
        got = ops.fully_fused_projection(g(cfg["means"]), None, g(cfg["quats"]), g(cfg["scales"]),
                                         g(cfg["velocities"]), g(cfg["viewmats"]), g(cfg["Ks"]), cfg["width"],
                                         cfg["height"], g(lin), g(ang), g(rs))
    # listed by the product (radius > 0 pixels) must be alive in the oracle and the other way round
    alive_p, alive_o = (got[3].abs().sum(-1) > 0).cpu(), want[3].abs().sum(-1) > 0
    seen_p, seen_o = (got[0][..., 0] > 0).cpu(), want[0][..., 0] > 0
    keep = ((alive_p == alive_o) & (seen_p == seen_o)).all(0)
    print(f"dropping {int((~keep).sum())} of {keep.numel()} Gaussians culled differently in float32 and float64")
    assert keep.float().mean() > 0.98
    return _subset(cfg, keep, GAUSS + ("colors",))


def _cotangents(shapes, seed):
    gen = torch.Generator().manual_seed(seed)
    return [None if s is None else torch.randn(s, generator=gen, dtype=torch.float64) for s in shapes]


def _lidar_step(cfg, names, label, **kw):
    import splatad_b200
    from oracle import pipeline
    from splatad_b200 import ops
    cfg = _drop_disputed_lidar(cfg)
    g = _to_gpu(cfg)
    leaves = {k: g[k].clone().requires_grad_(True) for k in names}
    with ops.velocity_grads(True):
        out_c, out_a, out_s, m = splatad_b200.lidar_rasterization(**dict(g, **leaves), **kw)
    cot = _cotangents([out_c.shape, out_a.shape, None if out_s is None else out_s.shape], 17)
    want, mask, f64 = pipeline.lidar_gradients_f64(cfg, n(m["isect_offsets"]), n(m["flatten_ids"]),
                                                   [None if c is None else c.numpy() for c in cot], names, **kw)
    print(f"{label}: {mask.mean():.4f} of the points take part in the loss")
    assert mask.mean() > 0.95
    mk = torch.from_numpy(mask[..., None]).to(DEV)
    assert_close(label + " forward", n(out_c * mk), f64["render_colors"] * mask[..., None], 2e-4, 2e-4,
                 max_bad_frac=1e-3)
    loss = (out_c * cot[0].float().to(DEV) * mk).sum() + (out_a * cot[1].float().to(DEV) * mk).sum()
    if out_s is not None:
        loss = loss + (out_s * cot[2].float().to(DEV) * mk).sum()
    with ops.velocity_grads(True):
        loss.backward()
    for k in names:
        assert leaves[k].grad is not None, f"{label}: no gradient for {k}"
        _grad_check(f"{label} d/d{k}", leaves[k].grad, want[k])


def _camera_step(cfg, names, label):
    import splatad_b200
    from oracle import pipeline
    from splatad_b200 import ops
    cfg = _drop_disputed_camera(cfg)
    g = _to_gpu(cfg)
    leaves = {k: g[k].clone().requires_grad_(True) for k in names}
    with ops.velocity_grads(True):
        out_c, out_a, m = splatad_b200.rasterization(**dict(g, **leaves))
    cot = _cotangents([out_c.shape, out_a.shape], 19)
    cam_ids = None if m["camera_ids"] is None else n(m["camera_ids"])
    gau_ids = None if m["gaussian_ids"] is None else n(m["gaussian_ids"])
    want, mask, f64 = pipeline.camera_gradients_f64(cfg, n(m["isect_offsets"]), n(m["flatten_ids"]),
                                                    [c.numpy() for c in cot], names, camera_ids=cam_ids,
                                                    gaussian_ids=gau_ids)
    print(f"{label}: {mask.mean():.4f} of the pixels take part in the loss")
    assert mask.mean() > 0.95
    mk = torch.from_numpy(mask[..., None]).to(DEV)
    assert_close(label + " forward", n(out_c * mk), f64["render_colors"] * mask[..., None], 2e-4, 2e-4,
                 max_bad_frac=1e-3)
    loss = (out_c * cot[0].float().to(DEV) * mk).sum() + (out_a * cot[1].float().to(DEV) * mk).sum()
    with ops.velocity_grads(True):
        loss.backward()
    for k in names:
        assert leaves[k].grad is not None, f"{label}: no gradient for {k}"
        got = leaves[k].grad
        _grad_check(f"{label} d/d{k}", got.to_dense() if got.is_sparse else got, want[k])


def test_lidar_training_step_gradients():
    """32 x 512 lidar without rolling shutter, 3000 Gaussians, 4 features."""
    from splatad_b200 import scenes
    _lidar_step(scenes.config0(N=3000), ("means", "quats", "scales", "opacities", "lidar_features"), "lidar 32x512")


def test_lidar_rolling_shutter_training_step_gradients():
    """128 x 1800 rolling-shutter lidar (the headline sensor) over 8000 moving Gaussians, 16 features,
    antialiased opacities: every parameter including the Gaussians' velocities."""
    from splatad_b200 import scenes
    cfg = scenes.config2(N=8000)
    cfg["velocities"] = torch.randn(8000, 3, generator=torch.Generator().manual_seed(3)) * 2.0
    _lidar_step(cfg, GAUSS + ("lidar_features",), "lidar 128x1800 rolling", rasterize_mode="antialiased")


@pytest.mark.parametrize("packed", [True, False])
def test_camera_training_step_gradients(packed):
    """Rolling-shutter camera (640 x 360), SH degree 3, RGB + depth, moving Gaussians, packed and
    [C, N] layouts: the packed path goes through the gathers with their index_add backward and the
    fused colour kernel's own VJP."""
    from splatad_b200 import scenes
    cfg = scenes.config1(N=6000, packed=packed)
    cfg.update(width=640, height=360)
    cfg["Ks"] = torch.tensor([[[400.0, 0.0, 320.0], [0.0, 400.0, 180.0], [0.0, 0.0, 1.0]]])
    _camera_step(cfg, GAUSS + ("colors",), f"camera 640x360 packed={packed}")


def test_config4_training_step_gradients_reduced():
    """The training configuration's rig - eight 1920 x 1080 rolling-shutter cameras and two 128-beam
    lidars - on 20,000 Gaussians: parameter gradients of the whole step against the float64 chain."""
    from splatad_b200 import scenes
    cfg = scenes.config4(N=20_000)
    _camera_step(cfg["camera"], ("means", "quats", "scales", "opacities", "colors"), "config4 cameras")
    _lidar_step(cfg["lidar"], ("means", "quats", "scales", "opacities", "lidar_features"), "config4 lidars")
