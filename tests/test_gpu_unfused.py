"""Parity of the unfused projection ops (through the C ABI) against the reference's own outputs
(fixture ``unfused_ops.npz``) and, for the gradients, against autograd through the float64 oracle.
Forward: 1e-4 relative + small absolute; backward: 1e-3 relative L2."""

import numpy as np
import pytest
import torch

from gpu_util import DEV, assert_close, n, rel_l2, t

pytestmark = pytest.mark.gpu


def _grad_pair(fn_gpu, fn_ref, inputs, grad_names, seed):
    """Runs fn on float32 GPU leaves and on float64 CPU leaves with the same seeded cotangents."""
    g = torch.Generator().manual_seed(seed)
    leaves_g = {k: (t(v).requires_grad_(k in grad_names) if isinstance(v, np.ndarray) else v) for k, v in inputs.items()}
    leaves_r = {k: (torch.as_tensor(v, dtype=torch.float64).requires_grad_(k in grad_names) if isinstance(v, np.ndarray)
                    else v) for k, v in inputs.items()}
    outs_g, outs_r = fn_gpu(**leaves_g), fn_ref(**leaves_r)
    outs_g = [o for o in (outs_g if isinstance(outs_g, tuple) else (outs_g,)) if o is not None]
    outs_r = [o for o in (outs_r if isinstance(outs_r, tuple) else (outs_r,)) if o is not None]
    loss_g, loss_r = 0.0, 0.0
    for og, orf in zip(outs_g, outs_r):
        w = torch.randn(orf.shape, generator=g, dtype=torch.float64)
        loss_g = loss_g + (og * w.to(DEV).float()).sum()
        loss_r = loss_r + (orf * w).sum()
    loss_g.backward()
    loss_r.backward()
    for k in grad_names:
        e = rel_l2(n(leaves_g[k].grad), leaves_r[k].grad.numpy())
        assert e < 1e-3, f"gradient of {k}: relative L2 error {e:.2e}"


def test_quat_scale_to_covar_preci(golden):
    from oracle import projection
    from splatad_b200 import ops
    g = golden("unfused_ops")
    covars, precis = ops.quat_scale_to_covar_preci(t(g["quats"]), t(g["scales"]))
    assert_close("covars", n(covars), g["covars"], 1e-5, 1e-6)
    assert_close("precis", n(precis), g["precis"], 1e-4, 1e-4)
    ct, pt = ops.quat_scale_to_covar_preci(t(g["quats"]), t(g["scales"]), triu=True)
    assert_close("covars triu", n(ct), g["covars_triu"], 1e-5, 1e-6)
    assert_close("precis triu", n(pt), g["precis_triu"], 1e-4, 1e-4)
    only, none = ops.quat_scale_to_covar_preci(t(g["quats"]), t(g["scales"]), compute_preci=False)
    assert none is None and torch.equal(only, covars)
    for triu in (False, True):
        _grad_pair(lambda quats, scales: ops.quat_scale_to_covar_preci(quats, scales, triu=triu),
                   lambda quats, scales: projection.quat_scale_to_covar_preci(quats, scales, triu=triu),
                   dict(quats=g["quats"], scales=g["scales"]), ("quats", "scales"), 1)
    _grad_pair(lambda quats, scales: ops.quat_scale_to_covar_preci(quats, scales, compute_covar=False),
               lambda quats, scales: projection.quat_scale_to_covar_preci(quats, scales, compute_covar=False),
               dict(quats=g["quats"], scales=g["scales"]), ("quats", "scales"), 2)


def test_world_to_cam(golden):
    from oracle import projection
    from splatad_b200 import ops
    g = golden("unfused_ops")
    want_m, want_c = projection.world_to_cam(*(torch.as_tensor(g[k]) for k in ("means", "covars", "viewmats")))
    means_c, covars_c = ops.world_to_cam(t(g["means"]), t(g["covars"]), t(g["viewmats"]))
    assert_close("means_c", n(means_c), n(want_m), 1e-5, 1e-5)
    assert_close("covars_c", n(covars_c), g["covars_c"], 1e-4, 1e-5)
    _grad_pair(ops.world_to_cam, projection.world_to_cam,
               dict(means=g["means"], covars=g["covars"], viewmats=g["viewmats"]), ("means", "covars", "viewmats"), 3)
    # only the pose asks for a gradient
    _grad_pair(ops.world_to_cam, projection.world_to_cam,
               dict(means=g["means"], covars=g["covars"], viewmats=g["viewmats"]), ("viewmats",), 4)


def test_persp_proj_and_pix_velocity(golden):
    from oracle import projection
    from splatad_b200 import ops
    g = golden("unfused_ops")
    W, H = int(g["width"]), int(g["height"])
    m2, c2 = ops.persp_proj(t(g["means_c"]), t(g["covars_c"]), t(g["Ks"]), W, H)
    assert_close("means2d", n(m2), g["means2d"], 1e-5, 1e-3)
    assert_close("covars2d", n(c2), g["covars2d"], 1e-4, 1e-3)
    pv = ops.compute_pix_velocity(t(g["means_c"]), t(g["lin"]), t(g["ang"]), t(g["vel_c"]), t(g["Ks"]), W, H)
    assert_close("pix_vel", n(pv), g["pix_vel"], 1e-4, 1e-3)
    _grad_pair(lambda means, covars, Ks: ops.persp_proj(means, covars, Ks, W, H),
               lambda means, covars, Ks: projection.persp_proj(means, covars, Ks, W, H),
               dict(means=g["means_c"], covars=g["covars_c"], Ks=g["Ks"]), ("means", "covars"), 5)
    _grad_pair(lambda p_view, lin, ang, vel, Ks: ops.compute_pix_velocity(p_view, lin, ang, vel, Ks, W, H),
               lambda p_view, lin, ang, vel, Ks: projection.compute_pix_velocity(p_view, lin, ang, vel, Ks, W, H),
               dict(p_view=g["means_c"], lin=g["lin"], ang=g["ang"], vel=g["vel_c"], Ks=g["Ks"]), ("p_view", "vel"), 6)


def test_lidar_proj_and_lidar_velocity(golden):
    from oracle import projection
    from splatad_b200 import ops
    g = golden("unfused_ops")
    eps = float(g["eps2d"])
    m2, c2, dc = ops.lidar_proj(t(g["means_c"]), t(g["covars_c"]), eps)
    assert_close("lidar means2d", n(m2), g["lidar_means2d"], 1e-5, 1e-4)
    assert_close("lidar covars2d", n(c2), g["lidar_covars2d"], 1e-4, 1e-5)
    assert_close("lidar depth comp", n(dc), g["lidar_depth_comp"], 1e-3, 1e-5)
    lv = ops.compute_lidar_velocity(t(g["means_c"]), t(g["lin"]), t(g["ang"]), t(g["vel_c"]))
    assert_close("lidar vel", n(lv), g["lidar_vel"], 1e-4, 1e-4)
    _grad_pair(lambda means, covars: ops.lidar_proj(means, covars, eps),
               lambda means, covars: projection.lidar_proj(means, covars, eps),
               dict(means=g["means_c"], covars=g["covars_c"]), ("means", "covars"), 7)
    _grad_pair(ops.compute_lidar_velocity, projection.compute_lidar_velocity,
               dict(p_view=g["means_c"], lin_vel=g["lin"], ang_vel=g["ang"], velocities=g["vel_c"]),
               ("p_view", "velocities"), 8)
