"""The oracle's unfused projection ops against the reference's own torch implementations
(fixture ``unfused_ops.npz`` written by tests/golden/make_golden.py from
gsplat/cuda/_torch_impl.py:10-262)."""

import numpy as np
import torch

from oracle import projection


def _t(x):
    return torch.as_tensor(np.asarray(x))


def _close(name, got, want, rtol=2e-5, atol=1e-6):
    got, want = got.detach().numpy(), np.asarray(want)
    assert got.shape == want.shape, (name, got.shape, want.shape)
    err = np.abs(got - want)
    assert (err <= atol + rtol * np.abs(want)).all(), f"{name}: max abs err {err.max():.3e}"


def test_unfused_ops_match_reference_outputs(golden):
    g = golden("unfused_ops")
    quats, scales = _t(g["quats"]), _t(g["scales"])
    covars, precis = projection.quat_scale_to_covar_preci(quats, scales)
    _close("covars", covars, g["covars"])
    _close("precis", precis, g["precis"], rtol=1e-4, atol=1e-4)
    ct, pt = projection.quat_scale_to_covar_preci(quats, scales, triu=True)
    _close("covars triu", ct, g["covars_triu"])
    _close("precis triu", pt, g["precis_triu"], rtol=1e-4, atol=1e-4)
    only_c, none_p = projection.quat_scale_to_covar_preci(quats, scales, compute_preci=False)
    assert none_p is None and torch.equal(only_c, covars)
    means_c, covars_c = projection.world_to_cam(_t(g["means"]), _t(g["covars"]), _t(g["viewmats"]))
    # the fixture moved the sensor-frame points in front of the sensor after this call
    _close("covars_c", covars_c, g["covars_c"], rtol=1e-4, atol=1e-5)
    mc, cc, Ks = _t(g["means_c"]), _t(g["covars_c"]), _t(g["Ks"])
    W, H = int(g["width"]), int(g["height"])
    m2, c2 = projection.persp_proj(mc, cc, Ks, W, H)
    _close("means2d", m2, g["means2d"], rtol=1e-5, atol=1e-3)
    _close("covars2d", c2, g["covars2d"], rtol=1e-4, atol=1e-3)
    lin, ang, vel = _t(g["lin"]), _t(g["ang"]), _t(g["vel_c"])
    _close("pix_vel", projection.compute_pix_velocity(mc, lin, ang, vel, Ks, W, H), g["pix_vel"], rtol=1e-4, atol=1e-3)
    lm, lc, ld = projection.lidar_proj(mc, cc, float(g["eps2d"]))
    _close("lidar means2d", lm, g["lidar_means2d"], rtol=1e-5, atol=1e-4)
    _close("lidar covars2d", lc, g["lidar_covars2d"], rtol=1e-4, atol=1e-5)
    _close("lidar depth comp", ld, g["lidar_depth_comp"], rtol=1e-3, atol=1e-5)
    _close("lidar vel", projection.compute_lidar_velocity(mc, lin, ang, vel), g["lidar_vel"], rtol=1e-4, atol=1e-4)
