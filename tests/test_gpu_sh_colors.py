"""Parity of the fused view-dependent colour op (through the C ABI) with the chain it replaces in
rasterization() - gathers by the packed ids, directions, spherical harmonics with the radii mask,
+ 0.5, clamp at zero, depth channel (gsplat/rendering.py:345-373, 383-384) - evaluated by the
oracle's SH (pinned to the reference's torch SH) in float64. Forward 1e-5, gradients 1e-4 relative
to the gradient's scale (float32 sums, atomics in arbitrary order)."""

import numpy as np
import pytest
import torch

from gpu_util import DEV, n

pytestmark = pytest.mark.gpu


def _case(C, N, K, packed, per_camera, seed):
    g = torch.Generator().manual_seed(seed)
    means = torch.randn(N, 3, generator=g) * 5
    camtoworlds = torch.eye(4).repeat(C, 1, 1)
    camtoworlds[:, :3, 3] = torch.randn(C, 3, generator=g) * 3
    coeffs = torch.randn((C, N, K, 3) if per_camera else (N, K, 3), generator=g) * 0.4
    if packed:
        keep = torch.rand(C, N, generator=g) < 0.6
        camera_ids, gaussian_ids = torch.where(keep)
        radii = torch.randint(1, 30, (camera_ids.numel(), 2), generator=g, dtype=torch.int32)
        depths = torch.rand(camera_ids.numel(), generator=g) * 50
    else:
        camera_ids = gaussian_ids = None
        radii = torch.randint(1, 30, (C, N, 2), generator=g, dtype=torch.int32)
        radii[torch.rand(C, N, generator=g) < 0.4] = 0
        depths = torch.rand(C, N, generator=g) * 50
    return means, camtoworlds, coeffs, radii, camera_ids, gaussian_ids, depths


def _chain(sh_degree, means, camtoworlds, coeffs, radii, camera_ids, gaussian_ids, depths):
    """The reference's chain in float64 on the CPU with the oracle's SH."""
    from oracle import projection
    C = camtoworlds.shape[0]
    if gaussian_ids is not None:
        dirs = means[gaussian_ids] - camtoworlds[camera_ids, :3, 3]
        shs = coeffs[gaussian_ids] if coeffs.dim() == 3 else coeffs[camera_ids, gaussian_ids]
    else:
        dirs = means[None] - camtoworlds[:, None, :3, 3]
        shs = coeffs.expand(C, -1, -1, -1) if coeffs.dim() == 3 else coeffs
    colors = projection.spherical_harmonics(sh_degree, dirs, shs, masks=radii[..., 0] > 0)
    colors = torch.clamp_min(colors + 0.5, 0.0)
    if depths is not None:
        colors = torch.cat([colors, depths[..., None]], dim=-1)
    return colors


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("per_camera", [False, True])
@pytest.mark.parametrize("sh_degree,K,with_depth", [(3, 16, True), (0, 1, False), (2, 16, False), (4, 25, True),
                                                    (1, 5, True)])
def test_view_dependent_colors(packed, per_camera, sh_degree, K, with_depth):
    from splatad_b200 import ops
    C, N = 3, 1500
    case = _case(C, N, K, packed, per_camera, 40 + sh_degree)
    means, camtoworlds, coeffs, radii, camera_ids, gaussian_ids, depths = case
    if not with_depth:
        depths = None
    dd = lambda x: None if x is None else x.double().requires_grad_(True)
    ref_in = [dd(means), dd(camtoworlds), dd(coeffs), dd(depths)]
    want = _chain(sh_degree, ref_in[0], ref_in[1], ref_in[2], radii, camera_ids, gaussian_ids, ref_in[3])
    dev = lambda x: None if x is None else x.to(DEV)
    leaf = lambda x: None if x is None else x.to(DEV).requires_grad_(True)
    got_in = [leaf(means), leaf(camtoworlds), leaf(coeffs), leaf(depths)]
    got = ops.view_dependent_colors(sh_degree, got_in[0], got_in[1][:, :3, 3], got_in[2], dev(radii),
                                    dev(camera_ids), dev(gaussian_ids), depths=got_in[3])
    assert got.shape == want.shape and got.dtype == torch.float32
    np.testing.assert_allclose(n(got), want.detach().numpy(), rtol=1e-5, atol=1e-5)
    assert (n(got)[..., :3] == 0).any() or sh_degree == 0   # the clamp is exercised
    if not packed:
        culled = (radii[..., 0] <= 0).numpy()
        assert culled.any() and (n(got)[culled][:, :3] == 0.5).all()
    v = torch.randn(want.shape, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    want.backward(v)
    got.backward(v.float().to(DEV))
    for name, a, b in zip(("means", "camtoworlds", "coeffs", "depths"), got_in, ref_in):
        if a is None:
            continue
        # degree 0 does not depend on the directions: autograd leaves those gradients unset
        gb = np.zeros(b.shape) if b.grad is None else b.grad.numpy()
        ga = n(a.grad)
        scale = np.sqrt((gb ** 2).mean()) + 1e-30
        assert np.abs(ga - gb).max() <= 1e-4 * max(scale, np.abs(gb).max()) + 1e-6, (name, np.abs(ga - gb).max(), scale)
        if name == "camtoworlds":
            assert (np.abs(gb[:, :3, 3]).max() > 0 or sh_degree == 0) and np.abs(ga[:, :3, :3]).max() == 0


def test_matches_the_unfused_ops_bit_for_bit():
    """Same basis arithmetic and summation order as spherical_harmonics(): identical floats."""
    from splatad_b200 import ops
    means, camtoworlds, coeffs, radii, camera_ids, gaussian_ids, depths = (
        x.to(DEV) for x in _case(2, 4000, 16, True, False, 77))
    dirs = means[gaussian_ids] - camtoworlds[camera_ids, :3, 3]
    want = torch.clamp_min(ops.spherical_harmonics(3, dirs, coeffs[gaussian_ids], masks=radii[..., 0] > 0) + 0.5, 0.0)
    got = ops.view_dependent_colors(3, means, camtoworlds[:, :3, 3], coeffs, radii, camera_ids, gaussian_ids,
                                    depths=depths)
    assert torch.equal(got[:, :3], want) and torch.equal(got[:, 3], depths)
    # no entries at all
    e = torch.zeros(0, dtype=torch.int64, device=DEV)
    out = ops.view_dependent_colors(3, means, camtoworlds[:, :3, 3], coeffs,
                                    torch.zeros(0, 2, dtype=torch.int32, device=DEV), e, e)
    assert out.shape == (0, 3)


def test_camera_centers():
    from splatad_b200 import ops
    g = torch.Generator().manual_seed(3)
    C = 70
    A = torch.eye(4).repeat(C, 1, 1)
    q, _ = torch.linalg.qr(torch.randn(C, 3, 3, generator=g))
    A[:, :3, :3] = q
    A[:, :3, 3] = torch.randn(C, 3, generator=g) * 20
    A[C // 2:] = A[C // 2:] + torch.randn(C - C // 2, 4, 4, generator=g) * 0.1   # not rigid, last row not 0 0 0 1
    ref_in = A.double().requires_grad_(True)
    want = torch.inverse(ref_in)[:, :3, 3]
    got_in = A.to(DEV).requires_grad_(True)
    got = ops.camera_centers(got_in)
    np.testing.assert_allclose(n(got), want.detach().numpy(), rtol=2e-6, atol=2e-6)
    v = torch.randn(C, 3, generator=g, dtype=torch.float64)
    want.backward(v)
    got.backward(v.float().to(DEV))
    np.testing.assert_allclose(n(got_in.grad), ref_in.grad.numpy(), rtol=1e-4, atol=1e-4)
