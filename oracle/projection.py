"""CPU restatement (torch, any float dtype, differentiable) of the fused projections and of the
spherical-harmonics colour evaluation. TEST INFRASTRUCTURE ONLY - see ``oracle/__init__.py``.

Follows the reference CUDA kernels where they and the reference's torch restatement differ
(the kernels are what the product replaces):
  lidar projection   gsplat/cuda/csrc/projection.cu:2268-2417, utils.cuh:281-318, 12-31,
                     helpers.cuh:120-153      (torch twin: _torch_impl.py:120-165, 341-418)
  camera projection  gsplat/cuda/csrc/projection.cu:605-751, utils.cuh:190-217,
                     helpers.cuh:80-118       (torch twin: _torch_impl.py:54-101, 265-338)
  quat/scale -> cov  gsplat/cuda/csrc/utils.cuh:57-119 (torch twin: _torch_impl.py:10-51)
  SH                 gsplat/cuda/csrc/sh.cu:13-93      (torch twin: _torch_impl.py:1025-1117)

Culled (sensor, Gaussian) entries are returned as zeros, like the product does; gradients are
obtained with torch.autograd through these functions (radii are not differentiable).
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import Tensor

RAD_TO_DEG = 57.2957795131


def quat_scale_to_covar(quats: Tensor, scales: Tensor) -> Tensor:
    """[N,4] (w,x,y,z, unnormalised), [N,3] -> [N,3,3] covariance (R S)(R S)^T."""
    q = quats / quats.norm(dim=-1, keepdim=True)
    w, x, y, z = q.unbind(-1)
    R = torch.stack(
        [
            1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y),
            2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x),
            2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y),
        ],
        dim=-1,
    ).reshape(-1, 3, 3)
    M = R * scales[:, None, :]
    return M @ M.transpose(-1, -2)


def covar_from_triu(c: Tensor) -> Tensor:
    """[N,6] upper triangle -> [N,3,3] symmetric."""
    return torch.stack(
        [c[:, 0], c[:, 1], c[:, 2], c[:, 1], c[:, 3], c[:, 4], c[:, 2], c[:, 4], c[:, 5]], dim=-1
    ).reshape(-1, 3, 3)


def _world_to_sensor(means, covars, viewmats):
    R = viewmats[:, :3, :3]
    t = viewmats[:, :3, 3]
    p = torch.einsum("cij,nj->cni", R, means) + t[:, None, :]
    cov = torch.einsum("cij,njk,clk->cnil", R, covars, R)
    return p, cov, R


def _blur(cov2d, eps2d):
    det_orig = cov2d[..., 0, 0] * cov2d[..., 1, 1] - cov2d[..., 0, 1] * cov2d[..., 1, 0]
    a = cov2d[..., 0, 0] + eps2d
    d = cov2d[..., 1, 1] + eps2d
    b = cov2d[..., 0, 1]
    c = cov2d[..., 1, 0]
    det = a * d - b * c
    comp = torch.sqrt(torch.clamp(det_orig / det, min=0.0))
    return a, b, d, det, comp


def lidar_jacobian(p: Tensor) -> Tensor:
    """[...,3] sensor-frame point -> [...,3,3] Jacobian of (azimuth deg, elevation deg, range)."""
    x, y, z = p.unbind(-1)
    s2 = x * x + y * y
    r2 = s2 + z * z
    rinv = torch.rsqrt(r2)
    sxy = torch.sqrt(s2)
    k = 1.0 / r2 / sxy
    zero = torch.zeros_like(x)
    J = torch.stack(
        [
            -y / s2 * RAD_TO_DEG, x / s2 * RAD_TO_DEG, zero,
            -x * z * k * RAD_TO_DEG, -y * z * k * RAD_TO_DEG, sxy / r2 * RAD_TO_DEG,
            x * rinv, y * rinv, z * rinv,
        ],
        dim=-1,
    )
    return J.reshape(p.shape[:-1] + (3, 3))


def fully_fused_lidar_projection(
    means: Tensor, covars: Optional[Tensor], quats: Optional[Tensor], scales: Optional[Tensor],
    velocities: Optional[Tensor], viewmats: Tensor, linear_velocity: Tensor, angular_velocity: Tensor,
    rolling_shutter_time: Tensor, min_elevation: float = -45, max_elevation: float = 45,
    min_azimuth: float = -180, max_azimuth: float = 180, eps2d: float = 0.01,
    near_plane: float = 0.01, far_plane: float = 1e10, radius_clip: float = 0.0,
    calc_compensations: bool = False,
) -> Tuple[Tensor, Tensor, Tensor, Tensor, Optional[Tensor], Tensor, Tensor]:
    """Returns (radii [C,N,2], means2d, depths, conics, compensations|None, pix_vels [C,N,3],
    depth_compensations [C,N,2]); ``covars`` is [N,6] (upper triangle) or None."""
    cov_w = covar_from_triu(covars) if covars is not None else quat_scale_to_covar(quats, scales)
    p, cov_c, R = _world_to_sensor(means, cov_w, viewmats)
    C, N = p.shape[:2]
    dist = p.norm(dim=-1)
    valid = ~((dist < near_plane) | (dist > far_plane))

    # keep the maths finite for culled points so autograd stays clean
    p_safe = torch.where(valid[..., None], p, torch.tensor([1.0, 0.0, 0.0], dtype=p.dtype).expand_as(p))
    x, y, z = p_safe.unbind(-1)
    J = lidar_jacobian(p_safe)
    cov_s = J @ cov_c @ J.transpose(-1, -2)
    rinv = torch.rsqrt(x * x + y * y + z * z)
    means2d = torch.stack([torch.atan2(y, x), torch.asin(torch.clamp(z * rinv, -1.0, 1.0))], dim=-1) * RAD_TO_DEG

    a1 = cov_s[..., 0, 0] + eps2d
    a2 = cov_s[..., 0, 1]
    b1 = cov_s[..., 1, 0]
    b2 = cov_s[..., 1, 1] + eps2d
    c1 = cov_s[..., 2, 0]
    c2 = cov_s[..., 2, 1]
    invD = 1.0 / (a1 * b2 - a2 * b1)
    depth_comp = torch.stack([(b1 * c2 - b2 * c1) * invD, (a2 * c1 - a1 * c2) * invD], dim=-1)

    a, b, d, det, comp = _blur(cov_s[..., :2, :2], eps2d)
    valid = valid & (det > 0)
    det_safe = torch.where(det > 0, det, torch.ones_like(det))
    ex = 3.0 * torch.sqrt(torch.clamp(a, min=0.0))
    ey = 3.0 * torch.sqrt(torch.clamp(d, min=0.0))
    valid = valid & ~((ex <= radius_clip) & (ey <= radius_clip))

    rs = rolling_shutter_time.reshape(C, 1)
    if velocities is not None:
        vel_c = torch.einsum("cij,nj->cni", R, velocities)
    else:
        vel_c = torch.zeros_like(p)
    total = linear_velocity[:, None, :] + torch.cross(angular_velocity[:, None, :].expand_as(p_safe), p_safe, dim=-1) - vel_c
    pix_vel = -(J @ total[..., None])[..., 0]
    pix_vel = pix_vel * (rs > 0)[..., None]
    ex = ex + pix_vel[..., 0].abs() * 0.5 * rs * (rs > 0)
    ey = ey + pix_vel[..., 1].abs() * 0.5 * rs * (rs > 0)

    outside = (
        (means2d[..., 1] + ey <= min_elevation)
        | (means2d[..., 1] - ey >= max_elevation)
        | (means2d[..., 0] + ex <= min_azimuth)
        | (means2d[..., 0] - ex >= max_azimuth)
    )
    valid = valid & ~outside
    conics = torch.stack([d / det_safe, -b / det_safe, a / det_safe], dim=-1)

    m = valid
    zero = torch.zeros((), dtype=p.dtype)
    radii = torch.stack([ex, ey], dim=-1).detach() * m[..., None]
    out = (
        radii,
        torch.where(m[..., None], means2d, zero),
        torch.where(m, dist, zero),
        torch.where(m[..., None], conics, zero),
        torch.where(m, comp, zero) if calc_compensations else None,
        torch.where(m[..., None], pix_vel, zero),
        torch.where(m[..., None], depth_comp, zero),
    )
    return out


def persp_jacobian(p: Tensor, Ks: Tensor, width: int, height: int):
    """Returns (J [C,N,2,3], tx, ty) with the 0.3*tan(fov) clamp of x/z and y/z."""
    x, y, z = p.unbind(-1)
    fx = Ks[:, 0, 0, None]
    fy = Ks[:, 1, 1, None]
    cx = Ks[:, 0, 2, None]
    cy = Ks[:, 1, 2, None]
    tan_fovx = 0.5 * width / fx
    tan_fovy = 0.5 * height / fy
    lim_x_pos = (width - cx) / fx + 0.3 * tan_fovx
    lim_x_neg = cx / fx + 0.3 * tan_fovx
    lim_y_pos = (height - cy) / fy + 0.3 * tan_fovy
    lim_y_neg = cy / fy + 0.3 * tan_fovy
    rz = 1.0 / z
    tx = z * torch.minimum(lim_x_pos.expand_as(x), torch.maximum(-lim_x_neg.expand_as(x), x * rz))
    ty = z * torch.minimum(lim_y_pos.expand_as(y), torch.maximum(-lim_y_neg.expand_as(y), y * rz))
    zero = torch.zeros_like(x)
    J = torch.stack([fx * rz, zero, -fx * tx * rz * rz, zero, fy * rz, -fy * ty * rz * rz], dim=-1)
    return J.reshape(p.shape[:-1] + (2, 3))


def fully_fused_projection(
    means: Tensor, covars: Optional[Tensor], quats: Optional[Tensor], scales: Optional[Tensor],
    velocities: Optional[Tensor], viewmats: Tensor, Ks: Tensor, width: int, height: int,
    linear_velocity: Tensor, angular_velocity: Tensor, rolling_shutter_time: Tensor,
    eps2d: float = 0.3, near_plane: float = 0.01, far_plane: float = 1e10, radius_clip: float = 0.0,
    calc_compensations: bool = False,
) -> Tuple[Tensor, Tensor, Tensor, Tensor, Optional[Tensor], Tensor]:
    """Returns (radii [C,N,2] int32, means2d, depths, conics, compensations|None, pix_vels [C,N,2])."""
    cov_w = covar_from_triu(covars) if covars is not None else quat_scale_to_covar(quats, scales)
    p, cov_c, R = _world_to_sensor(means, cov_w, viewmats)
    C, N = p.shape[:2]
    valid = ~((p[..., 2] < near_plane) | (p[..., 2] > far_plane))
    p_safe = torch.where(valid[..., None], p, torch.tensor([0.0, 0.0, 1.0], dtype=p.dtype).expand_as(p))
    x, y, z = p_safe.unbind(-1)
    J = persp_jacobian(p_safe, Ks, width, height)
    cov2d = J @ cov_c @ J.transpose(-1, -2)
    fx = Ks[:, 0, 0, None]
    fy = Ks[:, 1, 1, None]
    cx = Ks[:, 0, 2, None]
    cy = Ks[:, 1, 2, None]
    means2d = torch.stack([fx * x / z + cx, fy * y / z + cy], dim=-1)
    a, b, d, det, comp = _blur(cov2d, eps2d)
    valid = valid & (det > 0)
    det_safe = torch.where(det > 0, det, torch.ones_like(det))
    ex = 3.0 * torch.sqrt(torch.clamp(a, min=0.0))
    ey = 3.0 * torch.sqrt(torch.clamp(d, min=0.0))
    valid = valid & ~((ex <= radius_clip) & (ey <= radius_clip))

    rs = rolling_shutter_time.reshape(C, 1)
    if velocities is not None:
        vel_c = torch.einsum("cij,nj->cni", R, velocities)
    else:
        vel_c = torch.zeros_like(p)
    total = linear_velocity[:, None, :] + torch.cross(angular_velocity[:, None, :].expand_as(p_safe), p_safe, dim=-1) - vel_c
    pix_vel = -(J @ total[..., None])[..., 0]
    pix_vel = pix_vel * (rs > 0)[..., None]
    ex = ex + pix_vel[..., 0].abs() * 0.5 * rs * (rs > 0)
    ey = ey + pix_vel[..., 1].abs() * 0.5 * rs * (rs > 0)
    outside = (
        (means2d[..., 0] + ex <= 0) | (means2d[..., 0] - ex >= width)
        | (means2d[..., 1] + ey <= 0) | (means2d[..., 1] - ey >= height)
    )
    valid = valid & ~outside
    conics = torch.stack([d / det_safe, -b / det_safe, a / det_safe], dim=-1)
    m = valid
    zero = torch.zeros((), dtype=p.dtype)
    radii = (torch.stack([ex, ey], dim=-1).detach() * m[..., None]).to(torch.int32)
    return (
        radii,
        torch.where(m[..., None], means2d, zero),
        torch.where(m, p[..., 2], zero),
        torch.where(m[..., None], conics, zero),
        torch.where(m, comp, zero) if calc_compensations else None,
        torch.where(m[..., None], pix_vel, zero),
    )


def pack_projection(radii, means2d, depths, conics, compensations, pix_vels):
    """[C,N,..] camera projection -> packed rows (camera-major, Gaussian-minor) of the visible
    pairs, like gsplat/cuda/csrc/projection.cu:1300-1351. A pair is visible when it survived
    every cull (its conic is non-zero), even if its integer radius truncated to 0."""
    vis = conics.abs().sum(-1) > 0
    cam, gau = torch.nonzero(vis, as_tuple=True)
    comp = compensations[cam, gau] if compensations is not None else None
    return (cam, gau, radii[cam, gau], means2d[cam, gau], depths[cam, gau], conics[cam, gau], comp,
            pix_vels[cam, gau])


# ---------------------------------------------------------------------------------------------
# Spherical harmonics (degree 0..4)
# ---------------------------------------------------------------------------------------------
def sh_bases(degree: int, dirs: Tensor) -> Tensor:
    """[...,3] unit directions -> [..., (degree+1)^2] real SH basis values."""
    x, y, z = dirs.unbind(-1)
    b = [torch.full_like(x, 0.2820947917738781)]
    if degree >= 1:
        b += [-0.48860251190292 * y, 0.48860251190292 * z, -0.48860251190292 * x]
    if degree >= 2:
        z2 = z * z
        fTmp0B = -1.092548430592079 * z
        fC1 = x * x - y * y
        fS1 = 2 * x * y
        pSH6 = 0.9461746957575601 * z2 - 0.3153915652525201
        b += [0.5462742152960395 * fS1, fTmp0B * y, pSH6, fTmp0B * x, 0.5462742152960395 * fC1]
    if degree >= 3:
        fTmp0C = -2.285228997322329 * z2 + 0.4570457994644658
        fTmp1B = 1.445305721320277 * z
        fC2 = x * fC1 - y * fS1
        fS2 = x * fS1 + y * fC1
        pSH12 = z * (1.865881662950577 * z2 - 1.119528997770346)
        b += [-0.5900435899266435 * fS2, fTmp1B * fS1, fTmp0C * y, pSH12, fTmp0C * x, fTmp1B * fC1,
              -0.5900435899266435 * fC2]
    if degree >= 4:
        fTmp0D = z * (-4.683325804901025 * z2 + 2.007139630671868)
        fTmp1C = 3.31161143515146 * z2 - 0.47308734787878
        fTmp2B = -1.770130769779931 * z
        fC3 = x * fC2 - y * fS2
        fS3 = x * fS2 + y * fC2
        pSH20 = 1.984313483298443 * z * pSH12 - 1.006230589874905 * pSH6
        b += [0.6258357354491763 * fS3, fTmp2B * fS2, fTmp1C * fS1, fTmp0D * y, pSH20, fTmp0D * x,
              fTmp1C * fC1, fTmp2B * fC2, 0.6258357354491763 * fC3]
    return torch.stack(b, dim=-1)


def spherical_harmonics(degree: int, dirs: Tensor, coeffs: Tensor, masks: Optional[Tensor] = None) -> Tensor:
    """dirs [...,3] (unnormalised), coeffs [...,K,3] -> colours [...,3]; masked rows are zero."""
    n = dirs / dirs.norm(dim=-1, keepdim=True)
    nb = (degree + 1) ** 2
    bases = sh_bases(degree, n)
    out = (bases[..., None] * coeffs[..., :nb, :]).sum(dim=-2)
    if masks is not None:
        out = out * masks[..., None]
    return out


# ---------------------------------------------------------------------------------------------
# The unfused ops (torch twins in gsplat/cuda/_torch_impl.py:10-262), differentiable.
# ---------------------------------------------------------------------------------------------
def _triu(m: Tensor) -> Tensor:
    return torch.stack([m[..., 0, 0], m[..., 0, 1], m[..., 0, 2], m[..., 1, 1], m[..., 1, 2], m[..., 2, 2]], dim=-1)


def quat_scale_to_covar_preci(quats: Tensor, scales: Tensor, compute_covar: bool = True,
                              compute_preci: bool = True, triu: bool = False):
    """gsplat/cuda/_torch_impl.py:10-51: covariance (R S)(R S)^T and precision (R / S)(R / S)^T."""
    covars = quat_scale_to_covar(quats, scales) if compute_covar else None
    precis = quat_scale_to_covar(quats, 1.0 / scales) if compute_preci else None
    if triu:
        covars = _triu(covars) if covars is not None else None
        precis = _triu(precis) if precis is not None else None
    return covars, precis


def world_to_cam(means: Tensor, covars: Tensor, viewmats: Tensor) -> Tuple[Tensor, Tensor]:
    """gsplat/cuda/_torch_impl.py:168-190."""
    p, cov, _ = _world_to_sensor(means, covars, viewmats)
    return p, cov


def persp_proj(means: Tensor, covars: Tensor, Ks: Tensor, width: int, height: int) -> Tuple[Tensor, Tensor]:
    """gsplat/cuda/_torch_impl.py:54-101: sensor-frame Gaussians -> pixel means and 2x2 covariances."""
    J = persp_jacobian(means, Ks, width, height)
    cov2d = J @ covars @ J.transpose(-1, -2)
    x, y, z = means.unbind(-1)
    fx, fy, cx, cy = Ks[:, 0, 0, None], Ks[:, 1, 1, None], Ks[:, 0, 2, None], Ks[:, 1, 2, None]
    return torch.stack([fx * x / z + cx, fy * y / z + cy], dim=-1), cov2d


def compute_pix_velocity(p_view: Tensor, lin_vel: Tensor, ang_vel: Tensor, velocities: Tensor, Ks: Tensor,
                         width: int, height: int) -> Tensor:
    """gsplat/cuda/_torch_impl.py:193-224: -J (lin + ang x p - v)."""
    J = persp_jacobian(p_view, Ks, width, height)
    total = lin_vel[:, None, :] + torch.cross(ang_vel[:, None, :].expand_as(p_view), p_view, dim=-1) - velocities
    return -(J @ total[..., None])[..., 0]


def lidar_proj(means: Tensor, covars: Tensor, eps2d: float) -> Tuple[Tensor, Tensor, Tensor]:
    """gsplat/cuda/_torch_impl.py:104-165: (azimuth, elevation) in degrees, their 2x2 covariance
    (no blur added) and the depth compensation."""
    J = lidar_jacobian(means)
    cov_s = J @ covars @ J.transpose(-1, -2)
    x, y, z = means.unbind(-1)
    rinv = torch.rsqrt(x * x + y * y + z * z)
    means2d = torch.stack([torch.atan2(y, x), torch.asin(z * rinv)], dim=-1) * RAD_TO_DEG
    a1, a2 = cov_s[..., 0, 0] + eps2d, cov_s[..., 0, 1]
    b1, b2 = cov_s[..., 1, 0], cov_s[..., 1, 1] + eps2d
    c1, c2 = cov_s[..., 2, 0], cov_s[..., 2, 1]
    invD = 1.0 / (a1 * b2 - a2 * b1)
    depth_comp = torch.stack([(b1 * c2 - b2 * c1) * invD, (a2 * c1 - a1 * c2) * invD], dim=-1)
    return means2d, cov_s[..., :2, :2], depth_comp


def compute_lidar_velocity(p_view: Tensor, lin_vel: Tensor, ang_vel: Tensor, velocities: Tensor) -> Tensor:
    """gsplat/cuda/_torch_impl.py:227-262: -J (lin + ang x p - v) with the spherical Jacobian."""
    J = lidar_jacobian(p_view)
    total = lin_vel[:, None, :] + torch.cross(ang_vel[:, None, :].expand_as(p_view), p_view, dim=-1) - velocities
    return -(J @ total[..., None])[..., 0]
