"""Op-level API of the render hot path: same function names, argument order, defaults, return
tuples and gradient slots as ``gsplat/cuda/_wrapper.py`` of the reference, implemented on top
of the C-ABI CUDA library (``include/splatad_b200.h``).

Reference functions mirrored here (file:line in carlinds/splatad):
  spherical_harmonics            gsplat/cuda/_wrapper.py:17-43    (_SphericalHarmonics 2321-2351)
  fully_fused_projection         gsplat/cuda/_wrapper.py:230-387  (_FullyFusedProjection 1495-1640,
                                                                   _FullyFusedProjectionPacked 2107-2319)
  fully_fused_lidar_projection   gsplat/cuda/_wrapper.py:390-530  (_FullyFusedLidarProjection 1642-1794)
  isect_tiles                    gsplat/cuda/_wrapper.py:532-603
  isect_lidar_tiles              gsplat/cuda/_wrapper.py:605-676
  isect_offset_encode            gsplat/cuda/_wrapper.py:679-696
  rasterize_to_pixels            gsplat/cuda/_wrapper.py:811-949  (_RasterizeToPixels 1796-1930)
  rasterize_to_points            gsplat/cuda/_wrapper.py:951-1111 (_RasterizeToPoints 1932-2105)
  rasterize_to_indices_in_range  gsplat/cuda/_wrapper.py:1115-1196 (lidar twin 1198-1281)

Differences that are visible to a caller:
  * entries of culled (sensor, Gaussian) pairs are zero instead of uninitialised memory;
  * the fused projection backward can return the gradient of ``velocities`` (the reference
    computes it and throws it away); off by default, see ``velocity_grads``.
"""

from __future__ import annotations

import contextlib
import ctypes
import struct
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _lib

_RETURN_VELOCITY_GRADS = False
# (C, N, device, stream) -> packed row count of the last frame of that shape rendered on that stream.
# A hint only sizes the room a frame is given (too small -> the frame is redone), and a stream's
# frames are issued by one thread at a time, so streams never share or fight over an entry.
_packed_nnz_hint = {}


@contextlib.contextmanager
def velocity_grads(enabled: bool = True):
    """Within this context the fused projections also return d(loss)/d(velocities).

    The reference's fused backward kernels compute this gradient into a local variable and drop
    it (gsplat/cuda/csrc/projection.cu:874-877, 2538-2541), and its autograd functions return
    ``None`` for ``velocities``; that stays the default here.
    """
    global _RETURN_VELOCITY_GRADS
    prev = _RETURN_VELOCITY_GRADS
    _RETURN_VELOCITY_GRADS = enabled
    try:
        yield
    finally:
        _RETURN_VELOCITY_GRADS = prev


def _f(t: Optional[Tensor]) -> Optional[Tensor]:
    if t is None:
        return None
    if t.dtype != torch.float32:
        t = t.float()
    return t.contiguous()


_call = _lib.call   # device-guarded: see _lib.call


# =============================================================================================
# Spherical harmonics
# =============================================================================================
def spherical_harmonics(
    degrees_to_use: int,
    dirs: Tensor,  # [..., 3]
    coeffs: Tensor,  # [..., K, 3]
    masks: Optional[Tensor] = None,
) -> Tensor:
    """Computes spherical harmonics colours. Returns [..., 3]."""
    assert (degrees_to_use + 1) ** 2 <= coeffs.shape[-2], coeffs.shape
    assert dirs.shape[:-1] == coeffs.shape[:-2], (dirs.shape, coeffs.shape)
    assert dirs.shape[-1] == 3, dirs.shape
    assert coeffs.shape[-1] == 3, coeffs.shape
    if masks is not None:
        assert masks.shape == dirs.shape[:-1], masks.shape
        masks = masks.contiguous()
    return _SphericalHarmonics.apply(degrees_to_use, dirs.contiguous(), coeffs.contiguous(), masks)


class _SphericalHarmonics(torch.autograd.Function):
    @staticmethod
    def forward(ctx, sh_degree: int, dirs: Tensor, coeffs: Tensor, masks: Optional[Tensor]) -> Tensor:
        dirs = _f(dirs)
        coeffs = _f(coeffs)
        if masks is not None:
            masks = masks.to(torch.bool).contiguous()
        n = dirs.numel() // 3
        K = coeffs.shape[-2]
        colors = torch.empty_like(dirs)
        _call(
            "splatad_sh_fwd", n, K, sh_degree, _lib.ptr(dirs), _lib.ptr(coeffs), _lib.ptr(masks),
            _lib.ptr(colors), _lib.stream_ptr(dirs.device),
        )
        ctx.save_for_backward(dirs, coeffs, masks)
        ctx.sh_degree = sh_degree
        return colors

    @staticmethod
    def backward(ctx, v_colors: Tensor):
        dirs, coeffs, masks = ctx.saved_tensors
        n = dirs.numel() // 3
        K = coeffs.shape[-2]
        compute_v_dirs = ctx.needs_input_grad[1]
        v_coeffs = torch.empty_like(coeffs)
        v_dirs = torch.empty_like(dirs) if compute_v_dirs else None
        _call(
            "splatad_sh_bwd", n, K, ctx.sh_degree, _lib.ptr(dirs), _lib.ptr(coeffs), _lib.ptr(masks),
            _lib.ptr(_f(v_colors)), _lib.ptr(v_coeffs), _lib.ptr(v_dirs), _lib.stream_ptr(dirs.device),
        )
        return None, v_dirs, v_coeffs, None


def gather_rows(table: Tensor, ids: Tensor) -> Tensor:
    """``table[ids]`` along the first axis, with a backward pass that adds the gradient rows into a
    zero tensor with atomics (``index_add_``). torch's own backward of advanced indexing sorts the
    indices first, which takes 9.7 ms for the 350 k packed rows of a 500 k-Gaussian camera frame -
    three quarters of that frame's training step."""
    return _GatherRows.apply(table, ids)


class _GatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, table, ids):
        ctx.save_for_backward(ids)
        ctx.rows = table.shape[0]
        return table.index_select(0, ids)

    @staticmethod
    def backward(ctx, v_out):
        (ids,) = ctx.saved_tensors
        v_table = torch.zeros((ctx.rows,) + tuple(v_out.shape[1:]), dtype=v_out.dtype, device=v_out.device)
        v_table.index_add_(0, ids, v_out.contiguous())
        return v_table, None


def camera_centers(viewmats: Tensor) -> Tensor:
    """Camera centres in world coordinates, ``torch.inverse(viewmats)[:, :3, 3]`` ([C, 3]) from one
    tiny kernel (cofactors in double precision) instead of a batched LU with its error-check round
    trip to the host; differentiable with respect to ``viewmats``."""
    assert viewmats.dim() == 3 and viewmats.shape[1:] == (4, 4), viewmats.shape
    return _CameraCenters.apply(viewmats)


class _CameraCenters(torch.autograd.Function):
    @staticmethod
    def forward(ctx, viewmats):
        viewmats = _f(viewmats)
        campos = torch.empty((viewmats.shape[0], 3), dtype=torch.float32, device=viewmats.device)
        _call("splatad_camera_centers", viewmats.shape[0], _lib.ptr(viewmats), _lib.ptr(campos),
              _lib.stream_ptr(viewmats.device))
        ctx.save_for_backward(viewmats)
        return campos

    @staticmethod
    def backward(ctx, v_campos):
        # Y = A^-1: dA = -Y^T dY Y^T with dY zero except for its translation column
        (viewmats,) = ctx.saved_tensors
        inv = torch.linalg.inv_ex(viewmats).inverse
        v_inv = torch.zeros_like(viewmats)
        v_inv[:, :3, 3] = v_campos
        return -inv.transpose(1, 2) @ v_inv @ inv.transpose(1, 2)


def view_dependent_colors(
    sh_degree: int,
    means: Tensor,  # [N, 3]
    campos: Tensor,  # [C, 3] camera centres in world coordinates
    coeffs: Tensor,  # [N, K, 3] or [C, N, K, 3]
    radii: Tensor,  # [C, N, 2] or [nnz, 2]
    camera_ids: Optional[Tensor] = None,  # [nnz] (packed layout)
    gaussian_ids: Optional[Tensor] = None,  # [nnz]
    depths: Optional[Tensor] = None,  # [C, N] or [nnz]: appended as a fourth channel
) -> Tensor:
    """Colours of the projected Gaussians seen from their cameras, ``clamp_min(SH(dirs) + 0.5, 0)``
    with ``dirs = means - camera centre``, in one kernel; with ``depths`` the result carries the
    depth as last channel. This is the chain of gathers and elementwise torch ops around the SH
    kernel in the reference's ``rasterization()`` (gsplat/rendering.py:345-373, 383-384) - same
    values, same gradients (means, campos, coeffs, depths) - without materialising the gathered
    ``[nnz, K, 3]`` coefficients. Returns [C, N, 3|4] or [nnz, 3|4]."""
    N = means.shape[0]
    assert means.shape == (N, 3), means.shape
    C = campos.shape[0]
    assert campos.shape == (C, 3), campos.shape
    assert coeffs.shape[-1] == 3 and (sh_degree + 1) ** 2 <= coeffs.shape[-2], coeffs.shape
    assert (coeffs.dim() == 3 and coeffs.shape[0] == N) or (coeffs.dim() == 4 and coeffs.shape[:2] == (C, N)), \
        coeffs.shape
    packed = gaussian_ids is not None
    if packed:
        assert camera_ids is not None and radii.shape == (gaussian_ids.numel(), 2), radii.shape
    else:
        assert radii.shape == (C, N, 2), radii.shape
    if depths is not None:
        assert depths.shape == radii.shape[:-1], depths.shape
    return _ViewDependentColors.apply(sh_degree, means, campos, coeffs, depths, radii, camera_ids, gaussian_ids)


class _ViewDependentColors(torch.autograd.Function):
    @staticmethod
    def forward(ctx, sh_degree, means, campos, coeffs, depths, radii, camera_ids, gaussian_ids):
        means, campos, coeffs = _f(means), _f(campos), _f(coeffs)
        depths = _f(depths)
        radii = radii.to(torch.int32).contiguous()
        if gaussian_ids is not None:
            camera_ids = camera_ids.to(torch.int64).contiguous()
            gaussian_ids = gaussian_ids.to(torch.int64).contiguous()
        N, K = means.shape[0], coeffs.shape[-2]
        out_ch = 3 if depths is None else 4
        colors = torch.empty(radii.shape[:-1] + (out_ch,), dtype=torch.float32, device=means.device)
        n_elems = radii.numel() // 2
        _call("splatad_sh_colors_fwd", n_elems, N, K, sh_degree, _lib.ptr(means), _lib.ptr(campos),
              _lib.ptr(coeffs), int(coeffs.dim() == 4), _lib.ptr(camera_ids), _lib.ptr(gaussian_ids),
              _lib.ptr(radii), _lib.ptr(depths), out_ch, _lib.ptr(colors), _lib.stream_ptr(means.device))
        ctx.save_for_backward(means, campos, coeffs, radii, camera_ids, gaussian_ids)
        ctx.sh_degree, ctx.out_ch = sh_degree, out_ch
        return colors

    @staticmethod
    def backward(ctx, v_colors):
        means, campos, coeffs, radii, camera_ids, gaussian_ids = ctx.saved_tensors
        N, K = means.shape[0], coeffs.shape[-2]
        need_means, need_campos, need_coeffs, need_depths = ctx.needs_input_grad[1:5]
        v_means = torch.zeros_like(means) if need_means else None
        v_campos = torch.zeros_like(campos) if need_campos else None
        v_coeffs = torch.zeros_like(coeffs) if need_coeffs else None
        v_depths = (torch.empty(radii.shape[:-1], dtype=torch.float32, device=means.device)
                    if (need_depths and ctx.out_ch == 4) else None)
        _call("splatad_sh_colors_bwd", radii.numel() // 2, N, K, ctx.sh_degree, _lib.ptr(means),
              _lib.ptr(campos), _lib.ptr(coeffs), int(coeffs.dim() == 4), _lib.ptr(camera_ids),
              _lib.ptr(gaussian_ids), _lib.ptr(radii), ctx.out_ch, _lib.ptr(_f(v_colors)), _lib.ptr(v_coeffs),
              _lib.ptr(v_means), _lib.ptr(v_campos), _lib.ptr(v_depths), _lib.stream_ptr(means.device))
        return None, v_means, v_campos, v_coeffs, v_depths, None, None, None


# =============================================================================================
# Projection
# =============================================================================================
def fully_fused_projection(
    means: Tensor,  # [N, 3]
    covars: Optional[Tensor],  # [N, 6] or None
    quats: Optional[Tensor],  # [N, 4] or None
    scales: Optional[Tensor],  # [N, 3] or None
    velocities: Optional[Tensor],  # [N, 3] or None
    viewmats: Tensor,  # [C, 4, 4]
    Ks: Tensor,  # [C, 3, 3]
    width: int,
    height: int,
    linear_velocity: Tensor,  # [C, 3]
    angular_velocity: Tensor,  # [C, 3]
    rolling_shutter_time: Tensor,  # [C]
    eps2d: float = 0.3,
    near_plane: float = 0.01,
    far_plane: float = 1e10,
    radius_clip: float = 0.0,
    packed: bool = False,
    sparse_grad: bool = False,
    calc_compensations: bool = False,
    pending: Optional["PendingPackedCount"] = None,
):
    """Projects Gaussians to a batch of pinhole cameras (with rolling-shutter velocities).

    packed=False returns (radii [C,N,2] int32, means2d, depths, conics, compensations, pix_vels);
    packed=True returns (camera_ids, gaussian_ids, radii [nnz,2], means2d, depths, conics,
    compensations, pix_vels) with rows ordered camera-major, Gaussian-minor.

    ``pending`` (not in the reference, packed only): a :class:`PendingPackedCount` that lets the call
    return without waiting for the row count; see there.
    """
    C = viewmats.size(0)
    N = means.size(0)
    assert means.size() == (N, 3), means.size()
    assert viewmats.size() == (C, 4, 4), viewmats.size()
    assert Ks.size() == (C, 3, 3), Ks.size()
    assert linear_velocity.size() == (C, 3), linear_velocity.size()
    assert angular_velocity.size() == (C, 3), angular_velocity.size()
    assert rolling_shutter_time.size() == (C,), rolling_shutter_time.size()
    means = means.contiguous()
    if covars is not None:
        assert covars.size() == (N, 6), covars.size()
        covars = covars.contiguous()
    else:
        assert quats is not None, "covars or quats is required"
        assert scales is not None, "covars or scales is required"
        assert quats.size() == (N, 4), quats.size()
        assert scales.size() == (N, 3), scales.size()
        quats = quats.contiguous()
        scales = scales.contiguous()
    if velocities is not None:
        assert velocities.size() == (N, 3), velocities.size()
        velocities = velocities.contiguous()
    if sparse_grad:
        assert packed, "sparse_grad is only supported when packed is True"
    viewmats = viewmats.contiguous()
    Ks = Ks.contiguous()
    if packed:
        return _FullyFusedProjectionPacked.apply(
            means, covars, quats, scales, velocities, viewmats, Ks, width, height, linear_velocity,
            angular_velocity, rolling_shutter_time, eps2d, near_plane, far_plane, radius_clip,
            sparse_grad, calc_compensations, pending,
        )
    return _FullyFusedProjection.apply(
        means, covars, quats, scales, velocities, viewmats, Ks, width, height, linear_velocity,
        angular_velocity, rolling_shutter_time, eps2d, near_plane, far_plane, radius_clip,
        calc_compensations,
    )


def fully_fused_lidar_projection(
    means: Tensor,  # [N, 3]
    covars: Optional[Tensor],  # [N, 6] or None
    quats: Optional[Tensor],  # [N, 4] or None
    scales: Optional[Tensor],  # [N, 3] or None
    velocities: Optional[Tensor],  # [N, 3] or None
    viewmats: Tensor,  # [C, 4, 4]
    linear_velocity: Tensor,  # [C, 3]
    angular_velocity: Tensor,  # [C, 3]
    rolling_shutter_time: Tensor,  # [C]
    min_elevation: float = -45,
    max_elevation: float = 45,
    min_azimuth: float = -180,
    max_azimuth: float = 180,
    eps2d: float = 0.01,
    near_plane: float = 0.01,
    far_plane: float = 1e10,
    radius_clip: float = 0.0,
    packed: bool = False,
    sparse_grad: bool = False,
    calc_compensations: bool = False,
    frame: Optional["LidarFrame"] = None,
):
    """Projects Gaussians to a batch of spherical lidars (azimuth / elevation in degrees, range).

    Returns (radii [C,N,2] float degrees, means2d, depths (range), conics, compensations,
    pix_vels [C,N,3], depth_compensations [C,N,2]).

    ``frame`` (not part of the reference's API): a :class:`LidarFrame` that has already projected
    exactly these inputs; its outputs are returned with this op's backward attached and nothing is
    launched.
    """
    C = viewmats.size(0)
    N = means.size(0)
    assert means.size() == (N, 3), means.size()
    assert viewmats.size() == (C, 4, 4), viewmats.size()
    means = means.contiguous()
    if covars is not None:
        assert covars.size() == (N, 6), covars.size()
        covars = covars.contiguous()
    else:
        assert quats is not None, "covars or quats is required"
        assert scales is not None, "covars or scales is required"
        assert quats.size() == (N, 4), quats.size()
        assert scales.size() == (N, 3), scales.size()
        quats = quats.contiguous()
        scales = scales.contiguous()
    if velocities is not None:
        assert velocities.size() == (N, 3), velocities.size()
        velocities = velocities.contiguous()
    if sparse_grad:
        assert packed, "sparse_grad is only supported when packed is True"
    viewmats = viewmats.contiguous()
    if packed:
        raise NotImplementedError("FullyFusedLidarProjectionPacked is not implemented yet")
    return _FullyFusedLidarProjection.apply(
        means, covars, quats, scales, velocities, viewmats, min_elevation, max_elevation,
        min_azimuth, max_azimuth, linear_velocity, angular_velocity, rolling_shutter_time, eps2d,
        near_plane, far_plane, radius_clip, calc_compensations, frame,
    )


def _proj_inputs(means, covars, quats, scales, velocities, viewmats, lin, ang, rs):
    return (_f(means), _f(covars), _f(quats), _f(scales), _f(velocities), _f(viewmats), _f(lin),
            _f(ang), _f(rs))


class _FullyFusedProjection(torch.autograd.Function):
    @staticmethod
    def forward(ctx, means, covars, quats, scales, velocities, viewmats, Ks, width, height,
                linear_velocity, angular_velocity, rolling_shutter_time, eps2d, near_plane,
                far_plane, radius_clip, calc_compensations):
        means, covars, quats, scales, velocities, viewmats, lin, ang, rs = _proj_inputs(
            means, covars, quats, scales, velocities, viewmats, linear_velocity, angular_velocity,
            rolling_shutter_time)
        Ks = _f(Ks)
        C, N = viewmats.shape[0], means.shape[0]
        dev = means.device
        radii = torch.empty((C, N, 2), dtype=torch.int32, device=dev)
        means2d = torch.empty((C, N, 2), dtype=torch.float32, device=dev)
        depths = torch.empty((C, N), dtype=torch.float32, device=dev)
        conics = torch.empty((C, N, 3), dtype=torch.float32, device=dev)
        pix_vels = torch.empty((C, N, 2), dtype=torch.float32, device=dev)
        compensations = torch.empty((C, N), dtype=torch.float32, device=dev) if calc_compensations else None
        _call(
            "splatad_projection_fwd", C, N, _lib.ptr(means), _lib.ptr(covars), _lib.ptr(quats),
            _lib.ptr(scales), _lib.ptr(velocities), _lib.ptr(viewmats), _lib.ptr(Ks), width, height,
            _lib.ptr(lin), _lib.ptr(ang), _lib.ptr(rs), eps2d, near_plane, far_plane, radius_clip,
            _lib.ptr(radii), _lib.ptr(means2d), _lib.ptr(depths), _lib.ptr(conics),
            _lib.ptr(compensations), _lib.ptr(pix_vels), _lib.stream_ptr(dev),
        )
        ctx.save_for_backward(means, covars, quats, scales, velocities, viewmats, Ks, lin, ang, rs,
                              radii, conics, compensations)
        ctx.width, ctx.height, ctx.eps2d = width, height, eps2d
        ctx.want_vel = _RETURN_VELOCITY_GRADS
        ctx.mark_non_differentiable(radii)
        return radii, means2d, depths, conics, compensations, pix_vels

    @staticmethod
    def backward(ctx, v_radii, v_means2d, v_depths, v_conics, v_compensations, v_pix_vels):
        (means, covars, quats, scales, velocities, viewmats, Ks, lin, ang, rs, radii, conics,
         compensations) = ctx.saved_tensors
        C, N = viewmats.shape[0], means.shape[0]
        dev = means.device
        v_means = torch.empty_like(means)
        v_covars = torch.empty_like(covars) if covars is not None else None
        v_quats = torch.empty_like(quats) if covars is None else None
        v_scales = torch.empty_like(scales) if covars is None else None
        v_viewmats = torch.zeros_like(viewmats) if ctx.needs_input_grad[5] else None
        want_vel = ctx.want_vel and velocities is not None and ctx.needs_input_grad[4]
        v_vel = torch.empty_like(velocities) if want_vel else None
        _call(
            "splatad_projection_bwd", C, N, _lib.ptr(means), _lib.ptr(covars), _lib.ptr(quats),
            _lib.ptr(scales), _lib.ptr(velocities), _lib.ptr(viewmats), _lib.ptr(Ks), ctx.width,
            ctx.height, _lib.ptr(lin), _lib.ptr(ang), _lib.ptr(rs), ctx.eps2d, _lib.ptr(radii),
            _lib.ptr(conics), _lib.ptr(compensations), _lib.ptr(_f(v_means2d)), _lib.ptr(_f(v_depths)),
            _lib.ptr(_f(v_conics)),
            _lib.ptr(_f(v_compensations)) if compensations is not None else None,
            _lib.ptr(_f(v_pix_vels)), _lib.ptr(v_means), _lib.ptr(v_covars), _lib.ptr(v_quats),
            _lib.ptr(v_scales), _lib.ptr(v_viewmats), _lib.ptr(v_vel), _lib.stream_ptr(dev),
        )
        if not ctx.needs_input_grad[0]:
            v_means = None
        if not ctx.needs_input_grad[1]:
            v_covars = None
        if not ctx.needs_input_grad[2]:
            v_quats = None
        if not ctx.needs_input_grad[3]:
            v_scales = None
        return (v_means, v_covars, v_quats, v_scales, v_vel, v_viewmats) + (None,) * 11


class _FullyFusedLidarProjection(torch.autograd.Function):
    @staticmethod
    def forward(ctx, means, covars, quats, scales, velocities, viewmats, min_elevation,
                max_elevation, min_azimuth, max_azimuth, linear_velocity, angular_velocity,
                rolling_shutter_time, eps2d, near_plane, far_plane, radius_clip, calc_compensations,
                frame=None):
        means, covars, quats, scales, velocities, viewmats, lin, ang, rs = _proj_inputs(
            means, covars, quats, scales, velocities, viewmats, linear_velocity, angular_velocity,
            rolling_shutter_time)
        C, N = viewmats.shape[0], means.shape[0]
        dev = means.device
        f32 = dict(dtype=torch.float32, device=dev)
        if frame is not None:
            # projected by the single-call frame already: only the graph node is made here
            assert not calc_compensations and covars is None and frame.radii.shape == (C, N, 2)
            radii, means2d, depths, conics = frame.radii, frame.means2d, frame.depths, frame.conics
            pix_vels, depth_comps, compensations = frame.pix_vels, frame.depth_compensations, None
        else:
            radii = torch.empty((C, N, 2), **f32)
            means2d = torch.empty((C, N, 2), **f32)
            depths = torch.empty((C, N), **f32)
            conics = torch.empty((C, N, 3), **f32)
            pix_vels = torch.empty((C, N, 3), **f32)
            depth_comps = torch.empty((C, N, 2), **f32)
            compensations = torch.empty((C, N), **f32) if calc_compensations else None
            _call(
                "splatad_lidar_projection_fwd", C, N, _lib.ptr(means), _lib.ptr(covars), _lib.ptr(quats),
                _lib.ptr(scales), _lib.ptr(velocities), _lib.ptr(viewmats), min_elevation, max_elevation,
                min_azimuth, max_azimuth, _lib.ptr(lin), _lib.ptr(ang), _lib.ptr(rs), eps2d, near_plane,
                far_plane, radius_clip, _lib.ptr(radii), _lib.ptr(means2d), _lib.ptr(depths),
                _lib.ptr(conics), _lib.ptr(compensations), _lib.ptr(pix_vels), _lib.ptr(depth_comps),
                _lib.stream_ptr(dev),
            )
        ctx.save_for_backward(means, covars, quats, scales, velocities, viewmats, lin, ang, rs, radii,
                              conics, compensations)
        ctx.eps2d = eps2d
        ctx.want_vel = _RETURN_VELOCITY_GRADS
        ctx.mark_non_differentiable(radii)
        return radii, means2d, depths, conics, compensations, pix_vels, depth_comps

    @staticmethod
    def backward(ctx, v_radii, v_means2d, v_depths, v_conics, v_compensations, v_pix_vels,
                 v_depth_comps):
        (means, covars, quats, scales, velocities, viewmats, lin, ang, rs, radii, conics,
         compensations) = ctx.saved_tensors
        C, N = viewmats.shape[0], means.shape[0]
        dev = means.device
        v_means = torch.empty_like(means)
        v_covars = torch.empty_like(covars) if covars is not None else None
        v_quats = torch.empty_like(quats) if covars is None else None
        v_scales = torch.empty_like(scales) if covars is None else None
        v_viewmats = torch.zeros_like(viewmats) if ctx.needs_input_grad[5] else None
        want_vel = ctx.want_vel and velocities is not None and ctx.needs_input_grad[4]
        v_vel = torch.empty_like(velocities) if want_vel else None
        _call(
            "splatad_lidar_projection_bwd", C, N, _lib.ptr(means), _lib.ptr(covars), _lib.ptr(quats),
            _lib.ptr(scales), _lib.ptr(velocities), _lib.ptr(viewmats), _lib.ptr(lin), _lib.ptr(ang),
            _lib.ptr(rs), ctx.eps2d, _lib.ptr(radii), _lib.ptr(conics), _lib.ptr(compensations),
            _lib.ptr(_f(v_means2d)), _lib.ptr(_f(v_depths)), _lib.ptr(_f(v_conics)),
            _lib.ptr(_f(v_compensations)) if compensations is not None else None,
            _lib.ptr(_f(v_pix_vels)), _lib.ptr(_f(v_depth_comps)), _lib.ptr(v_means),
            _lib.ptr(v_covars), _lib.ptr(v_quats), _lib.ptr(v_scales), _lib.ptr(v_viewmats),
            _lib.ptr(v_vel), _lib.stream_ptr(dev),
        )
        if not ctx.needs_input_grad[0]:
            v_means = None
        if not ctx.needs_input_grad[1]:
            v_covars = None
        if not ctx.needs_input_grad[2]:
            v_quats = None
        if not ctx.needs_input_grad[3]:
            v_scales = None
        return (v_means, v_covars, v_quats, v_scales, v_vel, v_viewmats) + (None,) * 13


class PendingPackedCount:
    """Lets ``fully_fused_projection(packed=True, pending=...)`` return before the host knows the
    number of packed rows. From the second frame of a shape on, the outputs then come back with
    ``capacity`` rows (the previous count + 12.5 %, rounded up to 64 Ki): the first ``nnz`` rows are
    the packed rows, the rest are padding with radii 0 and ids 0, which every op of this package
    skips or leaves unused (no tiles, colour 0.5, never listed). ``resolve()`` waits for the count
    and returns it, or None when the rows outgrew the capacity and the projection has to be called
    again; until then ``active`` says whether the outputs are padded at all (a first frame, or an
    empty input, is returned at its exact length as usual). Tensors handed on to the caller are cut
    to ``[:nnz]`` views; the backward pass reads the count from here."""

    def __init__(self):
        self.active = False
        self.capacity = 0
        self.nnz: Optional[int] = None
        self._event = self._host = self._key = None

    def resolve(self) -> Optional[int]:
        if not self.active:
            return self.nnz
        if self.nnz is None:
            self._event.synchronize()
            nnz = int(self._host[0])
            _packed_nnz_hint[self._key] = nnz
            if nnz > self.capacity:
                return None
            self.nnz = nnz
        return self.nnz


class _FullyFusedProjectionPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, means, covars, quats, scales, velocities, viewmats, Ks, width, height,
                linear_velocity, angular_velocity, rolling_shutter_time, eps2d, near_plane,
                far_plane, radius_clip, sparse_grad, calc_compensations, pending=None):
        means, covars, quats, scales, velocities, viewmats, lin, ang, rs = _proj_inputs(
            means, covars, quats, scales, velocities, viewmats, linear_velocity, angular_velocity,
            rolling_shutter_time)
        Ks = _f(Ks)
        C, N = viewmats.shape[0], means.shape[0]
        dev = means.device
        lib = _lib.load()
        indptr = torch.zeros(C + 1, dtype=torch.int32, device=dev)

        def outputs(rows):
            # with room to spare the fill kernel itself gives the rows behind the last packed one
            # ids 0 and radii 0
            return (torch.empty(rows, dtype=torch.int64, device=dev),
                    torch.empty(rows, dtype=torch.int64, device=dev),
                    torch.empty((rows, 2), dtype=torch.int32, device=dev),
                    torch.empty((rows, 2), dtype=torch.float32, device=dev),
                    torch.empty(rows, dtype=torch.float32, device=dev),
                    torch.empty((rows, 3), dtype=torch.float32, device=dev),
                    torch.empty(rows, dtype=torch.float32, device=dev) if calc_compensations else None,
                    torch.empty((rows, 2), dtype=torch.float32, device=dev))

        nnz, out = 0, None
        if C > 0 and N > 0:
            ws_bytes = lib.splatad_projection_packed_workspace_bytes(C, N)
            ws = _lib.workspace("packed", ws_bytes, dev)
            nnz_dev = torch.zeros(1, dtype=torch.int64, device=dev)
            common = (
                C, N, _lib.ptr(means), _lib.ptr(covars), _lib.ptr(quats), _lib.ptr(scales),
                _lib.ptr(velocities), _lib.ptr(viewmats), _lib.ptr(Ks), width, height, _lib.ptr(lin),
                _lib.ptr(ang), _lib.ptr(rs), eps2d, near_plane, far_plane, radius_clip,
            )

            def fill(capacity, o):
                _call("splatad_projection_packed_fill", *common, _lib.ptr(ws), capacity, *(_lib.ptr(x) for x in o),
                      _lib.stream_ptr(dev))

            _call("splatad_projection_packed_count", *common, _lib.ptr(ws), ws.numel(),
                  _lib.ptr(indptr), _lib.ptr(nnz_dev), _lib.stream_ptr(dev))
            # From the second frame of a shape on, the rows are written while the host still waits
            # for the count: into buffers with the previous count + 12.5 % of room, cut to length
            # afterwards (views). A frame that outgrows its room is filled again at the exact size.
            key = (C, N, dev.index, int(_lib.stream_ptr(dev)))
            hint = _packed_nnz_hint.get(key)
            capacity = None
            if hint:
                capacity = min((hint + hint // 8 + 4096 + 0xFFFF) & ~0xFFFF, C * N)
                out = outputs(capacity)
                fill(capacity, out)
            if pending is not None and capacity is not None:
                # the caller carries on with padded outputs and asks for the count when it needs it
                host = torch.empty(1, dtype=torch.int64, pin_memory=True)
                host.copy_(nnz_dev, non_blocking=True)
                pending._event = torch.cuda.Event()
                pending._event.record(torch.cuda.current_stream(dev))
                pending._host, pending._key = host, key
                pending.active, pending.capacity = True, capacity
            else:
                nnz = int(nnz_dev.item())
                _packed_nnz_hint[key] = nnz
                if capacity is not None and nnz <= capacity:
                    out = tuple(None if x is None else x[:nnz] for x in out)
                else:
                    out = outputs(nnz)
                    if nnz > 0:
                        fill(-1, out)
        if out is None:
            out = outputs(0)
        if pending is not None and not pending.active:
            pending.nnz = nnz
        ctx.pending = pending if (pending is not None and pending.active) else None
        camera_ids, gaussian_ids, radii, means2d, depths, conics, compensations, pix_vels = out
        ctx.save_for_backward(camera_ids, gaussian_ids, means, covars, quats, scales, velocities,
                              viewmats, Ks, lin, ang, rs, conics, compensations)
        ctx.width, ctx.height, ctx.eps2d, ctx.sparse_grad = width, height, eps2d, sparse_grad
        ctx.want_vel = _RETURN_VELOCITY_GRADS
        ctx.mark_non_differentiable(camera_ids, gaussian_ids, radii)
        return camera_ids, gaussian_ids, radii, means2d, depths, conics, compensations, pix_vels

    @staticmethod
    def backward(ctx, v_camera_ids, v_gaussian_ids, v_radii, v_means2d, v_depths, v_conics,
                 v_compensations, v_pix_vels):
        (camera_ids, gaussian_ids, means, covars, quats, scales, velocities, viewmats, Ks, lin, ang,
         rs, conics, compensations) = ctx.saved_tensors
        C, N, nnz = viewmats.shape[0], means.shape[0], camera_ids.shape[0]
        if ctx.pending is not None:
            # padded outputs: the first nnz rows count (the gradients of the padding are zero)
            nnz = ctx.pending.resolve()
            assert nnz is not None, "backward through a packed projection whose rows outgrew their room"
            gaussian_ids = gaussian_ids[:nnz]
        dev = means.device
        sparse = ctx.sparse_grad
        rows = nnz if sparse else N

        def grad_like(t):
            if t is None:
                return None
            shape = (rows,) + tuple(t.shape[1:])
            return torch.zeros(shape, dtype=torch.float32, device=dev)

        v_means = grad_like(means)
        v_covars = grad_like(covars)
        v_quats = grad_like(quats) if covars is None else None
        v_scales = grad_like(scales) if covars is None else None
        v_viewmats = torch.zeros_like(viewmats) if ctx.needs_input_grad[5] else None
        want_vel = ctx.want_vel and velocities is not None and ctx.needs_input_grad[4] and not sparse
        v_vel = torch.zeros_like(velocities) if want_vel else None
        _call(
            "splatad_projection_packed_bwd", C, N, nnz, _lib.ptr(means), _lib.ptr(covars),
            _lib.ptr(quats), _lib.ptr(scales), _lib.ptr(velocities), _lib.ptr(viewmats), _lib.ptr(Ks),
            ctx.width, ctx.height, _lib.ptr(lin), _lib.ptr(ang), _lib.ptr(rs), ctx.eps2d,
            _lib.ptr(camera_ids), _lib.ptr(gaussian_ids), _lib.ptr(conics), _lib.ptr(compensations),
            _lib.ptr(_f(v_means2d)), _lib.ptr(_f(v_depths)), _lib.ptr(_f(v_conics)),
            _lib.ptr(_f(v_compensations)) if compensations is not None else None,
            _lib.ptr(_f(v_pix_vels)), int(sparse), _lib.ptr(v_means), _lib.ptr(v_covars),
            _lib.ptr(v_quats), _lib.ptr(v_scales), _lib.ptr(v_viewmats), _lib.ptr(v_vel),
            _lib.stream_ptr(dev),
        )

        def finish(v, ref, needed):
            if not needed or v is None:
                return None
            if sparse:
                return torch.sparse_coo_tensor(indices=gaussian_ids[None], values=v, size=ref.size())
            return v

        v_means = finish(v_means, means, ctx.needs_input_grad[0])
        v_covars = finish(v_covars, covars, ctx.needs_input_grad[1]) if covars is not None else None
        v_quats = finish(v_quats, quats, ctx.needs_input_grad[2]) if covars is None else None
        v_scales = finish(v_scales, scales, ctx.needs_input_grad[3]) if covars is None else None
        return (v_means, v_covars, v_quats, v_scales, v_vel, v_viewmats) + (None,) * 13


# =============================================================================================
# Unfused building blocks of the projection (gsplat/cuda/_wrapper.py:46-228, 1283-1493)
# =============================================================================================
def quat_scale_to_covar_preci(quats: Tensor, scales: Tensor, compute_covar: bool = True,
                              compute_preci: bool = True, triu: bool = False,
                              ) -> Tuple[Optional[Tensor], Optional[Tensor]]:
    """Quaternions (w, x, y, z; need not be normalised) and scales -> covariance and precision
    matrices, [N,3,3] each or [N,6] upper triangles with ``triu``."""
    assert quats.dim() == 2 and quats.size(1) == 4, quats.size()
    assert scales.dim() == 2 and scales.size(1) == 3, scales.size()
    covars, precis = _QuatScaleToCovarPreci.apply(quats.contiguous(), scales.contiguous(), compute_covar,
                                                  compute_preci, triu)
    return covars if compute_covar else None, precis if compute_preci else None


class _QuatScaleToCovarPreci(torch.autograd.Function):
    @staticmethod
    def forward(ctx, quats, scales, compute_covar, compute_preci, triu):
        N, dev = quats.shape[0], quats.device
        q, s = _f(quats), _f(scales)
        shape = (N, 6) if triu else (N, 3, 3)
        covars = torch.empty(shape, dtype=torch.float32, device=dev) if compute_covar else None
        precis = torch.empty(shape, dtype=torch.float32, device=dev) if compute_preci else None
        if compute_covar or compute_preci:
            _call("splatad_quat_scale_to_covar_preci_fwd", N, _lib.ptr(q), _lib.ptr(s), int(bool(triu)),
                  _lib.ptr(covars), _lib.ptr(precis), _lib.stream_ptr(dev))
        ctx.save_for_backward(q, s)
        ctx.flags = (compute_covar, compute_preci, triu)
        # autograd wants tensors: an output that was not asked for is an empty placeholder
        empty = torch.empty(0, device=dev)
        return (covars if compute_covar else empty), (precis if compute_preci else empty)

    @staticmethod
    def backward(ctx, v_covars, v_precis):
        q, s = ctx.saved_tensors
        compute_covar, compute_preci, triu = ctx.flags
        dev = q.device
        vc = _f(v_covars.to_dense() if v_covars.is_sparse else v_covars) if compute_covar else None
        vp = _f(v_precis.to_dense() if v_precis.is_sparse else v_precis) if compute_preci else None
        v_quats, v_scales = torch.zeros_like(q), torch.zeros_like(s)
        if compute_covar or compute_preci:
            _call("splatad_quat_scale_to_covar_preci_bwd", q.shape[0], _lib.ptr(q), _lib.ptr(s), _lib.ptr(vc),
                  _lib.ptr(vp), int(bool(triu)), _lib.ptr(v_quats), _lib.ptr(v_scales), _lib.stream_ptr(dev))
        return v_quats, v_scales, None, None, None


def world_to_cam(means: Tensor, covars: Tensor, viewmats: Tensor) -> Tuple[Tensor, Tensor]:
    """World-frame Gaussians [N,3] / [N,3,3] -> sensor frames [C,N,3] / [C,N,3,3]."""
    C, N = viewmats.size(0), means.size(0)
    assert means.size() == (N, 3), means.size()
    assert covars.size() == (N, 3, 3), covars.size()
    assert viewmats.size() == (C, 4, 4), viewmats.size()
    return _WorldToCam.apply(means.contiguous(), covars.contiguous(), viewmats.contiguous())


class _WorldToCam(torch.autograd.Function):
    @staticmethod
    def forward(ctx, means, covars, viewmats):
        C, N, dev = viewmats.shape[0], means.shape[0], means.device
        m, c, v = _f(means), _f(covars), _f(viewmats)
        means_c = torch.empty((C, N, 3), dtype=torch.float32, device=dev)
        covars_c = torch.empty((C, N, 3, 3), dtype=torch.float32, device=dev)
        _call("splatad_world_to_cam_fwd", C, N, _lib.ptr(m), _lib.ptr(c), _lib.ptr(v), _lib.ptr(means_c),
              _lib.ptr(covars_c), _lib.stream_ptr(dev))
        ctx.save_for_backward(m, c, v)
        return means_c, covars_c

    @staticmethod
    def backward(ctx, v_means_c, v_covars_c):
        m, c, v = ctx.saved_tensors
        need = ctx.needs_input_grad
        v_means = torch.zeros_like(m) if need[0] else None
        v_covars = torch.zeros_like(c) if need[1] else None
        v_viewmats = torch.zeros_like(v) if need[2] else None
        _call("splatad_world_to_cam_bwd", v.shape[0], m.shape[0], _lib.ptr(m), _lib.ptr(c), _lib.ptr(v),
              _lib.ptr(_f(v_means_c)), _lib.ptr(_f(v_covars_c)), _lib.ptr(v_means), _lib.ptr(v_covars),
              _lib.ptr(v_viewmats), _lib.stream_ptr(m.device))
        return v_means, v_covars, v_viewmats


def persp_proj(means: Tensor, covars: Tensor, Ks: Tensor, width: int, height: int) -> Tuple[Tensor, Tensor]:
    """Pinhole projection of sensor-frame Gaussians: means2d [C,N,2], covars2d [C,N,2,2]."""
    C, N, _ = means.shape
    assert means.shape == (C, N, 3), means.size()
    assert covars.shape == (C, N, 3, 3), covars.size()
    assert Ks.shape == (C, 3, 3), Ks.size()
    return _PerspProj.apply(means.contiguous(), covars.contiguous(), Ks.contiguous(), width, height)


class _PerspProj(torch.autograd.Function):
    @staticmethod
    def forward(ctx, means, covars, Ks, width, height):
        C, N, dev = means.shape[0], means.shape[1], means.device
        m, c, k = _f(means), _f(covars), _f(Ks)
        means2d = torch.empty((C, N, 2), dtype=torch.float32, device=dev)
        covars2d = torch.empty((C, N, 2, 2), dtype=torch.float32, device=dev)
        _call("splatad_persp_proj_fwd", C, N, _lib.ptr(m), _lib.ptr(c), _lib.ptr(k), int(width), int(height),
              _lib.ptr(means2d), _lib.ptr(covars2d), _lib.stream_ptr(dev))
        ctx.save_for_backward(m, c, k)
        ctx.size = (int(width), int(height))
        return means2d, covars2d

    @staticmethod
    def backward(ctx, v_means2d, v_covars2d):
        m, c, k = ctx.saved_tensors
        v_means, v_covars = torch.empty_like(m), torch.empty_like(c)
        _call("splatad_persp_proj_bwd", m.shape[0], m.shape[1], _lib.ptr(m), _lib.ptr(c), _lib.ptr(k), *ctx.size,
              _lib.ptr(_f(v_means2d)), _lib.ptr(_f(v_covars2d)), _lib.ptr(v_means), _lib.ptr(v_covars),
              _lib.stream_ptr(m.device))
        return v_means, v_covars, None, None, None


def _check_velocity_args(p_view, lin_vel, ang_vel, velocities):
    C, N, _ = p_view.shape
    assert p_view.shape == (C, N, 3), p_view.size()
    assert lin_vel.shape == (C, 3), lin_vel.size()
    assert ang_vel.shape == (C, 3), ang_vel.size()
    assert velocities.shape == (C, N, 3), velocities.size()
    return C, N


def compute_pix_velocity(p_view: Tensor, lin_vel: Tensor, ang_vel: Tensor, velocities: Tensor, Ks: Tensor,
                         width: int, height: int) -> Tensor:
    """Velocity of sensor-frame Gaussians on the image plane, [C,N,2]: -J (lin + ang x p - v)."""
    C, _ = _check_velocity_args(p_view, lin_vel, ang_vel, velocities)
    assert Ks.shape == (C, 3, 3), Ks.size()
    return _ComputePixVelocity.apply(p_view.contiguous(), lin_vel.contiguous(), ang_vel.contiguous(),
                                     velocities.contiguous(), Ks.contiguous(), width, height)


class _ComputePixVelocity(torch.autograd.Function):
    @staticmethod
    def forward(ctx, p_view, lin_vel, ang_vel, velocities, Ks, width, height):
        C, N, dev = p_view.shape[0], p_view.shape[1], p_view.device
        args = tuple(_f(x) for x in (p_view, lin_vel, ang_vel, velocities, Ks))
        out = torch.empty((C, N, 2), dtype=torch.float32, device=dev)
        _call("splatad_compute_pix_velocity_fwd", C, N, *(_lib.ptr(x) for x in args), int(width), int(height),
              _lib.ptr(out), _lib.stream_ptr(dev))
        ctx.save_for_backward(*args)
        ctx.size = (int(width), int(height))
        return out

    @staticmethod
    def backward(ctx, v_out):
        args = ctx.saved_tensors
        p_view, velocities = args[0], args[3]
        v_p, v_v = torch.empty_like(p_view), torch.empty_like(velocities)
        _call("splatad_compute_pix_velocity_bwd", p_view.shape[0], p_view.shape[1], *(_lib.ptr(x) for x in args),
              *ctx.size, _lib.ptr(_f(v_out)), _lib.ptr(v_p), _lib.ptr(v_v), _lib.stream_ptr(p_view.device))
        return v_p, None, None, v_v, None, None, None


def lidar_proj(means: Tensor, covars: Tensor, eps2d: float) -> Tuple[Tensor, Tensor, Tensor]:
    """Spherical projection of sensor-frame Gaussians: (azimuth, elevation) in degrees [C,N,2], their
    covariance [C,N,2,2] and the depth compensation [C,N,2]."""
    C, N, _ = means.shape
    assert means.shape == (C, N, 3), means.size()
    assert covars.shape == (C, N, 3, 3), covars.size()
    return _LidarProj.apply(means.contiguous(), covars.contiguous(), eps2d)


class _LidarProj(torch.autograd.Function):
    @staticmethod
    def forward(ctx, means, covars, eps2d):
        C, N, dev = means.shape[0], means.shape[1], means.device
        m, c = _f(means), _f(covars)
        means2d = torch.empty((C, N, 2), dtype=torch.float32, device=dev)
        covars2d = torch.empty((C, N, 2, 2), dtype=torch.float32, device=dev)
        depth_comps = torch.empty((C, N, 2), dtype=torch.float32, device=dev)
        _call("splatad_lidar_proj_fwd", C, N, _lib.ptr(m), _lib.ptr(c), float(eps2d), _lib.ptr(means2d),
              _lib.ptr(covars2d), _lib.ptr(depth_comps), _lib.stream_ptr(dev))
        ctx.save_for_backward(m, c)
        ctx.eps2d = float(eps2d)
        return means2d, covars2d, depth_comps

    @staticmethod
    def backward(ctx, v_means2d, v_covars2d, v_depth_comps):
        m, c = ctx.saved_tensors
        v_means, v_covars = torch.empty_like(m), torch.empty_like(c)
        _call("splatad_lidar_proj_bwd", m.shape[0], m.shape[1], _lib.ptr(m), _lib.ptr(c), ctx.eps2d,
              _lib.ptr(_f(v_means2d)), _lib.ptr(_f(v_covars2d)), _lib.ptr(_f(v_depth_comps)), _lib.ptr(v_means),
              _lib.ptr(v_covars), _lib.stream_ptr(m.device))
        return v_means, v_covars, None


def compute_lidar_velocity(p_view: Tensor, lin_vel: Tensor, ang_vel: Tensor, velocities: Tensor) -> Tensor:
    """Velocity of sensor-frame Gaussians in (azimuth, elevation, range), [C,N,3]."""
    _check_velocity_args(p_view, lin_vel, ang_vel, velocities)
    return _ComputeLidarVelocity.apply(p_view.contiguous(), lin_vel.contiguous(), ang_vel.contiguous(),
                                       velocities.contiguous())


class _ComputeLidarVelocity(torch.autograd.Function):
    @staticmethod
    def forward(ctx, p_view, lin_vel, ang_vel, velocities):
        C, N, dev = p_view.shape[0], p_view.shape[1], p_view.device
        args = tuple(_f(x) for x in (p_view, lin_vel, ang_vel, velocities))
        out = torch.empty((C, N, 3), dtype=torch.float32, device=dev)
        _call("splatad_compute_lidar_velocity_fwd", C, N, *(_lib.ptr(x) for x in args), _lib.ptr(out),
              _lib.stream_ptr(dev))
        ctx.save_for_backward(*args)
        return out

    @staticmethod
    def backward(ctx, v_out):
        args = ctx.saved_tensors
        p_view, velocities = args[0], args[3]
        v_p, v_v = torch.empty_like(p_view), torch.empty_like(velocities)
        _call("splatad_compute_lidar_velocity_bwd", p_view.shape[0], p_view.shape[1],
              *(_lib.ptr(x) for x in args), _lib.ptr(_f(v_out)), _lib.ptr(v_p), _lib.ptr(v_v),
              _lib.stream_ptr(p_view.device))
        return v_p, None, None, v_v


# =============================================================================================
# Tile intersection
# =============================================================================================
def _isect_common(kind, means2d, radii, depths, packed, n_cameras, camera_ids, gaussian_ids, sort,
                  geom_args, n_tiles, deferred=False):
    """Shared two-phase driver of both isect ops: plan -> read n_isects on the host -> fill.

    ``kind`` ("tiles" or "lidar_tiles") is spliced into the C symbol name; ``n_tiles`` is the number
    of tiles per sensor. With ``deferred`` a :class:`DeferredIsect` is returned instead: when a call
    of the same shape has been seen before, plan and fill are enqueued without the host round trip.
    """
    if packed:
        nnz = means2d.size(0)
        assert means2d.shape == (nnz, 2), means2d.size()
        assert radii.shape == (nnz, 2), radii.size()
        assert depths.shape == (nnz,), depths.size()
        assert camera_ids is not None, "camera_ids is required if packed is True"
        assert gaussian_ids is not None, "gaussian_ids is required if packed is True"
        assert n_cameras is not None, "n_cameras is required if packed is True"
        camera_ids = camera_ids.to(torch.int64).contiguous()
        C, N, total = n_cameras, 0, nnz
    else:
        C, N, _ = means2d.shape
        assert means2d.shape == (C, N, 2), means2d.size()
        assert radii.shape == (C, N, 2), radii.size()
        assert depths.shape == (C, N), depths.size()
        camera_ids = None
        total = C * N
    dev = means2d.device
    n_tiles_total = C * n_tiles
    means2d = _f(means2d)
    depths = _f(depths)
    if kind == "tiles":
        radii = radii.to(torch.int32).contiguous()
    else:
        radii = _f(radii)
    lib = _lib.load()
    tiles_per_gauss = torch.empty(depths.shape, dtype=torch.int32, device=dev)
    if total == 0:
        out = (tiles_per_gauss, torch.empty(0, dtype=torch.int64, device=dev),
               torch.empty(0, dtype=torch.int32, device=dev))
        return DeferredIsect.done(*out, C, n_tiles_total) if deferred else out
    plan_bytes = lib.splatad_isect_plan_workspace_bytes(total)
    plan_ws = _lib.workspace("isect_plan", plan_bytes, dev)
    # where the plan's count arrives: the two-step protocol reads it before returning and can share
    # one slot per device; a deferred call reads it later and owns its slot until then
    host = _lib.pinned_counts("isect", dev)
    stream = _lib.stream_ptr(dev)
    head = (C, N, total, _lib.ptr(means2d), _lib.ptr(radii), _lib.ptr(depths), _lib.ptr(camera_ids))
    # packed inputs: the row count changes from frame to frame, the hint only sizes the room
    key = (kind, C, N, None if packed else total, n_tiles_total, dev.index, int(stream))
    hint = _isect_count_hint.get(key) if (deferred and sort) else None

    # sorted lists: 1 = depth order by buckets (four kernels); 2 = by radix passes (twelve), for scenes
    # whose depths crowd into few buckets (the plan says so with status bit 4; remembered per shape)
    mode = [0 if not sort else _depth_sort_mode.get(key, 1)]

    def plan(slot=None):
        _call(f"splatad_isect_{kind}_plan", *head, *geom_args, mode[0], _lib.ptr(tiles_per_gauss),
              _lib.ptr(plan_ws), plan_ws.numel(), (host if slot is None else slot).data_ptr(), stream)

    def fill(capacity):
        isect_ids = torch.empty(capacity, dtype=torch.int64, device=dev)
        flatten_ids = torch.empty(capacity, dtype=torch.int32, device=dev)
        offsets = None
        if capacity > 0:
            fill_ws = None
            if sort:
                fill_bytes = lib.splatad_isect_fill_workspace_bytes(capacity)
                fill_ws = _lib.workspace("isect_fill", fill_bytes, dev)
                # the fill knows where every tile starts (and appends the total); kept for
                # isect_offset_encode on this tensor
                offsets = torch.empty(n_tiles_total + 1, dtype=torch.int32, device=dev)
            _call(f"splatad_isect_{kind}_fill", *head, *geom_args, mode[0],
                  _lib.ptr(tiles_per_gauss), _lib.ptr(plan_ws), _lib.ptr(fill_ws),
                  fill_ws.numel() if fill_ws is not None else 0, capacity, _lib.ptr(isect_ids),
                  _lib.ptr(flatten_ids), _lib.ptr(offsets), None, stream)
        return isect_ids, flatten_ids, offsets

    def read_count(slot=None, sequence=0, event=None):
        if slot is None:
            n_isects, status = int(host[0]), int(host[2])
        else:
            n_isects, status = _lib.wait_for_count(slot, sequence, event)
            _lib.release_pinned_slot(slot)
        if status & 2 or n_isects > 0x7FFFFFFF:
            raise RuntimeError(f"isect: {n_isects} intersections do not fit int32 flatten ids / offsets")
        _isect_count_hint[key] = n_isects
        if status & 4 and mode[0] == 1:
            _depth_sort_mode[key] = 2
            return -1          # the depth buckets were too crowded: the order is not final
        return n_isects

    def exact():
        plan()
        torch.cuda.current_stream(dev).synchronize()
        n_isects = read_count()
        if n_isects < 0:       # once more, with the radix depth sort
            mode[0] = 2
            plan()
            torch.cuda.current_stream(dev).synchronize()
            n_isects = read_count()
        isect_ids, flatten_ids, offsets = fill(n_isects)
        if offsets is not None:
            isect_ids._splatad_tile_offsets = (C, offsets[:n_tiles_total])
        return tiles_per_gauss, isect_ids, flatten_ids

    if not deferred:
        return exact()
    if hint is None:
        return DeferredIsect.done(*exact(), C, n_tiles_total)
    # Enqueue plan and fill back to back with room for somewhat more intersections than last time;
    # the count is read when the caller asks for the exact tensors.
    capacity = hint + hint // 8 + 65536
    slot = _lib.acquire_pinned_slot(dev)
    # the rectangle count kernel hands the count to the host itself (slot[4:6]) when the lists are
    # built by the row / column split; the event behind the plan is the fallback
    sequence = _lib.next_sequence()
    lib.splatad_isect_set_early_count(slot.data_ptr() + 32, sequence)
    try:
        plan(slot)
    finally:
        lib.splatad_isect_set_early_count(None, 0)
    counted = torch.cuda.Event()
    counted.record(torch.cuda.current_stream(dev))
    isect_buf, flat_buf, offsets = fill(capacity)
    return DeferredIsect(tiles_per_gauss, isect_buf, flat_buf, offsets, C, n_tiles_total, capacity,
                         counted, lambda: read_count(slot, sequence, counted), exact)


# (kind, shape, tile grid, device, stream) -> intersection count of the last frame of that shape on
# that stream (see _packed_nnz_hint for why the stream is part of the key)
_isect_count_hint: dict = {}
_depth_range_hint: dict = {}    # per frame shape and stream: (lo bits, hi bits) of the last frame's listed depths
_depth_sort_mode: dict = {}   # same keys -> 2 once a frame of the shape needed the radix depth sort


class DeferredIsect:
    """Tile intersection whose count may still be on the device.

    ``flatten_ids`` (at least as long as the count) and ``offsets`` ([C * tiles] tile starts followed
    by the total) can be handed to the compositing ops at once; ``resolve()`` waits for the count
    and returns (isect_ids, flatten_ids) of the exact length - or None when the count outgrew the
    room given to it, in which case ``redo()`` runs the two-step protocol and everything composited
    from this object has to be repeated.
    """

    def __init__(self, tiles_per_gauss, isect_buf, flat_buf, offsets, C, n_tiles_total, capacity, counted,
                 read_count, exact):
        self.tiles_per_gauss = tiles_per_gauss
        self.flatten_ids = flat_buf
        self._isect_buf = isect_buf
        self._offsets = offsets
        self._C, self._n_tiles_total = C, n_tiles_total
        self._capacity, self._counted, self._read_count, self._exact = capacity, counted, read_count, exact
        self._resolved = None

    @classmethod
    def done(cls, tiles_per_gauss, isect_ids, flatten_ids, C, n_tiles_total):
        d = cls(tiles_per_gauss, isect_ids, flatten_ids, None, C, n_tiles_total, isect_ids.numel(), None,
                None, None)
        d._resolved = (isect_ids, flatten_ids)
        return d

    def offsets(self, tile_height: int, tile_width: int) -> Tensor:
        """[C, tile_height, tile_width] tile starts for the compositing ops."""
        if self._offsets is None or self._C * tile_height * tile_width != self._n_tiles_total:
            resolved = self.resolve()
            if resolved is None:
                raise RuntimeError("isect: count outgrew its room and the tile grid does not match")
            return isect_offset_encode(resolved[0], self._C, tile_width, tile_height)
        return self._offsets[: self._n_tiles_total].view(self._C, tile_height, tile_width)

    def total_follows(self, tile_height: int, tile_width: int) -> bool:
        """Whether :meth:`offsets` for this grid is a view of a buffer that holds the intersection
        count right behind the last tile start (pass it on as ``total_follows`` to the compositing
        ops, which then take the end of the last tile from there instead of ``len(flatten_ids)``)."""
        return self._offsets is not None and self._C * tile_height * tile_width == self._n_tiles_total

    def resolve(self):
        if self._resolved is None:
            n_isects = self._read_count()
            if n_isects < 0 or n_isects > self._capacity:
                return None
            isect_ids = self._isect_buf[:n_isects]
            isect_ids._splatad_tile_offsets = (self._C, self._offsets[: self._n_tiles_total])
            self._resolved = (isect_ids, self.flatten_ids[:n_isects])
        return self._resolved

    def redo(self):
        tiles_per_gauss, isect_ids, flatten_ids = self._exact()
        return DeferredIsect.done(tiles_per_gauss, isect_ids, flatten_ids, self._C, self._n_tiles_total)


def validate_lists(flatten_ids: Tensor, n_rows: int, isect_offsets: Optional[Tensor] = None,
                   total_follows: bool = False, camera_ids: Optional[Tensor] = None,
                   gaussian_ids: Optional[Tensor] = None, n_cameras: int = 0, n_gaussians: int = 0):
    """Checks, without dereferencing anything through them, the indices the compositing kernels are
    about to follow: flatten ids within ``n_rows``, tile offsets ordered and within the list, packed
    ids within range. Returns (violations, site, index, limit) - all zero for consistent lists.
    Called before every compositing launch when ``SPLATAD_DEBUG=1`` (where a violation raises)."""
    dev = flatten_ids.device
    report = torch.zeros(4, dtype=torch.int64, device=dev)
    flat = flatten_ids.to(torch.int32).contiguous()
    offs = None if isect_offsets is None else isect_offsets
    n_tiles = 0 if offs is None else offs.numel()
    n_packed = 0 if gaussian_ids is None else gaussian_ids.numel()
    _call("splatad_debug_validate_lists", flat.numel(), _lib.ptr(flat) if flat.numel() else None, int(n_rows),
          _lib.ptr(offs), n_tiles, int(bool(total_follows)),
          _lib.ptr(camera_ids.to(torch.int64).contiguous()) if camera_ids is not None and n_packed else None,
          _lib.ptr(gaussian_ids.to(torch.int64).contiguous()) if n_packed else None, n_packed, int(n_cameras),
          int(n_gaussians), _lib.ptr(report), _lib.stream_ptr(dev))
    return tuple(int(v) for v in report.tolist())


def _debug_check_lists(what: str, flatten_ids: Tensor, n_rows: int, isect_offsets: Tensor, total_follows: bool):
    if _lib.DEBUG and flatten_ids.numel():
        bad, site, index, limit = validate_lists(flatten_ids, n_rows, isect_offsets.contiguous(), total_follows)
        if bad:
            names = {1: "flatten id", 2: "tile offsets out of order at tile", 3: "tile offset out of range at tile"}
            raise RuntimeError(f"{what}: {bad} inconsistent list entries; first: {names.get(site, site)} {index} "
                               f"(limit {limit})")


def _zeros_like_many(*tensors: Optional[Tensor]) -> list:
    """float32 zeros shaped like each given tensor (None stays None), as views of ONE zero-filled
    buffer: one allocation and one fill for all the gradient accumulators of a backward call. Every
    view starts a multiple of 256 bytes behind the buffer's start."""
    live = [t for t in tensors if t is not None]
    if not live:
        return [None] * len(tensors)
    starts, total = [], 0
    for t in live:
        starts.append(total)
        total += (t.numel() + 63) // 64 * 64
    buf = torch.zeros(total, dtype=torch.float32, device=live[0].device)
    views = iter(buf[s:s + t.numel()].view(t.shape) for s, t in zip(starts, live))
    return [None if t is None else next(views) for t in tensors]


def _n_isects_arg(isect_offsets: Tensor, flatten_ids: Tensor, total_follows: bool = False) -> int:
    """What the compositing entry points get as n_isects: the length of flatten_ids, or -1 when the
    caller states that the total sits behind the tile starts on the device (see DeferredIsect)."""
    if not total_follows:
        return flatten_ids.numel()
    room = isect_offsets.untyped_storage().nbytes() // isect_offsets.element_size()
    if not (isect_offsets.is_contiguous() and isect_offsets.dtype == torch.int32
            and room >= isect_offsets.storage_offset() + isect_offsets.numel() + 1):
        raise ValueError("total_follows: isect_offsets is not a contiguous int32 view with one more entry behind it")
    return -1


class LidarFrame:
    """A lidar frame enqueued by :func:`lidar_frame_fwd`: the outputs are on their way, the
    intersection count arrives in a pinned slot. ``finish()`` waits for the count and returns the
    exact-length (isect_ids, flatten_ids), or None when the count outgrew the room the frame was
    given (the frame then has to be rendered the ordinary way)."""

    def __init__(self, tensors, capacity, counted, slot, key, sequence, ranged=False):
        self.__dict__.update(tensors)
        self._capacity, self._counted, self._slot, self._key = capacity, counted, slot, key
        self._sequence, self._ranged = sequence, ranged

    def finish(self):
        n_isects, status = _lib.wait_for_count(self._slot, self._sequence, self._counted)
        depth_range = _lib.early_depth_range(self._slot, self._sequence)
        _lib.release_pinned_slot(self._slot)
        if status & 2 or n_isects > 0x7FFFFFFF:
            raise RuntimeError(f"isect: {n_isects} intersections do not fit int32 flatten ids / offsets")
        _isect_count_hint[self._key] = n_isects
        if status & 4:
            if self._ranged:
                # an end bucket overflowed under the depth range carried over from the last frame:
                # the frame is rendered again without one
                _depth_range_hint.pop(self._key, None)
            else:
                _depth_sort_mode[self._key] = 2   # crowded depth buckets: this shape takes the radix sort from now on
            return None
        if depth_range is not None:
            _depth_range_hint[self._key] = depth_range
        if n_isects > self._capacity:
            return None
        isect_ids = self.isect_buf[:n_isects]
        isect_ids._splatad_tile_offsets = (self.C, self.offsets_buf[:-1])
        return isect_ids, self.flatten_buf[:n_isects]


@torch.no_grad()
def lidar_frame_fwd(means, quats, scales, velocities, opacities_cn, lidar_features, viewmats, linear_velocity,
                    angular_velocity, rolling_shutter_time, raster_pts, tile_elevation_boundaries,
                    azimuth_resolution, tile_width, tile_height, min_azimuth, max_azimuth, min_elevation,
                    max_elevation, eps2d, near_plane, far_plane, radius_clip, compute_alpha_sum,
                    alpha_sum_threshold, expected_grid=None) -> Optional["LidarFrame"]:
    """Forward pass of a whole lidar frame (projection, tile intersection, compositing) through ONE
    library call (``splatad_lidar_frame_fwd``), for frames that need no gradients: the host work
    between the 22 launches of a frame, not the GPU, is what limits the frame rate of small frames.
    Needs the intersection count of an earlier frame of the same shape on this stream to size the
    lists (returns None when there is none yet: render that frame with the individual ops).
    Not part of the reference's API; used by ``splatad_b200.lidar_rasterization``."""
    C, N = viewmats.shape[0], means.shape[0]
    D = lidar_features.shape[-1]
    dev = means.device
    if C * N == 0 or D + 1 > _lib.MAX_CHANNELS:
        return None
    lib = _lib.load()
    eb = _f(tile_elevation_boundaries)
    n_rows = int(eb.numel()) - 1
    tile_az = float(azimuth_resolution) * int(tile_width)
    n_cols = int(lib.splatad_lidar_azimuth_tiles(tile_az))
    if expected_grid is not None and tuple(expected_grid) != (n_rows, n_cols):
        return None   # the caller's tile grid is not the one the intersection builds
    n_tiles_total = C * n_cols * n_rows
    stream = _lib.stream_ptr(dev)
    key = ("lidar_tiles", C, N, C * N, n_tiles_total, dev.index, int(stream))
    hint = _isect_count_hint.get(key)
    if hint is None or _depth_sort_mode.get(key, 1) != 1:
        return None
    capacity = hint + hint // 8 + 65536
    H, W = raster_pts.shape[1:3]
    f32 = dict(dtype=torch.float32, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    t = dict(
        C=C, grid=(n_rows, n_cols),
        radii=torch.empty((C, N, 2), **f32), means2d=torch.empty((C, N, 2), **f32),
        depths=torch.empty((C, N), **f32), conics=torch.empty((C, N, 3), **f32),
        pix_vels=torch.empty((C, N, 3), **f32), depth_compensations=torch.empty((C, N, 2), **f32),
        tiles_per_gauss=torch.empty((C, N), **i32),
        isect_buf=torch.empty(capacity, dtype=torch.int64, device=dev), flatten_buf=torch.empty(capacity, **i32),
        offsets_buf=torch.empty(n_tiles_total + 1, **i32),
        render=torch.empty((C, H, W, D + 1), **f32), alphas=torch.empty((C, H, W, 1), **f32),
        alpha_sum=torch.empty((C, H, W, 1), **f32) if compute_alpha_sum else None,
        last_ids=torch.empty((C, H, W), **i32), median_depths=torch.empty((C, H, W, 1), **f32),
    )
    plan_ws = _lib.workspace("isect_plan", lib.splatad_isect_plan_workspace_bytes(C * N), dev)
    fill_ws = _lib.workspace("isect_fill", lib.splatad_isect_fill_workspace_bytes(capacity), dev)
    slot = _lib.acquire_pinned_slot(dev)
    sequence = _lib.next_sequence()   # the count kernel stores the count + this number into slot[4:6]
    # the depth range of the last frame of this shape, widened by a tenth on either side, spans this
    # frame's depth buckets: the rectangle count then fills them and one kernel less is launched
    ranged = False
    last_range = _depth_range_hint.get(key)
    if last_range is not None:
        lo, hi = (struct.unpack("<f", struct.pack("<I", b))[0] for b in last_range)
        if 0.0 <= lo <= hi < float("inf"):
            pad = 0.1 * (hi - lo) + 1e-3
            lo_bits, hi_bits = (struct.unpack("<I", struct.pack("<f", v))[0] for v in (max(lo - pad, 0.0), hi + pad))
            lib.splatad_isect_set_depth_range_hint(lo_bits, hi_bits)
            ranged = True
    p = _lib.ptr
    try:
        _call("splatad_lidar_frame_fwd", C, N, p(_f(means)), p(_f(quats)), p(_f(scales)), p(_f(velocities)),
              p(_f(opacities_cn)), p(_f(lidar_features)), D, p(_f(viewmats)), p(_f(linear_velocity)),
              p(_f(angular_velocity)), p(_f(rolling_shutter_time)), p(_f(raster_pts)), W, H, p(eb), n_rows + 1,
              float(azimuth_resolution), int(tile_width), int(tile_height), float(min_azimuth), float(max_azimuth),
              float(min_elevation), float(max_elevation), float(eps2d), float(near_plane), float(far_plane),
              float(radius_clip), int(bool(compute_alpha_sum)), float(alpha_sum_threshold), p(t["radii"]),
              p(t["means2d"]), p(t["depths"]), p(t["conics"]), p(t["pix_vels"]), p(t["depth_compensations"]),
              p(t["tiles_per_gauss"]), capacity, p(t["isect_buf"]), p(t["flatten_buf"]), p(t["offsets_buf"]),
              p(t["render"]), p(t["alphas"]), p(t["alpha_sum"]), p(t["last_ids"]), p(t["median_depths"]),
              p(plan_ws), plan_ws.numel(), p(fill_ws), fill_ws.numel(), slot.data_ptr(), slot.data_ptr() + 32, sequence,
              stream)
    except BaseException:
        if ranged:
            lib.splatad_isect_set_depth_range_hint(1, 0)   # disarm: no later plan of this thread inherits the range
        _lib.release_pinned_slot(slot)
        raise
    counted = torch.cuda.Event()      # fallback: the counters the plan copies at its end
    counted.record(torch.cuda.current_stream(dev))
    return LidarFrame(t, capacity, counted, slot, key, sequence, ranged)


@torch.no_grad()
def isect_tiles(
    means2d: Tensor,  # [C, N, 2] or [nnz, 2]
    radii: Tensor,  # [C, N, 2] or [nnz, 2]
    depths: Tensor,  # [C, N] or [nnz]
    tile_size: int,
    tile_width: int,
    tile_height: int,
    sort: bool = True,
    packed: bool = False,
    n_cameras: Optional[int] = None,
    camera_ids: Optional[Tensor] = None,
    gaussian_ids: Optional[Tensor] = None,
) -> Tuple[Tensor, Tensor, Tensor]:
    """Maps projected Gaussians to the camera tiles they touch.

    Returns (tiles_per_gauss int32, isect_ids int64 [n_isects] = sensor | tile | depth bits,
    flatten_ids int32 [n_isects]), sorted by isect id (ties in flatten order) when ``sort``.
    """
    return _isect_common("tiles", means2d, radii, depths, packed, n_cameras, camera_ids, gaussian_ids,
                         sort, (int(tile_size), int(tile_width), int(tile_height)),
                         int(tile_width) * int(tile_height))


@torch.no_grad()
def isect_lidar_tiles(
    means2d: Tensor,  # [C, N, 2] or [nnz, 2]
    radii: Tensor,  # [C, N, 2] or [nnz, 2]
    depths: Tensor,  # [C, N] or [nnz]
    elev_boundaries: Tensor,
    tile_azim_resolution: float,
    min_azim: float,
    sort: bool = True,
    packed: bool = False,
    n_cameras: Optional[int] = None,
    camera_ids: Optional[Tensor] = None,
    gaussian_ids: Optional[Tensor] = None,
) -> Tuple[Tensor, Tensor, Tensor]:
    """Maps projected Gaussians to lidar tiles (uniform azimuth tiles with wrap-around, elevation
    tiles given by ``elev_boundaries``). Same returns as :func:`isect_tiles`."""
    eb = _f(elev_boundaries)
    return _isect_common("lidar_tiles", means2d, radii, depths, packed, n_cameras, camera_ids,
                         gaussian_ids, sort,
                         (_lib.ptr(eb), int(eb.numel()), float(tile_azim_resolution), float(min_azim)),
                         int(_lib.load().splatad_lidar_azimuth_tiles(float(tile_azim_resolution)))
                         * (int(eb.numel()) - 1))


@torch.no_grad()
def isect_tiles_deferred(means2d, radii, depths, tile_size, tile_width, tile_height, packed=False,
                         n_cameras=None, camera_ids=None, gaussian_ids=None) -> "DeferredIsect":
    """:func:`isect_tiles` (sorted) without the wait for the intersection count in the middle; see
    :class:`DeferredIsect`. Used by ``splatad_b200.rasterization``."""
    return _isect_common("tiles", means2d, radii, depths, packed, n_cameras, camera_ids, gaussian_ids,
                         True, (int(tile_size), int(tile_width), int(tile_height)),
                         int(tile_width) * int(tile_height), deferred=True)


@torch.no_grad()
def isect_lidar_tiles_deferred(means2d, radii, depths, elev_boundaries, tile_azim_resolution, min_azim,
                               packed=False, n_cameras=None, camera_ids=None,
                               gaussian_ids=None) -> "DeferredIsect":
    """:func:`isect_lidar_tiles` (sorted) without the wait for the intersection count in the middle;
    see :class:`DeferredIsect`. Used by ``splatad_b200.lidar_rasterization``."""
    eb = _f(elev_boundaries)
    n_tiles = int(_lib.load().splatad_lidar_azimuth_tiles(float(tile_azim_resolution))) * (int(eb.numel()) - 1)
    return _isect_common("lidar_tiles", means2d, radii, depths, packed, n_cameras, camera_ids,
                         gaussian_ids, True,
                         (_lib.ptr(eb), int(eb.numel()), float(tile_azim_resolution), float(min_azim)),
                         n_tiles, deferred=True)


@torch.no_grad()
def isect_offset_encode(isect_ids: Tensor, n_cameras: int, tile_width: int, tile_height: int) -> Tensor:
    """Encodes sorted intersection ids to per-tile start offsets [C, tile_height, tile_width]."""
    cached = getattr(isect_ids, "_splatad_tile_offsets", None)
    if cached is not None and cached[0] == n_cameras and cached[1].numel() == n_cameras * tile_height * tile_width:
        return cached[1].view(n_cameras, tile_height, tile_width)
    isect_ids = isect_ids.contiguous()
    dev = isect_ids.device
    offsets = torch.empty((n_cameras, tile_height, tile_width), dtype=torch.int32, device=dev)
    if offsets.numel() == 0:
        return offsets
    _call("splatad_isect_offset_encode", _lib.ptr(isect_ids) if isect_ids.numel() else None,
          isect_ids.numel(), n_cameras, tile_width, tile_height, _lib.ptr(offsets), _lib.stream_ptr(dev))
    return offsets


# =============================================================================================
# Lidar points -> tiles -> raster image
# =============================================================================================
@torch.no_grad()
def map_points_to_lidar_tiles(
    points2d: Tensor,  # [C, N, 2] or [nnz, 2]
    elev_boundaries: Tensor,
    tile_azim_resolution: float,
    min_azim: float,
    packed: bool = False,
    n_cameras: Optional[int] = None,
    camera_ids: Optional[Tensor] = None,
    sort: bool = True,
) -> Tuple[Tensor, Tensor]:
    """Maps (azimuth, elevation) points to the lidar tile that holds them (zero radius), as
    ``gsplat.cuda._wrapper.map_points_to_lidar_tiles`` (gsplat/cuda/_wrapper.py:697-758).

    Returns (tile ids int64 [total] = sensor << 32 | tile, flatten ids int32 [total]), ordered by
    tile id (ties in point order) when ``sort``."""
    if packed:
        nnz = points2d.size(0)
        assert points2d.shape == (nnz, 2), points2d.size()
        assert camera_ids is not None, "camera_ids is required if packed is True"
        assert n_cameras is not None, "n_cameras is required if packed is True"
        camera_ids = camera_ids.to(torch.int64).contiguous()
        C, N, total = n_cameras, 0, nnz
    else:
        C, N, _ = points2d.shape
        assert points2d.shape == (C, N, 2), points2d.size()
        camera_ids, total = None, C * N
    dev = points2d.device
    pts, eb = _f(points2d), _f(elev_boundaries)
    tile_ids = torch.empty(total, dtype=torch.int64, device=dev)
    flatten_ids = torch.empty(total, dtype=torch.int32, device=dev)
    if total == 0:
        return tile_ids, flatten_ids
    lib = _lib.load()
    ws = _lib.workspace("map_points", lib.splatad_map_points_workspace_bytes(total), dev) if sort else None
    _call("splatad_map_points_to_lidar_tiles", C, N, total, _lib.ptr(pts), _lib.ptr(camera_ids), _lib.ptr(eb),
          int(eb.numel()), float(tile_azim_resolution), float(min_azim), int(bool(sort)), _lib.ptr(ws),
          ws.numel() if ws is not None else 0, _lib.ptr(tile_ids), _lib.ptr(flatten_ids), _lib.stream_ptr(dev))
    return tile_ids, flatten_ids


@torch.no_grad()
def points_mapping_offset_encode(point_ids: Tensor, n_lidars: int, tile_width: int, tile_height: int) -> Tensor:
    """Sorted point tile ids -> start of every tile's list, [C, tile_height, tile_width] int32
    (gsplat/cuda/_wrapper.py:760-776)."""
    point_ids = point_ids.contiguous()
    dev = point_ids.device
    offsets = torch.empty((n_lidars, tile_height, tile_width), dtype=torch.int32, device=dev)
    if offsets.numel() == 0:
        return offsets
    _call("splatad_points_mapping_offset_encode", _lib.ptr(point_ids) if point_ids.numel() else None,
          point_ids.numel(), n_lidars, tile_width, tile_height, _lib.ptr(offsets), _lib.stream_ptr(dev))
    return offsets


@torch.no_grad()
def populate_image_from_points(
    points: Tensor,  # [C, N, 5] or [nnz, 5]
    image_width: int,
    image_height: int,
    tile_width: int,
    tile_height: int,
    tile_offsets: Tensor,  # [C, tile grid height, tile grid width]
    flatten_id: Tensor,  # [n_points]
) -> Tensor:
    """Raster image [C, image_height, image_width, 5] whose pixels take the values of the points
    listed for their tile, in list order (gsplat/cuda/_wrapper.py:778-809)."""
    assert points.shape[-1] == 5, points.shape
    pts = _f(points)
    dev = pts.device
    C, grid_h, grid_w = tile_offsets.shape
    offs = tile_offsets.to(torch.int32).contiguous()
    flat = flatten_id.to(torch.int32).contiguous()
    image = torch.empty((C, image_height, image_width, 5), dtype=torch.float32, device=dev)
    if image.numel() == 0:
        return image
    _call("splatad_populate_image_from_points", C, flat.numel(), _lib.ptr(pts) if pts.numel() else None,
          image_width, image_height, tile_width, tile_height, grid_w, grid_h, _lib.ptr(offs),
          _lib.ptr(flat) if flat.numel() else None, _lib.ptr(image), _lib.stream_ptr(dev))
    return image


# =============================================================================================
# Compositing
# =============================================================================================
def rasterize_to_pixels(
    means2d: Tensor,  # [C, N, 2] or [nnz, 2]
    conics: Tensor,  # [C, N, 3] or [nnz, 3]
    colors: Tensor,  # [C, N, channels] or [nnz, channels]
    opacities: Tensor,  # [C, N] or [nnz]
    pix_vels: Tensor,  # [C, N, 2] or [nnz, 2]
    image_width: int,
    image_height: int,
    tile_size: int,
    isect_offsets: Tensor,  # [C, tile_height, tile_width]
    flatten_ids: Tensor,  # [n_isects]
    rolling_shutter_time: Optional[Tensor] = None,  # [C]
    backgrounds: Optional[Tensor] = None,  # [C, channels]
    packed: bool = False,
    absgrad: bool = False,
    total_follows: bool = False,
) -> Tuple[Tensor, Tensor]:
    """Rasterizes Gaussians to pixels. Returns (colors [C,H,W,channels], alphas [C,H,W,1]).

    ``total_follows`` (not in the reference): ``isect_offsets`` is a view of a buffer that holds the
    number of intersections right behind the last tile start (:meth:`DeferredIsect.offsets`) and
    ``flatten_ids`` may be longer than that number; the kernels then read the end of the last tile
    from the device instead of taking ``len(flatten_ids)``."""
    C = isect_offsets.size(0)
    device = means2d.device
    if packed:
        nnz = means2d.size(0)
        assert means2d.shape == (nnz, 2), means2d.shape
        assert conics.shape == (nnz, 3), conics.shape
        assert colors.shape[0] == nnz, colors.shape
        assert opacities.shape == (nnz,), opacities.shape
        assert pix_vels.shape == (nnz, 2), pix_vels.shape
    else:
        N = means2d.size(1)
        assert means2d.shape == (C, N, 2), means2d.shape
        assert conics.shape == (C, N, 3), conics.shape
        assert colors.shape[:2] == (C, N), colors.shape
        assert opacities.shape == (C, N), opacities.shape
        assert pix_vels.shape == (C, N, 2), pix_vels.shape
    if rolling_shutter_time is not None:
        assert rolling_shutter_time.shape == (C,), rolling_shutter_time.shape
    else:
        rolling_shutter_time = torch.zeros(C, device=device)
    if backgrounds is not None:
        assert backgrounds.shape == (C, colors.shape[-1]), backgrounds.shape
        backgrounds = backgrounds.contiguous()
    channels = colors.shape[-1]
    if channels > 513 or channels == 0:
        raise ValueError(f"Unsupported number of color channels: {channels}")
    tile_height, tile_width = isect_offsets.shape[1:3]
    assert tile_height * tile_size >= image_height, f"Assert Failed: {tile_height} * {tile_size} >= {image_height}"
    assert tile_width * tile_size >= image_width, f"Assert Failed: {tile_width} * {tile_size} >= {image_width}"

    means2d_c = means2d.contiguous()
    args = (conics.contiguous(), opacities.contiguous(), pix_vels.contiguous(),
            rolling_shutter_time.contiguous())
    tail = (image_width, image_height, tile_size, isect_offsets.contiguous(), flatten_ids.contiguous(),
            absgrad, total_follows)
    if channels <= _lib.MAX_CHANNELS:
        return _RasterizeToPixels.apply(means2d_c, args[0], colors.contiguous(), args[1], args[2],
                                        args[3], backgrounds, *tail)
    # more channels than one launch renders: chunks share geometry, alphas are identical
    renders, alphas = [], None
    for lo in range(0, channels, _lib.MAX_CHANNELS):
        hi = min(lo + _lib.MAX_CHANNELS, channels)
        bg = backgrounds[..., lo:hi].contiguous() if backgrounds is not None else None
        r, a = _RasterizeToPixels.apply(means2d_c, args[0], colors[..., lo:hi].contiguous(), args[1],
                                        args[2], args[3], bg, *tail)
        renders.append(r)
        alphas = a if alphas is None else alphas
    return torch.cat(renders, dim=-1), alphas


class _RasterizeToPixels(torch.autograd.Function):
    @staticmethod
    def forward(ctx, means2d, conics, colors, opacities, pix_vels, rolling_shutter_time, backgrounds,
                width, height, tile_size, isect_offsets, flatten_ids, absgrad, total_follows=False):
        dev = means2d.device
        assert means2d.dtype == torch.float32, means2d.dtype
        C, tile_h, tile_w = isect_offsets.shape
        channels = colors.shape[-1]
        colors_f, conics_f, opac_f, vels_f = _f(colors), _f(conics), _f(opacities), _f(pix_vels)
        rs = _f(rolling_shutter_time)
        bg = _f(backgrounds)
        render_colors = torch.empty((C, height, width, channels), dtype=torch.float32, device=dev)
        render_alphas = torch.empty((C, height, width, 1), dtype=torch.float32, device=dev)
        last_ids = torch.empty((C, height, width), dtype=torch.int32, device=dev)
        n_isects = _n_isects_arg(isect_offsets, flatten_ids, total_follows)
        _debug_check_lists("rasterize_to_pixels", flatten_ids, means2d.numel() // 2, isect_offsets, total_follows)
        ctx.n_isects_arg = n_isects
        _call(
            "splatad_rasterize_to_pixels_fwd", C, n_isects, _lib.ptr(means2d), _lib.ptr(conics_f),
            _lib.ptr(colors_f), channels, _lib.ptr(opac_f), _lib.ptr(vels_f), _lib.ptr(rs), _lib.ptr(bg),
            width, height, tile_size, tile_w, tile_h, _lib.ptr(isect_offsets), _lib.ptr(flatten_ids),
            _lib.ptr(render_colors), _lib.ptr(render_alphas), _lib.ptr(last_ids), _lib.stream_ptr(dev),
        )
        ctx.save_for_backward(means2d, conics_f, colors_f, opac_f, vels_f, rs, bg, isect_offsets,
                              flatten_ids, render_alphas, last_ids)
        ctx.width, ctx.height, ctx.tile_size, ctx.absgrad = width, height, tile_size, absgrad
        return render_colors, render_alphas

    @staticmethod
    def backward(ctx, v_render_colors, v_render_alphas):
        (means2d, conics, colors, opacities, pix_vels, rs, bg, isect_offsets, flatten_ids,
         render_alphas, last_ids) = ctx.saved_tensors
        dev = means2d.device
        C, tile_h, tile_w = isect_offsets.shape
        channels = colors.shape[-1]
        v_render_colors = _f(v_render_colors)
        v_render_alphas = _f(v_render_alphas)
        v_means2d, v_conics, v_colors, v_opacities, v_pix_vels, v_abs = _zeros_like_many(
            means2d, conics, colors, opacities, pix_vels, means2d if ctx.absgrad else None)
        _call(
            "splatad_rasterize_to_pixels_bwd", C, ctx.n_isects_arg, _lib.ptr(means2d),
            _lib.ptr(conics), _lib.ptr(colors), channels, _lib.ptr(opacities), _lib.ptr(pix_vels),
            _lib.ptr(rs), _lib.ptr(bg), ctx.width, ctx.height, ctx.tile_size, tile_w, tile_h,
            _lib.ptr(isect_offsets), _lib.ptr(flatten_ids), _lib.ptr(render_alphas), _lib.ptr(last_ids),
            _lib.ptr(v_render_colors), _lib.ptr(v_render_alphas), _lib.ptr(v_abs), _lib.ptr(v_means2d),
            _lib.ptr(v_conics), _lib.ptr(v_colors), _lib.ptr(v_opacities), _lib.ptr(v_pix_vels),
            _lib.stream_ptr(dev),
        )
        if ctx.absgrad:
            means2d.absgrad = v_abs
        v_backgrounds = None
        if ctx.needs_input_grad[6]:
            v_backgrounds = (v_render_colors * (1.0 - render_alphas).float()).sum(dim=(1, 2))
        return (v_means2d, v_conics, v_colors, v_opacities, v_pix_vels, None, v_backgrounds, None,
                None, None, None, None, None, None)


def rasterize_to_points(
    means2d: Tensor,  # [C, N, 2] or [nnz, 2]
    conics: Tensor,  # [C, N, 3] or [nnz, 3]
    lidar_features: Tensor,  # [C, N, channels] or [nnz, channels]
    opacities: Tensor,  # [C, N] or [nnz]
    pix_vels: Tensor,  # [C, N, 3] or [nnz, 3]
    depth_compensations: Tensor,  # [C, N, 2] or [nnz, 2]
    raster_pts: Tensor,  # [C, H, W, 4]
    image_width: int,
    image_height: int,
    tile_width: int,
    tile_height: int,
    isect_offsets: Tensor,  # [C, tile_height, tile_width]
    flatten_ids: Tensor,  # [n_isects]
    compute_alpha_sum_until_points: bool,
    compute_alpha_sum_until_points_threshold: float,
    backgrounds: Optional[Tensor] = None,  # [C, channels]
    packed: bool = False,
    absgrad: bool = False,
    total_follows: bool = False,  # see rasterize_to_pixels
) -> Tuple[Tensor, Tensor, Optional[Tensor], Tensor]:
    """Rasterizes Gaussians to lidar points; the last feature channel is the Gaussian's range.

    Returns (features [C,H,W,channels], alphas [C,H,W,1], alpha_sum_until_points [C,H,W,1] or
    None, median_depths [C,H,W,1]).
    """
    C = isect_offsets.size(0)
    if packed:
        nnz = means2d.size(0)
        assert means2d.shape == (nnz, 2), means2d.shape
        assert conics.shape == (nnz, 3), conics.shape
        assert lidar_features.shape[0] == nnz, lidar_features.shape
        assert opacities.shape == (nnz,), opacities.shape
        assert pix_vels.shape == (nnz, 3), pix_vels.shape
        assert depth_compensations.shape == (nnz, 2), depth_compensations.shape
    else:
        N = means2d.size(1)
        assert means2d.shape == (C, N, 2), means2d.shape
        assert conics.shape == (C, N, 3), conics.shape
        assert lidar_features.shape[:2] == (C, N), lidar_features.shape
        assert opacities.shape == (C, N), opacities.shape
        assert pix_vels.shape == (C, N, 3), pix_vels.shape
        assert depth_compensations.shape == (C, N, 2), depth_compensations.shape
    if backgrounds is not None:
        assert backgrounds.shape == (C, lidar_features.shape[-1]), backgrounds.shape
        backgrounds = backgrounds.contiguous()
    channels = lidar_features.shape[-1]
    depth_channel_idx = channels - 1
    if channels > 513 or channels == 0:
        raise ValueError(f"Unsupported number of lidar_features channels: {channels}")
    tile_grid_height, tile_grid_width = isect_offsets.shape[1:3]
    assert tile_grid_height * tile_height >= image_height, (
        f"Assert Failed: {tile_grid_height} * {tile_height} >= {image_height}")
    assert tile_grid_width * tile_width >= image_width, (
        f"Assert Failed: {tile_grid_width} * {tile_width} >= {image_width}")
    assert raster_pts.shape == (C, image_height, image_width, 4), "raster_pts does not have the correct shape"

    fixed = (means2d.contiguous(), conics.contiguous())
    mid = (opacities.contiguous(), pix_vels.contiguous(), depth_compensations.contiguous())
    tail = (raster_pts.contiguous(), image_width, image_height, tile_width, tile_height,
            isect_offsets.contiguous(), flatten_ids.contiguous(), compute_alpha_sum_until_points,
            compute_alpha_sum_until_points_threshold, absgrad)
    if channels <= _lib.MAX_CHANNELS:
        return _RasterizeToPoints.apply(*fixed, lidar_features.contiguous(), None, *mid, backgrounds, *tail,
                                        depth_channel_idx, total_follows)
    # more channels than one launch renders: every chunk carries the range as its last channel
    step = _lib.MAX_CHANNELS - 1
    n_feat = channels - 1
    depth = lidar_features[..., -1:]
    outs, first = [], None
    for lo in range(0, n_feat, step):
        hi = min(lo + step, n_feat)
        feats = torch.cat([lidar_features[..., lo:hi], depth], dim=-1).contiguous()
        bg = None
        if backgrounds is not None:
            bg = torch.cat([backgrounds[..., lo:hi], backgrounds[..., -1:]], dim=-1).contiguous()
        r, a, s, m = _RasterizeToPoints.apply(*fixed, feats, None, *mid, bg, *tail, feats.shape[-1] - 1,
                                              total_follows)
        if first is None:
            first = (a, s, m)
        outs.append(r if hi == n_feat else r[..., :-1])
    return torch.cat(outs, dim=-1), first[0], first[1], first[2]


def rasterize_to_points_split(
    means2d: Tensor, conics: Tensor, lidar_features: Tensor, ranges: Tensor, opacities: Tensor,
    pix_vels: Tensor, depth_compensations: Tensor, raster_pts: Tensor, image_width: int, image_height: int,
    tile_width: int, tile_height: int, isect_offsets: Tensor, flatten_ids: Tensor,
    compute_alpha_sum_until_points: bool, compute_alpha_sum_until_points_threshold: float,
    absgrad: bool = False, total_follows: bool = False, frame: Optional["LidarFrame"] = None,
) -> Tuple[Tensor, Tensor, Optional[Tensor], Tensor]:
    """:func:`rasterize_to_points` with the Gaussians' ranges given as their own [C,N] tensor instead
    of being concatenated to the features as last channel (what ``lidar_rasterization`` of the
    reference does per frame, gsplat/rendering.py:746, 779): same outputs, D + 1 <= 32 channels, no
    [C,N,D+1] copy. Not part of the reference's API; used by ``splatad_b200.lidar_rasterization``."""
    assert lidar_features.shape[-1] + 1 <= _lib.MAX_CHANNELS
    assert ranges.shape == lidar_features.shape[:-1], (ranges.shape, lidar_features.shape)
    return _RasterizeToPoints.apply(
        means2d.contiguous(), conics.contiguous(), lidar_features.contiguous(), ranges.contiguous(),
        opacities.contiguous(), pix_vels.contiguous(), depth_compensations.contiguous(), None,
        raster_pts.contiguous(), image_width, image_height, tile_width, tile_height,
        isect_offsets.contiguous(), flatten_ids.contiguous(), compute_alpha_sum_until_points,
        compute_alpha_sum_until_points_threshold, absgrad, lidar_features.shape[-1], total_follows, frame)


class _RasterizeToPoints(torch.autograd.Function):
    @staticmethod
    def forward(ctx, means2d, conics, colors, ranges, opacities, pix_vels, depth_compensations, backgrounds,
                raster_pts, width, height, tile_width, tile_height, isect_offsets, flatten_ids,
                compute_alpha_sum_until_points, compute_alpha_sum_until_points_threshold, absgrad,
                depth_channel_idx, total_follows=False, frame=None):
        # ``frame`` (optional): a LidarFrame that has composited exactly these inputs over exactly
        # these lists; its images are returned with this op's backward attached, nothing is launched.
        # ``ranges`` (optional, [C,N] / [nnz]): the Gaussians' ranges as a separate array; the rendered
        # channel count is then colors.shape[-1] + 1 with the range as last channel.
        dev = means2d.device
        assert means2d.dtype == torch.float32, means2d.dtype
        C, grid_h, grid_w = isect_offsets.shape
        channels = colors.shape[-1] + (1 if ranges is not None else 0)
        ranges_f = _f(ranges)
        colors_f, conics_f, opac_f = _f(colors), _f(conics), _f(opacities)
        vels_f, dc_f, pts_f, bg = _f(pix_vels), _f(depth_compensations), _f(raster_pts), _f(backgrounds)
        f32 = dict(dtype=torch.float32, device=dev)
        ctx.n_isects_arg = _n_isects_arg(isect_offsets, flatten_ids, total_follows)
        _debug_check_lists("rasterize_to_points", flatten_ids, means2d.numel() // 2, isect_offsets, total_follows)
        if frame is not None:
            render_colors, render_alphas, median_depths = frame.render, frame.alphas, frame.median_depths
            alpha_sum, last_ids = frame.alpha_sum, frame.last_ids
            assert render_colors.shape == (C, height, width, channels) and ranges is not None and bg is None
        else:
            render_colors = torch.empty((C, height, width, channels), **f32)
            render_alphas = torch.empty((C, height, width, 1), **f32)
            median_depths = torch.empty((C, height, width, 1), **f32)
            alpha_sum = torch.empty((C, height, width, 1), **f32) if compute_alpha_sum_until_points else None
            last_ids = torch.empty((C, height, width), dtype=torch.int32, device=dev)
            _call(
                "splatad_rasterize_to_points_fwd", C, ctx.n_isects_arg, _lib.ptr(means2d),
                _lib.ptr(conics_f), _lib.ptr(colors_f) if colors_f.numel() else None, _lib.ptr(ranges_f), channels,
                _lib.ptr(opac_f), _lib.ptr(vels_f),
                _lib.ptr(dc_f), _lib.ptr(bg), _lib.ptr(pts_f), width, height, tile_width, tile_height,
                grid_w, grid_h, int(bool(compute_alpha_sum_until_points)),
                float(compute_alpha_sum_until_points_threshold), _lib.ptr(isect_offsets),
                _lib.ptr(flatten_ids), depth_channel_idx, _lib.ptr(render_colors), _lib.ptr(render_alphas),
                _lib.ptr(alpha_sum), _lib.ptr(last_ids), _lib.ptr(median_depths), _lib.stream_ptr(dev),
            )
        ctx.save_for_backward(means2d, conics_f, colors_f, ranges_f, opac_f, vels_f, dc_f, bg, pts_f,
                              isect_offsets, flatten_ids, render_alphas, last_ids)
        ctx.meta = (width, height, tile_width, tile_height, absgrad,
                    bool(compute_alpha_sum_until_points),
                    float(compute_alpha_sum_until_points_threshold), depth_channel_idx)
        ctx.mark_non_differentiable(median_depths)
        return render_colors, render_alphas, alpha_sum, median_depths

    @staticmethod
    def backward(ctx, v_render_colors, v_render_alphas, v_alpha_sum, v_median_depths):
        (means2d, conics, colors, ranges, opacities, pix_vels, depth_comps, bg, raster_pts, isect_offsets,
         flatten_ids, render_alphas, last_ids) = ctx.saved_tensors
        width, height, tile_width, tile_height, absgrad, compute_asum, thr, depth_idx = ctx.meta
        dev = means2d.device
        C, grid_h, grid_w = isect_offsets.shape
        channels = colors.shape[-1] + (1 if ranges is not None else 0)
        v_render_colors = _f(v_render_colors)
        v_render_alphas = _f(v_render_alphas)
        v_asum = _f(v_alpha_sum) if (compute_asum and v_alpha_sum is not None) else None
        v_means2d, v_conics, v_colors, v_opacities, v_pix_vels, v_depth_comps, v_ranges, v_abs = _zeros_like_many(
            means2d, conics, colors, opacities, pix_vels, depth_comps, ranges, means2d if absgrad else None)
        _call(
            "splatad_rasterize_to_points_bwd", C, ctx.n_isects_arg, _lib.ptr(means2d),
            _lib.ptr(conics), _lib.ptr(colors) if colors.numel() else None, _lib.ptr(ranges), channels,
            _lib.ptr(opacities), _lib.ptr(pix_vels),
            _lib.ptr(depth_comps), _lib.ptr(bg), _lib.ptr(raster_pts), width, height, tile_width,
            tile_height, grid_w, grid_h, int(compute_asum), thr, _lib.ptr(isect_offsets),
            _lib.ptr(flatten_ids), depth_idx, _lib.ptr(render_alphas), _lib.ptr(last_ids),
            _lib.ptr(v_render_colors), _lib.ptr(v_render_alphas), _lib.ptr(v_asum), _lib.ptr(v_abs),
            _lib.ptr(v_means2d), _lib.ptr(v_conics), _lib.ptr(v_colors) if v_colors.numel() else None,
            _lib.ptr(v_opacities), _lib.ptr(v_pix_vels), _lib.ptr(v_depth_comps), _lib.ptr(v_ranges),
            _lib.stream_ptr(dev),
        )
        if absgrad:
            means2d.absgrad = v_abs
        v_backgrounds = None
        if ctx.needs_input_grad[7]:
            v_backgrounds = (v_render_colors * (1.0 - render_alphas).float()).sum(dim=(1, 2))
        return (v_means2d, v_conics, v_colors, v_ranges, v_opacities, v_pix_vels, v_depth_comps,
                v_backgrounds) + (None,) * 13


# =============================================================================================
# Indices of contributing (Gaussian, pixel) pairs
# =============================================================================================
_RANGE_MAX = 2 ** 32 - 1   # the range arguments are uint32 in the reference's kernels


def _indices_in_range(kind, range_start, range_end, transmittances, means2d, conics, opacities, pix_vels,
                      sensor, image_width, image_height, tile_w, tile_h, isect_offsets, flatten_ids):
    C, N, _ = means2d.shape
    dev = means2d.device
    grid_h, grid_w = isect_offsets.shape[1:3]
    n_isects = _n_isects_arg(isect_offsets, flatten_ids)
    offs = isect_offsets if isect_offsets.dtype == torch.int32 and isect_offsets.is_contiguous() \
        else isect_offsets.to(torch.int32).contiguous()
    flat = flatten_ids.to(torch.int32).contiguous()
    tensors = tuple(_f(x) for x in (transmittances, means2d, conics, opacities, pix_vels, sensor))
    n_pix = C * image_height * image_width
    empty = torch.empty(0, dtype=torch.int64, device=dev)
    if n_pix == 0 or flat.numel() == 0:
        return empty, empty.clone(), empty.clone()
    lib = _lib.load()
    ws = _lib.workspace("indices", lib.splatad_rasterize_to_indices_workspace_bytes(C, image_width, image_height), dev)
    starts = torch.empty(n_pix + 1, dtype=torch.int64, device=dev)
    total = ctypes.c_int64(0)
    head = (min(max(int(range_start), 0), _RANGE_MAX), min(max(int(range_end), 0), _RANGE_MAX), C, N, n_isects,
            *(_lib.ptr(x) for x in tensors), image_width, image_height)
    grid = (tile_w, grid_w, grid_h) if kind == "camera" else (tile_w, tile_h, grid_w, grid_h)
    name = "splatad_rasterize_to_indices_in_range" + ("" if kind == "camera" else "_lidar")
    _call(name + "_count", *head, *grid, _lib.ptr(offs), _lib.ptr(flat), _lib.ptr(ws), ws.numel(),
          _lib.ptr(starts), ctypes.addressof(total), _lib.stream_ptr(dev))
    m = int(total.value)
    gaussian_ids = torch.empty(m, dtype=torch.int64, device=dev)
    pixel_ids = torch.empty(m, dtype=torch.int64, device=dev)
    camera_ids = torch.empty(m, dtype=torch.int64, device=dev)
    if m:
        _call(name + "_write", *head, *grid, _lib.ptr(offs), _lib.ptr(flat), _lib.ptr(starts),
              _lib.ptr(gaussian_ids), _lib.ptr(pixel_ids), _lib.ptr(camera_ids), _lib.stream_ptr(dev))
    return gaussian_ids, pixel_ids, camera_ids


@torch.no_grad()
def rasterize_to_indices_in_range(
    range_start: int,
    range_end: int,
    transmittances: Tensor,  # [C, image_height, image_width]
    means2d: Tensor,  # [C, N, 2]
    conics: Tensor,  # [C, N, 3]
    opacities: Tensor,  # [C, N]
    pix_vels: Tensor,  # [C, N, 2]
    image_width: int,
    image_height: int,
    tile_size: int,
    isect_offsets: Tensor,  # [C, tile_height, tile_width]
    flatten_ids: Tensor,  # [n_isects]
    rolling_shutter_time: Optional[Tensor] = None,  # [C]
) -> Tuple[Tensor, Tensor, Tensor]:
    """Lists the (Gaussian, pixel, camera) triples that contribute to the image within list batches
    ``[range_start, range_end)`` (a batch is ``tile_size ** 2`` entries of a tile's list), starting
    from the given transmittances: ``gsplat.cuda._wrapper.rasterize_to_indices_in_range``
    (gsplat/cuda/_wrapper.py:1115-1196). Returns int64 (gaussian_ids, pixel_ids, camera_ids), each
    [M], ordered by camera, pixel (row-major) and list position."""
    C, N, _ = means2d.shape
    assert conics.shape == (C, N, 3), conics.shape
    assert opacities.shape == (C, N), opacities.shape
    assert isect_offsets.shape[0] == C, isect_offsets.shape
    assert pix_vels.shape == (C, N, 2), pix_vels.shape
    assert transmittances.shape == (C, image_height, image_width), transmittances.shape
    if rolling_shutter_time is not None:
        assert rolling_shutter_time.shape == (C,), rolling_shutter_time.shape
    else:
        rolling_shutter_time = torch.zeros(C, device=means2d.device)
    tile_height, tile_width = isect_offsets.shape[1:3]
    assert tile_height * tile_size >= image_height, f"Assert Failed: {tile_height} * {tile_size} >= {image_height}"
    assert tile_width * tile_size >= image_width, f"Assert Failed: {tile_width} * {tile_size} >= {image_width}"
    return _indices_in_range("camera", range_start, range_end, transmittances, means2d, conics, opacities,
                             pix_vels, rolling_shutter_time, image_width, image_height, tile_size, tile_size,
                             isect_offsets, flatten_ids)


@torch.no_grad()
def rasterize_to_indices_in_range_lidar(
    range_start: int,
    range_end: int,
    transmittances: Tensor,  # [C, image_height, image_width]
    means2d: Tensor,  # [C, N, 2]
    conics: Tensor,  # [C, N, 3]
    opacities: Tensor,  # [C, N]
    pix_vels: Tensor,  # [C, N, 3]
    raster_pts: Tensor,  # [C, image_height, image_width, 4]
    image_width: int,
    image_height: int,
    tile_width: int,
    tile_height: int,
    isect_offsets: Tensor,  # [C, tile grid height, tile grid width]
    flatten_ids: Tensor,  # [n_isects]
) -> Tuple[Tensor, Tensor, Tensor]:
    """Lidar twin of :func:`rasterize_to_indices_in_range` (gsplat/cuda/_wrapper.py:1198-1281): a
    batch is ``tile_width * tile_height`` entries, points with range <= 0 list nothing."""
    C, N, _ = means2d.shape
    assert conics.shape == (C, N, 3), conics.shape
    assert opacities.shape == (C, N), opacities.shape
    assert isect_offsets.shape[0] == C, isect_offsets.shape
    assert pix_vels.shape == (C, N, 3), pix_vels.shape
    assert transmittances.shape == (C, image_height, image_width), transmittances.shape
    assert raster_pts.shape == (C, image_height, image_width, 4), raster_pts.shape
    tile_grid_height, tile_grid_width = isect_offsets.shape[1:3]
    assert tile_grid_height * tile_height >= image_height, \
        f"Assert Failed: {tile_grid_height} * {tile_height} >= {image_height}"
    assert tile_grid_width * tile_width >= image_width, \
        f"Assert Failed: {tile_grid_width} * {tile_width} >= {image_width}"
    return _indices_in_range("lidar", range_start, range_end, transmittances, means2d, conics, opacities,
                             pix_vels, raster_pts, image_width, image_height, tile_width, tile_height,
                             isect_offsets, flatten_ids)


@torch.no_grad()
def count_composited_pairs(
    means2d: Tensor,  # [C, N, 2] or [nnz, 2]
    conics: Tensor,
    opacities: Tensor,
    pix_vels: Tensor,  # [..., 2] camera, [..., 3] lidar
    isect_offsets: Tensor,  # [C, tile rows, tile columns]
    flatten_ids: Tensor,
    image_width: int,
    image_height: int,
    tile_width: int,
    tile_height: int,
    rolling_shutter_time: Optional[Tensor] = None,  # [C]: camera
    raster_pts: Optional[Tensor] = None,  # [C, H, W, 4]: lidar
) -> Tuple[int, int]:
    """(tested, contributing) pair counts of a frame: how many (pixel, Gaussian) pairs the
    compositing evaluates before every pixel has stopped, and how many of them it blends. A
    measurement aid for the compositing flop model (not part of the reference's API); ``raster_pts``
    selects the lidar rules, otherwise ``rolling_shutter_time`` (zeros if missing) the camera's."""
    C, grid_h, grid_w = isect_offsets.shape
    dev = means2d.device
    lidar = raster_pts is not None
    n_pix = C * image_height * image_width
    counters = torch.zeros(2, dtype=torch.int64, device=dev)
    if n_pix == 0 or flatten_ids.numel() == 0:
        return 0, 0
    ones = torch.ones((C, image_height, image_width), dtype=torch.float32, device=dev)
    per_pixel = torch.empty(n_pix, dtype=torch.int32, device=dev)
    flat = flatten_ids.to(torch.int32).contiguous()
    offs = isect_offsets.to(torch.int32).contiguous()
    n_rows = means2d.numel() // 2
    head = (C, max(n_rows // max(C, 1), 1), flat.numel(), _lib.ptr(ones), _lib.ptr(_f(means2d)), _lib.ptr(_f(conics)),
            _lib.ptr(_f(opacities)), _lib.ptr(_f(pix_vels)))
    tail = (_lib.ptr(offs), _lib.ptr(flat), _lib.ptr(per_pixel), _lib.ptr(counters), _lib.stream_ptr(dev))
    if lidar:
        _call("splatad_count_composited_pairs_lidar", *head, _lib.ptr(_f(raster_pts)), image_width, image_height,
              tile_width, tile_height, grid_w, grid_h, *tail)
    else:
        assert tile_width == tile_height
        rs = _f(rolling_shutter_time) if rolling_shutter_time is not None else torch.zeros(C, device=dev)
        _call("splatad_count_composited_pairs", *head, _lib.ptr(rs), image_width, image_height, tile_width, grid_w,
              grid_h, *tail)
    tested, contributing = counters.tolist()
    return int(tested), int(contributing)
