"""Generates the golden fixtures in this directory by running the REFERENCE's own PyTorch
implementation (gsplat/cuda/_torch_impl.py of carlinds/splatad) on the CPU.

Run once, in a container where the reference is mounted:

    PYTHONPATH=<reference root> PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py

The reference cannot travel to the GPU machine, the ``.npz`` files written here can. Every file
holds the seeded inputs and the reference outputs of one function. The compositing fixtures
drive the reference's ``accumulate`` / ``accumulate_lidar`` on explicit (pixel, Gaussian) pair
lists; those two functions import ``nerfacc`` (an unpinned dependency of the reference that is
not installed anywhere here), so its two helpers are restated below from their published
definitions:

  render_weight_from_alpha(alphas, ray_indices, n_rays) -> (w_i, T_i) with
      T_i = prod over earlier samples j of the same ray of (1 - alpha_j),  w_i = alpha_i * T_i
  accumulate_along_rays(weights, values, ray_indices, n_rays) -> out[r] = sum_i w_i * values_i
      over the samples of ray r (values None -> the weights themselves, one column).
"""

import math
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _install_nerfacc_stub():
    mod = types.ModuleType("nerfacc")

    def render_weight_from_alpha(alphas, ray_indices=None, n_rays=None):
        trans = torch.ones_like(alphas)
        run = {}
        for i in range(alphas.numel()):
            r = int(ray_indices[i])
            t = run.get(r, torch.ones((), dtype=alphas.dtype))
            trans[i] = t
            run[r] = t * (1 - alphas[i])
        return alphas * trans, trans

    def accumulate_along_rays(weights, values, ray_indices=None, n_rays=None):
        if values is None:
            values = torch.ones(weights.shape[0], 1, dtype=weights.dtype)
        out = torch.zeros(n_rays, values.shape[-1], dtype=weights.dtype)
        out.index_add_(0, ray_indices, weights[:, None] * values)
        return out

    mod.render_weight_from_alpha = render_weight_from_alpha
    mod.accumulate_along_rays = accumulate_along_rays
    sys.modules["nerfacc"] = mod


def save(name, **arrays):
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().cpu().numpy()
        out[k] = np.asarray(v)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print("wrote", name, {k: tuple(v.shape) for k, v in out.items()})


def rand_rigid(g, C, spread=1.0):
    """C world->sensor matrices: random rotations (QR) and small translations."""
    mats = []
    for _ in range(C):
        q, _ = torch.linalg.qr(torch.randn(3, 3, generator=g))
        if torch.det(q) < 0:
            q[:, 0] = -q[:, 0]
        M = torch.eye(4)
        M[:3, :3] = q
        M[:3, 3] = torch.randn(3, generator=g) * spread
        mats.append(M)
    return torch.stack(mats)


def main():
    from gsplat.cuda import _torch_impl as ref

    _install_nerfacc_stub()

    # ------------------------------------------------------------------ quat/scale -> covariance
    g = torch.Generator().manual_seed(100)
    quats = torch.randn(64, 4, generator=g)
    scales = torch.rand(64, 3, generator=g) * 0.5 + 0.05
    covars, _ = ref._quat_scale_to_covar_preci(quats, scales, True, False, False)
    save("quat_scale_to_covar", quats=quats, scales=scales, covars=covars)

    # ------------------------------------------------------------------ lidar projection
    g = torch.Generator().manual_seed(101)
    N, C = 600, 2
    means = torch.empty(N, 3)
    means[:, 0] = torch.rand(N, generator=g) * 60 - 30
    means[:, 1] = torch.rand(N, generator=g) * 60 - 30
    means[:, 2] = torch.rand(N, generator=g) * 8 - 3
    quats = torch.randn(N, 4, generator=g)
    scales = torch.exp(torch.randn(N, 3, generator=g) * 0.5 - 1.0)
    velocities = torch.randn(N, 3, generator=g) * 2
    viewmats = rand_rigid(g, C)
    # keep the sensors roughly upright so elevations stay inside the supported band
    for c in range(C):
        yaw = float(torch.rand(1, generator=g)) * 2 * math.pi
        cy, sy = math.cos(yaw), math.sin(yaw)
        viewmats[c, :3, :3] = torch.tensor([[cy, sy, 0.0], [-sy, cy, 0.0], [0.0, 0.0, 1.0]])
    lin = torch.randn(C, 3, generator=g) * 5
    ang = torch.randn(C, 3, generator=g) * 0.2
    rs = torch.tensor([0.1, 0.0])
    covars, _ = ref._quat_scale_to_covar_preci(quats, scales, True, False, False)
    kw = dict(min_elevation=-30.0, max_elevation=25.0, min_azimuth=-180.0, max_azimuth=180.0, eps2d=0.017,
              near_plane=0.5, far_plane=60.0, calc_compensations=True)
    radii, means2d, depths, conics, comps, pix_vels, depth_comp = ref._fully_fused_lidar_projection(
        means, covars, velocities, viewmats, lin, ang, rs, **kw)
    save("lidar_projection", means=means, quats=quats, scales=scales, velocities=velocities,
         viewmats=viewmats, lin=lin, ang=ang, rs=rs, radii=radii, means2d=means2d, depths=depths,
         conics=conics, compensations=comps, pix_vels=pix_vels, depth_compensations=depth_comp,
         **{k: np.float64(v) for k, v in kw.items() if k != "calc_compensations"})

    # ------------------------------------------------------------------ camera projection
    g = torch.Generator().manual_seed(102)
    N, C = 600, 2
    means = torch.empty(N, 3)
    means[:, 0] = torch.rand(N, generator=g) * 40 - 20
    means[:, 1] = torch.rand(N, generator=g) * 10 - 5
    means[:, 2] = torch.rand(N, generator=g) * 60 - 10
    quats = torch.randn(N, 4, generator=g)
    scales = torch.exp(torch.randn(N, 3, generator=g) * 0.7 - 1.5)
    velocities = torch.randn(N, 3, generator=g) * 2
    viewmats = torch.eye(4)[None].repeat(C, 1, 1)
    viewmats[1, :3, 3] = torch.tensor([0.5, -0.2, 1.0])
    c1, s1 = math.cos(0.2), math.sin(0.2)
    viewmats[1, :3, :3] = torch.tensor([[c1, 0.0, s1], [0.0, 1.0, 0.0], [-s1, 0.0, c1]])
    Ks = torch.tensor([[[300.0, 0.0, 160.0], [0.0, 310.0, 120.0], [0.0, 0.0, 1.0]]]).repeat(C, 1, 1)
    W, H = 320, 240
    lin = torch.tensor([[10.0, 0.0, 0.0], [0.0, 0.0, 3.0]])
    ang = torch.tensor([[0.0, 0.1, 0.0], [0.05, 0.0, -0.1]])
    rs = torch.tensor([0.03, 0.0])
    covars, _ = ref._quat_scale_to_covar_preci(quats, scales, True, False, False)
    radii, means2d, depths, conics, comps, pix_vels = ref._fully_fused_projection(
        means, covars, velocities, viewmats, Ks, W, H, lin, ang, rs, eps2d=0.3, near_plane=0.2,
        far_plane=45.0, calc_compensations=True)
    save("camera_projection", means=means, quats=quats, scales=scales, velocities=velocities,
         viewmats=viewmats, Ks=Ks, width=W, height=H, lin=lin, ang=ang, rs=rs, radii=radii,
         means2d=means2d, depths=depths, conics=conics, compensations=comps, pix_vels=pix_vels,
         eps2d=0.3, near_plane=0.2, far_plane=45.0)

    # ------------------------------------------------------------------ isect (camera), as tests/test_basic.py:698-723
    torch.manual_seed(42)
    C, N = 3, 1000
    width, height = 40, 60
    means2d = torch.randn(C, N, 2) * width
    radii = torch.randint(0, width, (C, N, 2), dtype=torch.int32)
    depths = torch.rand(C, N)
    tile_size = 16
    tile_width = math.ceil(width / tile_size)
    tile_height = math.ceil(height / tile_size)
    tpg, ids, flat = ref._isect_tiles(means2d, radii, depths, tile_size, tile_width, tile_height)
    offs = ref._isect_offset_encode(ids, C, tile_width, tile_height)
    save("isect_tiles", means2d=means2d, radii=radii, depths=depths, tile_size=tile_size,
         tile_width=tile_width, tile_height=tile_height, tiles_per_gauss=tpg, isect_ids=ids,
         flatten_ids=flat, isect_offsets=offs)

    # ------------------------------------------------------------------ isect (lidar), as tests/test_basic.py:727-766
    torch.manual_seed(42)
    C, N = 3, 100
    width, height = 360.0, 90.0
    min_azimuth = -180
    tile_azim_resolution = 0.2 * 16
    n_azim_tiles = math.ceil(360 / tile_azim_resolution)
    n_elev_tiles = 16
    elev_boundaries = torch.linspace(-height / 2.0, height / 2.0, n_elev_tiles + 1)
    means2d = torch.zeros((C, N, 2))
    means2d[:, :, 0] = torch.rand(C, N) * width - width / 2
    means2d[:, :, 1] = torch.rand(C, N) * height - height / 2
    radii = torch.rand(C, N, 2, dtype=torch.float32) / 2
    depths = torch.rand(C, N)
    tpg, ids, flat = ref._isect_lidar_tiles(means2d, radii, depths, elev_boundaries, tile_azim_resolution, min_azimuth)
    offs = ref._isect_offset_encode(ids, C, n_azim_tiles, n_elev_tiles)
    save("isect_lidar_tiles", means2d=means2d, radii=radii, depths=depths, elev_boundaries=elev_boundaries,
         tile_azim_resolution=tile_azim_resolution, min_azimuth=min_azimuth, n_azim_tiles=n_azim_tiles,
         n_elev_tiles=n_elev_tiles, tiles_per_gauss=tpg, isect_ids=ids, flatten_ids=flat, isect_offsets=offs)

    # a second lidar case with large radii: wrap-around on both sides of the azimuth range
    torch.manual_seed(43)
    C, N = 2, 300
    means2d = torch.zeros((C, N, 2))
    means2d[:, :, 0] = torch.rand(C, N) * 360 - 180
    means2d[:, :, 1] = torch.rand(C, N) * 50 - 30
    radii = torch.rand(C, N, 2) * torch.tensor([40.0, 6.0])
    radii[:, ::7, 0] = 0.0
    depths = torch.rand(C, N) * 80
    depths[:, 1::5] = depths[:, 0::5][:, : depths[:, 1::5].shape[1]]  # ties in depth
    elev_boundaries = torch.tensor([-26.0, -20.5, -14.0, -6.5, -2.0, 1.5, 6.0, 16.0])
    tile_azim_resolution = 6.4
    # The fixture contains equal (tile, depth) keys. The reference CUDA path sorts them with a
    # stable radix sort (ties stay in flatten-index order) whereas the torch twin's torch.sort is
    # not stable, so the unsorted emission of the reference is sorted stably here.
    tpg, ids, flat = ref._isect_lidar_tiles(means2d, radii, depths, elev_boundaries, tile_azim_resolution, -180.0,
                                            sort=False)
    ids, order = torch.sort(ids, stable=True)
    flat = flat[order]
    n_azim_tiles = math.ceil(360 / tile_azim_resolution)
    offs = ref._isect_offset_encode(ids, C, n_azim_tiles, 7)
    save("isect_lidar_tiles_wrap", means2d=means2d, radii=radii, depths=depths, elev_boundaries=elev_boundaries,
         tile_azim_resolution=tile_azim_resolution, min_azimuth=-180.0, n_azim_tiles=n_azim_tiles,
         n_elev_tiles=7, tiles_per_gauss=tpg, isect_ids=ids, flatten_ids=flat, isect_offsets=offs)

    # ------------------------------------------------------------------ spherical harmonics
    g = torch.Generator().manual_seed(103)
    dirs = torch.randn(200, 3, generator=g)
    coeffs = torch.randn(200, 25, 3, generator=g)
    out = {f"colors_deg{d}": ref._spherical_harmonics(d, dirs, coeffs) for d in range(5)}
    save("spherical_harmonics", dirs=dirs, coeffs=coeffs, **out)

    # ------------------------------------------------------------------ compositing arithmetic (camera)
    g = torch.Generator().manual_seed(104)
    C, N, W, H, ch = 2, 10, 6, 4, 5
    means2d = torch.rand(C, N, 2, generator=g) * torch.tensor([W, H])
    sig = torch.rand(C, N, 2, generator=g) * 3 + 4  # broad Gaussians: every pair stays above 1/255
    rho = torch.rand(C, N, generator=g) * 0.6 - 0.3
    cov = torch.stack([sig[..., 0] ** 2, rho * sig[..., 0] * sig[..., 1], rho * sig[..., 0] * sig[..., 1],
                       sig[..., 1] ** 2], dim=-1).reshape(C, N, 2, 2)
    inv = torch.linalg.inv(cov)
    conics = torch.stack([inv[..., 0, 0], inv[..., 0, 1], inv[..., 1, 1]], dim=-1)
    opac = torch.rand(C, N, generator=g) * 0.3 + 0.1
    colors = torch.randn(C, N, ch, generator=g)
    pix_vels = torch.randn(C, N, 2, generator=g) * 5
    rs = torch.tensor([0.03, 0.0])
    cam_ids = torch.arange(C).repeat_interleave(W * H * N)
    pix_ids = torch.arange(W * H).repeat_interleave(N).repeat(C)
    g_ids = torch.arange(N).repeat(C * W * H)
    renders, alphas = ref.accumulate(means2d, conics, opac, colors, pix_vels, rs, g_ids, pix_ids, cam_ids, W, H)
    save("accumulate_pixels", means2d=means2d, conics=conics, opacities=opac, colors=colors, pix_vels=pix_vels,
         rs=rs, width=W, height=H, renders=renders, alphas=alphas)

    # ------------------------------------------------------------------ compositing arithmetic (lidar)
    g = torch.Generator().manual_seed(105)
    C, N, W, H, ch = 2, 10, 8, 4, 4
    az = torch.linspace(-179.0, 179.0, W)  # spans the +-180 seam so the wrap is exercised
    el = torch.linspace(-10.0, 10.0, H)
    raster_pts = torch.zeros(C, H, W, 4)
    raster_pts[..., 0] = az[None, None, :]
    raster_pts[..., 1] = el[None, :, None]
    raster_pts[..., 2] = torch.rand(C, H, W, generator=g) * 60 + 5
    raster_pts[..., 3] = (torch.rand(C, H, W, generator=g) - 0.5) * 0.1
    means2d = torch.stack([torch.rand(C, N, generator=g) * 360 - 180, torch.rand(C, N, generator=g) * 20 - 10], dim=-1)
    sig = torch.stack([torch.rand(C, N, generator=g) * 60 + 150, torch.rand(C, N, generator=g) * 6 + 12], dim=-1)
    rho = torch.rand(C, N, generator=g) * 0.4 - 0.2
    cov = torch.stack([sig[..., 0] ** 2, rho * sig[..., 0] * sig[..., 1], rho * sig[..., 0] * sig[..., 1],
                       sig[..., 1] ** 2], dim=-1).reshape(C, N, 2, 2)
    inv = torch.linalg.inv(cov)
    conics = torch.stack([inv[..., 0, 0], inv[..., 0, 1], inv[..., 1, 1]], dim=-1)
    opac = torch.rand(C, N, generator=g) * 0.3 + 0.1
    feats = torch.randn(C, N, ch, generator=g)
    feats[..., -1] = torch.rand(C, N, generator=g) * 70  # range channel
    pix_vels = torch.randn(C, N, 3, generator=g) * 3
    depth_comps = torch.randn(C, N, 2, generator=g) * 0.05
    cam_ids = torch.arange(C).repeat_interleave(W * H * N)
    pix_ids = torch.arange(W * H).repeat_interleave(N).repeat(C)
    g_ids = torch.arange(N).repeat(C * W * H)
    renders, alphas, asum = ref.accumulate_lidar(means2d, conics, opac, feats, pix_vels, depth_comps, raster_pts,
                                                 g_ids, pix_ids, cam_ids, W, H, True, 0.5)
    save("accumulate_points", means2d=means2d, conics=conics, opacities=opac, features=feats, pix_vels=pix_vels,
         depth_compensations=depth_comps, raster_pts=raster_pts, width=W, height=H, threshold=0.5,
         renders=renders, alphas=alphas, alpha_sum=asum)

    # ------------------------------------------------------------------ unfused ops
    g = torch.Generator().manual_seed(110)
    N, C = 300, 2
    quats = torch.randn(N, 4, generator=g)
    scales = torch.exp(torch.randn(N, 3, generator=g) * 0.5 - 1.0)
    covars, precis = ref._quat_scale_to_covar_preci(quats, scales, True, True, False)
    covars_triu, precis_triu = ref._quat_scale_to_covar_preci(quats, scales, True, True, True)
    means = torch.empty(N, 3)
    means[:, 0] = torch.rand(N, generator=g) * 30 - 15
    means[:, 1] = torch.rand(N, generator=g) * 12 - 6
    means[:, 2] = torch.rand(N, generator=g) * 40 + 1.0
    viewmats = rand_rigid(g, C, spread=0.3)
    means_c, covars_c = ref._world_to_cam(means, covars, viewmats)
    means_c[..., 2] = means_c[..., 2].abs() + 0.5      # in front of the sensor for the pinhole ops
    Ks = torch.tensor([[[300.0, 0.0, 160.0], [0.0, 310.0, 120.0], [0.0, 0.0, 1.0]]]).repeat(C, 1, 1)
    W, H = 320, 240
    lin = torch.randn(C, 3, generator=g) * 5
    ang = torch.randn(C, 3, generator=g) * 0.2
    vel_c = torch.randn(C, N, 3, generator=g) * 2
    means2d, covars2d = ref._persp_proj(means_c, covars_c, Ks, W, H)
    pix_vel = ref._compute_pix_velocity(means_c, lin, ang, vel_c, Ks, W, H)
    l_means2d, l_covars2d, _, l_depth_comp = ref._lidar_proj(means_c, covars_c, 0.017)
    lidar_vel = ref._compute_lidar_velocity(means_c, lin, ang, vel_c)
    save("unfused_ops", quats=quats, scales=scales, covars=covars, precis=precis, covars_triu=covars_triu,
         precis_triu=precis_triu, means=means, viewmats=viewmats, means_c=means_c, covars_c=covars_c, Ks=Ks,
         width=np.int64(W), height=np.int64(H), lin=lin, ang=ang, vel_c=vel_c, means2d=means2d,
         covars2d=covars2d, pix_vel=pix_vel, lidar_means2d=l_means2d, lidar_covars2d=l_covars2d,
         lidar_depth_comp=l_depth_comp, lidar_vel=lidar_vel, eps2d=np.float64(0.017))


    # ------------------------------------------------------------------ densification statistics
    # DefaultStrategy._update_state (gsplat/strategy/default.py:203-258) is pure torch: two frames
    # accumulated in the [C, N] layout (grad and absgrad), and one in the packed layout whose
    # Gaussian ids are unique, so that the reference's indexed radii assignment is well defined
    # (it keeps an arbitrary candidate when a Gaussian appears twice).
    from gsplat.strategy.default import DefaultStrategy

    g = torch.Generator().manual_seed(120)
    C, N, W, H = 3, 400, 320, 200
    out = {}
    for absgrad in (False, True):
        strat = DefaultStrategy(absgrad=absgrad, refine_scale2d_stop_iter=0)
        state = strat.initialize_state()
        params = {"means": torch.zeros(N, 3)}
        for frame in range(2):
            radii = torch.randint(0, 40, (C, N, 2), generator=g, dtype=torch.int32)
            radii[torch.rand(C, N, generator=g) < 0.4] = 0
            means2d = torch.randn(C, N, 2, generator=g)
            means2d.grad = torch.randn(C, N, 2, generator=g) * 1e-3
            means2d.absgrad = means2d.grad.abs() * 1.5
            info = dict(width=W, height=H, n_cameras=C, radii=radii, gaussian_ids=None, means2d=means2d)
            strat._update_state(params, state, info, packed=False)
            tag = f"{'abs' if absgrad else 'grad'}_f{frame}"
            out.update({f"{tag}_radii": radii, f"{tag}_grads": means2d.absgrad if absgrad else means2d.grad,
                        f"{tag}_grad2d": state["grad2d"].clone(), f"{tag}_count": state["count"].clone()})
    strat = DefaultStrategy(absgrad=False, refine_scale2d_stop_iter=1000)
    state = strat.initialize_state()
    for frame in range(2):
        nnz = 250
        ids = torch.randperm(N, generator=g)[:nnz]
        radii = torch.randint(1, 60, (nnz, 2), generator=g, dtype=torch.int32)
        means2d = torch.randn(nnz, 2, generator=g)
        means2d.grad = torch.randn(nnz, 2, generator=g) * 1e-3
        info = dict(width=W, height=H, n_cameras=C, radii=radii, gaussian_ids=ids, means2d=means2d)
        strat._update_state({"means": torch.zeros(N, 3)}, state, info, packed=True)
        tag = f"packed_f{frame}"
        out.update({f"{tag}_radii": radii, f"{tag}_grads": means2d.grad, f"{tag}_ids": ids,
                    f"{tag}_grad2d": state["grad2d"].clone(), f"{tag}_count": state["count"].clone(),
                    f"{tag}_state_radii": state["radii"].clone()})
    save("densify_state", C=np.int64(C), N=np.int64(N), width=np.int64(W), height=np.int64(H), **out)


if __name__ == "__main__":
    main()
