"""Seeded synthetic scenes and sensors for the five benchmark configurations.

There is no public dataset behind these numbers: the reference measures on none and ships only
a small test fixture, so every configuration is generated from a ``torch.Generator`` on the CPU
with a fixed seed, drawing tensors in the order listed in each function, and then moved to the
requested device. Shapes, sizes and value distributions:

  config 0  20 000 Gaussians, one 32-beam x 512-column lidar, no rolling shutter
  config 1  500 000 Gaussians, one 1920x1080 rolling-shutter pinhole camera, SH degree 3, RGB+D
  config 2  1 000 000 Gaussians, one 128-beam x 1800-column rolling-shutter lidar, 16 features
  config 3  2 000 000 Gaussians, 6 cameras (config 1, yawed 60 deg apart) + the config 2 lidar
  config 4  8 000 000 Gaussians, 8 cameras (45 deg apart) + 2 lidars, forward + backward

Each ``config*`` function returns keyword arguments for ``rasterization`` /
``lidar_rasterization`` (the camera and lidar parts of configs 3 and 4 come separately).
"""

from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn.functional as F


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def lidar_box_gaussians(N: int, g: torch.Generator, log_scale_mu: float = -1.0, log_scale_sd: float = 0.5):
    """means x,y ~ U(-40,40) m, z ~ U(-2,4) m; scales = exp(N(mu, sd)); unit quaternions from
    N(0,1)^4; opacities = sigmoid(N(0,1)). Draw order: means x, y, z, log-scales, quats, logits."""
    means = torch.empty(N, 3)
    means[:, 0] = torch.rand(N, generator=g) * 80 - 40
    means[:, 1] = torch.rand(N, generator=g) * 80 - 40
    means[:, 2] = torch.rand(N, generator=g) * 6 - 2
    scales = torch.exp(torch.randn(N, 3, generator=g) * log_scale_sd + log_scale_mu)
    quats = F.normalize(torch.randn(N, 4, generator=g), dim=-1)
    opacities = torch.sigmoid(torch.randn(N, generator=g))
    return means, quats, scales, opacities


def camera_box_gaussians(N: int, g: torch.Generator):
    """Camera-frame box: x ~ U(-50,50), y ~ U(-5,5), z ~ U(0.5,100.5) (+z forward);
    scales = exp(N(-1.5, 0.7)). Same draw order as :func:`lidar_box_gaussians`."""
    means = torch.empty(N, 3)
    means[:, 0] = torch.rand(N, generator=g) * 100 - 50
    means[:, 1] = torch.rand(N, generator=g) * 10 - 5
    means[:, 2] = torch.rand(N, generator=g) * 100 + 0.5
    scales = torch.exp(torch.randn(N, 3, generator=g) * 0.7 - 1.5)
    quats = F.normalize(torch.randn(N, 4, generator=g), dim=-1)
    opacities = torch.sigmoid(torch.randn(N, generator=g))
    return means, quats, scales, opacities


def beams_32() -> torch.Tensor:
    return torch.linspace(-25.0, 15.0, 32)


def beams_128() -> torch.Tensor:
    """128 beams in [-25, 15] deg: 0.1 deg spacing within +-5 deg of the horizon, coarser outside."""
    e = torch.cat([torch.linspace(-25, -5, 19)[:-1], torch.linspace(-5, 5, 101), torch.linspace(5, 15, 10)[1:]])
    assert e.numel() == 128
    return e


def elevation_boundaries(elevations: torch.Tensor, tile_height: int) -> torch.Tensor:
    """Tile boundaries in elevation: midpoints between consecutive groups of ``tile_height`` beams,
    extended by one degree at both ends (the recipe of examples/lidar_rendering.ipynb, cell 8)."""
    return torch.cat(
        [
            elevations[0:1] - 1.0,
            (elevations[tile_height::tile_height] + elevations[tile_height - 1 : -1 : tile_height]) / 2,
            elevations[-1:] + 1.0,
        ]
    )


def lidar_sensor(elevations: torch.Tensor, width: int, g: torch.Generator, sweep_time: float = 0.0) -> torch.Tensor:
    """raster_pts [1, H, W, 4] = (azimuth deg at column centres over 360 deg, elevation deg,
    range ~ U(2, 80) m, time offset linear over the sweep)."""
    H = elevations.numel()
    az = -180.0 + (torch.arange(width, dtype=torch.float32) + 0.5) * (360.0 / width)
    pts = torch.empty(1, H, width, 4)
    pts[0, :, :, 0] = az[None, :]
    pts[0, :, :, 1] = elevations[:, None]
    pts[0, :, :, 2] = torch.rand(H, width, generator=g) * 78 + 2
    if sweep_time > 0:
        pts[0, :, :, 3] = torch.linspace(-0.5 * sweep_time, 0.5 * sweep_time, width)[None, :]
    else:
        pts[0, :, :, 3] = 0.0
    return pts


def _to(d: Dict, device) -> Dict:
    return {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


def _lidar_kwargs(elevations, width, azimuth_resolution, raster_pts, rolling: bool, C: int = 1):
    tile_width, tile_height = 32, 8
    kw = dict(
        viewmats=torch.eye(4)[None].repeat(C, 1, 1),
        raster_pts=raster_pts,
        tile_elevation_boundaries=elevation_boundaries(elevations, tile_height),
        min_azimuth=-180.0,
        max_azimuth=180.0,
        min_elevation=float(elevations[0]) - 1.0,
        max_elevation=float(elevations[-1]) + 1.0,
        n_elevation_channels=int(elevations.numel()),
        azimuth_resolution=azimuth_resolution,
        tile_width=tile_width,
        tile_height=tile_height,
        eps2d=0.017,
    )
    if rolling:
        kw.update(
            linear_velocity=torch.tensor([[15.0, 0.0, 0.0]]).repeat(C, 1),
            angular_velocity=torch.tensor([[0.0, 0.0, 0.1]]).repeat(C, 1),
            rolling_shutter_time=torch.full((C,), 0.1),
        )
    return kw


def config0(device="cpu", N: int = 20_000, seed: int = 0) -> Dict:
    """20k Gaussians, 32 x 512 lidar at the origin, no rolling shutter, 4 features."""
    g = _gen(seed)
    means, quats, scales, opacities = lidar_box_gaussians(N, g)
    features = torch.randn(1, N, 4, generator=g)
    elev = beams_32()
    pts = lidar_sensor(elev, 512, g)
    kw = dict(means=means, quats=quats, scales=scales, opacities=opacities, lidar_features=features,
              velocities=None)
    kw.update(_lidar_kwargs(elev, 512, 360.0 / 512, pts, rolling=False))
    return _to(kw, device)


def config2(device="cpu", N: int = 1_000_000, seed: int = 2, width: int = 1800) -> Dict:
    """1M Gaussians, 128 x 1800 rolling-shutter lidar (100 ms sweep, 15 m/s ego speed, 0.1 rad/s
    yaw rate), 16 features."""
    g = _gen(seed)
    means, quats, scales, opacities = lidar_box_gaussians(N, g)
    features = torch.randn(1, N, 16, generator=g)
    elev = beams_128()
    pts = lidar_sensor(elev, width, g, sweep_time=0.1)
    kw = dict(means=means, quats=quats, scales=scales, opacities=opacities, lidar_features=features,
              velocities=None)
    kw.update(_lidar_kwargs(elev, width, 360.0 / width, pts, rolling=True))
    return _to(kw, device)


def camera_intrinsics(C: int = 1) -> torch.Tensor:
    K = torch.tensor([[1200.0, 0.0, 960.0], [0.0, 1200.0, 540.0], [0.0, 0.0, 1.0]])
    return K[None].repeat(C, 1, 1)


def yawed_camera_viewmats(yaws_deg) -> torch.Tensor:
    """World (x forward, y left, z up) -> camera (x right, y down, z forward) for cameras at the
    origin looking along the horizontal direction at each yaw."""
    mats = []
    for yaw in yaws_deg:
        c, s = math.cos(math.radians(yaw)), math.sin(math.radians(yaw))
        R = torch.tensor([[s, -c, 0.0], [0.0, 0.0, -1.0], [c, s, 0.0]])
        M = torch.eye(4)
        M[:3, :3] = R
        mats.append(M)
    return torch.stack(mats)


def _camera_kwargs(C: int, viewmats: torch.Tensor) -> Dict:
    return dict(
        viewmats=viewmats,
        Ks=camera_intrinsics(C),
        width=1920,
        height=1080,
        linear_velocity=torch.tensor([[10.0, 0.0, 0.0]]).repeat(C, 1),
        angular_velocity=torch.zeros(C, 3),
        rolling_shutter_time=torch.full((C,), 0.03),
        tile_size=16,
        sh_degree=3,
        render_mode="RGB+D",
    )


def config1(device="cpu", N: int = 500_000, seed: int = 1, packed: bool = True) -> Dict:
    """500k Gaussians in front of one 1920x1080 rolling-shutter camera (30 ms readout, 10 m/s ego
    speed along +x), SH degree 3 (K = 16), 10 % of the Gaussians moving with N(0, 2) m/s."""
    g = _gen(seed)
    means, quats, scales, opacities = camera_box_gaussians(N, g)
    sh = torch.randn(N, 16, 3, generator=g) * 0.3
    vel = torch.randn(N, 3, generator=g) * 2.0
    moving = torch.rand(N, generator=g) < 0.1
    vel = vel * moving[:, None]
    kw = dict(means=means, quats=quats, scales=scales, opacities=opacities, colors=sh, velocities=vel,
              packed=packed)
    kw.update(_camera_kwargs(1, torch.eye(4)[None]))
    return _to(kw, device)


def config3(device="cpu", N: int = 2_000_000, seed: int = 3) -> Dict:
    """2M Gaussians (lidar box) with SH degree 3 and 16 lidar features; 6 cameras yawed 60 deg
    apart plus the config 2 lidar. Returns {"camera": kwargs, "lidar": kwargs}; the Gaussian
    tensors are shared between the two."""
    g = _gen(seed)
    means, quats, scales, opacities = lidar_box_gaussians(N, g)
    sh = torch.randn(N, 16, 3, generator=g) * 0.3
    features = torch.randn(1, N, 16, generator=g)
    elev = beams_128()
    pts = lidar_sensor(elev, 1800, g, sweep_time=0.1)
    base = _to(dict(means=means, quats=quats, scales=scales, opacities=opacities), device)
    cam = dict(base, colors=sh.to(device), velocities=None, packed=True)
    cam.update(_to(_camera_kwargs(6, yawed_camera_viewmats([0, 60, 120, 180, 240, 300])), device))
    lid = dict(base, lidar_features=features.to(device), velocities=None)
    lid.update(_to(_lidar_kwargs(elev, 1800, 0.2, pts, rolling=True), device))
    return {"camera": cam, "lidar": lid}


def config4(device="cpu", N: int = 8_000_000, seed: int = 4, n_cameras: int = 8, n_lidars: int = 2) -> Dict:
    """8M Gaussians (lidar box), 8 cameras yawed 45 deg apart and 2 lidars (the second one offset
    by 1 m along x). Returns {"camera": kwargs, "lidar": kwargs} for all sensors; callers shard."""
    g = _gen(seed)
    means, quats, scales, opacities = lidar_box_gaussians(N, g)
    sh = torch.randn(N, 16, 3, generator=g) * 0.3
    features = torch.randn(1, N, 16, generator=g)
    elev = beams_128()
    pts = torch.cat([lidar_sensor(elev, 1800, g, sweep_time=0.1) for _ in range(n_lidars)], dim=0)
    base = _to(dict(means=means, quats=quats, scales=scales, opacities=opacities), device)
    cam = dict(base, colors=sh.to(device), velocities=None, packed=True)
    yaws = [i * 360.0 / n_cameras for i in range(n_cameras)]
    cam.update(_to(_camera_kwargs(n_cameras, yawed_camera_viewmats(yaws)), device))
    lid = dict(base, lidar_features=features.expand(n_lidars, -1, -1).contiguous().to(device), velocities=None)
    lk = _lidar_kwargs(elev, 1800, 0.2, pts, rolling=True, C=n_lidars)
    for i in range(n_lidars):
        lk["viewmats"][i, 0, 3] = -float(i)  # sensor i sits at x = i metres: world->sensor shifts by -i
    lid.update(_to(lk, device))
    return {"camera": cam, "lidar": lid}


def config4_shard(rank: int, world: int, n_local: int = 1_000_000, seed: int = 4) -> Dict:
    """Rank ``rank``'s part of the Gaussian-sharded training configuration at ``world`` ranks:
    ``n_local`` Gaussians of its own (lidar box, SH degree 3, 16 lidar features; seeded by
    ``seed`` and the rank, so the scene of ``world * n_local`` Gaussians never has to exist on one
    host), and ALL sensors - ``world`` cameras yawed 360 / world degrees apart and min(2, world)
    lidars a metre apart - which every rank generates alike. Returns {"camera": kwargs, "lidar":
    kwargs, "n_total", "start"} for the two ``*_gaussian_sharded`` render functions."""
    g = _gen(seed * 1000 + rank)
    means, quats, scales, opacities = lidar_box_gaussians(n_local, g)
    sh = torch.randn(n_local, 16, 3, generator=g) * 0.3
    features = torch.randn(n_local, 16, generator=g)
    gs = _gen(seed)                                   # sensors: the same on every rank
    n_lidars = min(2, world)
    elev = beams_128()
    pts = torch.cat([lidar_sensor(elev, 1800, gs, sweep_time=0.1) for _ in range(n_lidars)], dim=0)
    base = dict(means=means, quats=quats, scales=scales, opacities=opacities, velocities=None,
                n_gaussians_total=world * n_local, gaussian_start=rank * n_local)
    cam = dict(base, colors=sh)
    cam.update(_camera_kwargs(world, yawed_camera_viewmats([i * 360.0 / world for i in range(world)])))
    lid = dict(base, lidar_features=features)
    lk = _lidar_kwargs(elev, 1800, 0.2, pts, rolling=True, C=n_lidars)
    for i in range(n_lidars):
        lk["viewmats"][i, 0, 3] = -float(i)
    lid.update(lk)
    return {"camera": cam, "lidar": lid, "n_total": world * n_local, "start": rank * n_local}
