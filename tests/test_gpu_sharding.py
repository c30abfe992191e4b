"""Gaussian-sharded camera render on two GPUs (NCCL) against the single-GPU render: each rank
projects its half of the Gaussians for all cameras, the visible 2-D records travel to the rank
owning each camera in one all-to-all, and that rank's tile lists and images must equal the
single-GPU ones exactly. Skipped on a box with one GPU."""

import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _scene():
    """Config 1's Gaussians in front of three 640 x 360 cameras half a metre apart."""
    from splatad_b200 import scenes
    cfg = scenes.config1(N=20_000, packed=True)
    C = 3
    viewmats = torch.eye(4).repeat(C, 1, 1)
    viewmats[:, 0, 3] = torch.tensor([-0.5, 0.0, 0.5])
    Ks = torch.tensor([[400.0, 0.0, 320.0], [0.0, 400.0, 180.0], [0.0, 0.0, 1.0]]).repeat(C, 1, 1)
    cfg.update(viewmats=viewmats, Ks=Ks, width=640, height=360,
               linear_velocity=cfg["linear_velocity"][:1].repeat(C, 1),
               angular_velocity=cfg["angular_velocity"][:1].repeat(C, 1),
               rolling_shutter_time=cfg["rolling_shutter_time"][:1].repeat(C))
    return cfg


def _worker(rank, world, port, out_path):
    import torch.distributed as dist

    import splatad_b200
    from splatad_b200 import sharding
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device(f"cuda:{rank}")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        cfg = _scene()
        N = cfg["means"].shape[0]
        lo, hi = sharding.gaussian_slice(N, world, rank)
        g = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in cfg.items()}
        colors, alphas, meta = sharding.rasterization_gaussian_sharded(
            g["means"][lo:hi], g["quats"][lo:hi], g["scales"][lo:hi], g["opacities"][lo:hi], g["colors"][lo:hi],
            g["velocities"][lo:hi], g["viewmats"], g["Ks"], g["width"], g["height"], N, lo,
            linear_velocity=g["linear_velocity"], angular_velocity=g["angular_velocity"],
            rolling_shutter_time=g["rolling_shutter_time"], sh_degree=3, render_mode="RGB+D")
        # single-GPU render of everything on this rank's GPU
        full = dict(g, sh_degree=3, render_mode="RGB+D")
        ref_c, ref_a, ref_m = splatad_b200.rasterization(**full)
        mine = meta["sensor_ids"]
        ok = torch.equal(colors, ref_c[mine]) and torch.equal(alphas, ref_a[mine])
        # the lists of this rank's cameras are the single-GPU lists of those cameras
        cam_of = ref_m["camera_ids"][ref_m["flatten_ids"].long()]
        keep = torch.isin(cam_of, torch.tensor(mine, device=dev))
        same_lists = torch.equal(meta["gaussian_ids"][meta["flatten_ids"].long()],
                                 ref_m["gaussian_ids"][ref_m["flatten_ids"].long()][keep])
        torch.save(dict(ok=bool(ok), lists=bool(same_lists), n=int(meta["flatten_ids"].numel()), mine=mine),
                   f"{out_path}.{rank}")
    finally:
        dist.destroy_process_group()


def test_gaussian_sharded_render_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = _free_port()
    out = str(tmp_path / "res")
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(f"{out}.{r}")
        assert res["n"] > 10_000, res
        assert res["lists"], f"rank {r}: tile lists differ from the single-GPU render"
        assert res["ok"], f"rank {r}: images differ from the single-GPU render"
