"""Gaussian-sharded rendering (the large-scene training configuration's path): each rank projects
its slice of the Gaussians for all sensors, the visible 2-D records travel to the rank owning each
sensor in one all-to-all of fixed-width rows, and that rank's tile lists, images and - through the
mirrored all-to-all - parameter gradients must be those of a single-GPU render.

Three layers: the device kernels of the exchange with two ranks emulated on one GPU (the
all-to-all replaced by slicing), the sharded render functions in a world of one, and the real
thing on two GPUs over NCCL (skipped on a box with one GPU)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from gpu_util import DEV, n, rel_l2

pytestmark = pytest.mark.gpu

LEAVES = ("means", "quats", "scales", "opacities")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _camera_scene(N=20_000):
    """Config 1's Gaussians in front of three 640 x 360 rolling-shutter cameras half a metre apart."""
    from splatad_b200 import scenes
    cfg = scenes.config1(N=N, packed=True)
    C = 3
    viewmats = torch.eye(4).repeat(C, 1, 1)
    viewmats[:, 0, 3] = torch.tensor([-0.5, 0.0, 0.5])
    Ks = torch.tensor([[400.0, 0.0, 320.0], [0.0, 400.0, 180.0], [0.0, 0.0, 1.0]]).repeat(C, 1, 1)
    cfg.update(viewmats=viewmats, Ks=Ks, width=640, height=360,
               linear_velocity=cfg["linear_velocity"][:1].repeat(C, 1),
               angular_velocity=cfg["angular_velocity"][:1].repeat(C, 1),
               rolling_shutter_time=cfg["rolling_shutter_time"][:1].repeat(C))
    return cfg


def _lidar_scene(N=20_000):
    """Two 128 x 1800 rolling-shutter lidars a metre apart over config 4's kind of scene."""
    from splatad_b200 import scenes
    return scenes.config4(N=N, n_cameras=1, n_lidars=2)["lidar"]


def _to(cfg, dev):
    return {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in cfg.items()}


def test_exchange_kernels_with_two_emulated_ranks():
    """visible_rows / pack / segment map / unpack on one GPU, the all-to-all replaced by slicing the
    send buffers: every emulated rank ends up with exactly the packed projection rows of the
    cameras it owns (ids, order, values bit for bit), and gradients sent back through the row
    buffers equal those of the single-GPU packed projection."""
    from splatad_b200 import ops, sharding
    with ops.velocity_grads(True):      # the projection decides in its forward pass whether to return them
        _emulated_ranks(ops, sharding)


def _emulated_ranks(ops, sharding):
    cfg = _to(_camera_scene(), DEV)
    N, C, world = cfg["means"].shape[0], 3, 2
    owners = [0, 1, 0]
    order = sharding.sensor_send_order(owners)
    sel = torch.tensor(order, device=DEV)
    geom = (cfg["width"], cfg["height"])
    motion = lambda s: (cfg["linear_velocity"][s], cfg["angular_velocity"][s], cfg["rolling_shutter_time"][s])  # noqa: E731

    leaves, sends, counts = [], [], []
    for r in range(world):
        lo, hi = sharding.gaussian_slice(N, world, r)
        L = {k: cfg[k][lo:hi].clone().requires_grad_(True) for k in LEAVES + ("velocities",)}
        radii, means2d, depths, conics, _, pix_vels = ops.fully_fused_projection(
            L["means"], None, L["quats"], L["scales"], L["velocities"], cfg["viewmats"][sel], cfg["Ks"][sel], *geom,
            *motion(sel))
        row_index, indptr = sharding.visible_rows(radii)
        cnt = (indptr[1:] - indptr[:-1]).tolist()
        fields = [radii, means2d, depths[..., None], conics, pix_vels]
        flat = [f.reshape(C * (hi - lo), -1) for f in fields]
        rows = sharding._PackRows.apply(row_index, sum(cnt), sel.int(), hi - lo, lo, *flat)
        assert rows.shape == (sum(cnt), 2 + 2 + 2 + 1 + 3 + 2)
        leaves.append(L), sends.append(rows), counts.append(cnt)

    # single-GPU packed projection of everything
    F = {k: cfg[k].clone().requires_grad_(True) for k in LEAVES + ("velocities",)}
    cam, gau, p_radii, p_means2d, p_depths, p_conics, _, p_vels = ops.fully_fused_projection(
        F["means"], None, F["quats"], F["scales"], F["velocities"], cfg["viewmats"], cfg["Ks"], *geom,
        cfg["linear_velocity"], cfg["angular_velocity"], cfg["rolling_shutter_time"], packed=True)
    listed = p_radii[:, 0] > 0
    gen = torch.Generator().manual_seed(2)
    loss_sharded, loss_single = 0.0, 0.0
    for d in range(world):
        plan = sharding.plan_exchange(counts, order, owners, d)
        starts = [[sum(sharding.plan_exchange(counts, order, owners, s).send_splits[:k]) for k in range(world)]
                  for s in range(world)]
        received = torch.cat([sends[s][starts[s][d]: starts[s][d] + plan.recv_splits[s]] for s in range(world)])
        row_map, local_ids = sharding.segment_row_map(plan, DEV)
        assert torch.equal(torch.sort(row_map).values, torch.arange(received.shape[0], device=DEV, dtype=torch.int32))
        sid, gid, radii, means2d, depths, conics, pix_vels = sharding._UnpackRows.apply(
            received, row_map, (2, 2, 1, 3, 2), (True, False, False, False, False))
        keep = listed & torch.isin(cam, torch.tensor(plan.mine, device=DEV))
        assert torch.equal(sid, cam[keep]) and torch.equal(gid, gau[keep])
        assert torch.equal(torch.tensor(plan.mine, device=DEV)[local_ids], sid)
        assert torch.equal(radii, p_radii[keep]) and torch.equal(means2d, p_means2d[keep])
        assert torch.equal(depths[:, 0], p_depths[keep]) and torch.equal(conics, p_conics[keep])
        assert torch.equal(pix_vels, p_vels[keep])
        assert plan.sensor_start[-1] == int(keep.sum())
        for a, b in ((means2d, p_means2d[keep]), (depths[:, 0], p_depths[keep]), (conics, p_conics[keep]),
                     (pix_vels, p_vels[keep])):
            w = torch.randn(a.shape, generator=gen).to(DEV)
            loss_sharded = loss_sharded + (a * w).sum()
            loss_single = loss_single + (b * w).sum()
    loss_sharded.backward()
    loss_single.backward()
    for k in LEAVES[:3] + ("velocities",):
        got = torch.cat([L[k].grad for L in leaves])
        assert rel_l2(n(got), n(F[k].grad)) < 1e-5, k


def _grads(loss, leaves):
    loss.backward()
    return {k: v.grad.clone() for k, v in leaves.items()}


def test_sharded_functions_in_a_world_of_one_equal_the_single_gpu_render():
    import splatad_b200
    from splatad_b200 import sharding
    gen = torch.Generator().manual_seed(4)
    # cameras: SH colours, RGB + depth
    cfg = _to(_camera_scene(), DEV)
    N = cfg["means"].shape[0]
    names = LEAVES + ("colors",)
    A = {k: cfg[k].clone().requires_grad_(True) for k in names}
    B = {k: cfg[k].clone().requires_grad_(True) for k in names}
    kw = {k: v for k, v in cfg.items() if k not in names + ("packed",)}
    ref_c, ref_a, ref_m = splatad_b200.rasterization(**dict(kw, **A), packed=True)
    out_c, out_a, m = sharding.rasterization_gaussian_sharded(**dict(kw, **B), n_gaussians_total=N, gaussian_start=0)
    assert torch.equal(out_c, ref_c) and torch.equal(out_a, ref_a)
    assert torch.equal(m["gaussian_ids"][m["flatten_ids"].long()], ref_m["gaussian_ids"][ref_m["flatten_ids"].long()])
    w = torch.randn(ref_c.shape, generator=gen).to(DEV)
    ga, gb = _grads((ref_c * w).sum() + ref_a.sum(), A), _grads((out_c * w).sum() + out_a.sum(), B)
    for k in names:
        assert rel_l2(n(gb[k]), n(ga[k])) < 1e-4, f"camera d/d{k}: {rel_l2(n(gb[k]), n(ga[k])):.2e}"
    # lidars
    cfg = _to(_lidar_scene(), DEV)
    N = cfg["means"].shape[0]
    names = LEAVES + ("lidar_features",)
    A = {k: cfg[k].clone().requires_grad_(True) for k in names}
    B = {k: cfg[k].clone().requires_grad_(True) for k in names}
    kw = {k: v for k, v in cfg.items() if k not in names}
    ref = splatad_b200.lidar_rasterization(**dict(kw, **A))
    out = sharding.lidar_rasterization_gaussian_sharded(**dict(kw, **B), n_gaussians_total=N, gaussian_start=0)
    for a, b in zip(out[:3], ref[:3]):
        assert torch.equal(a, b)
    assert torch.equal(out[3]["median_depths"], ref[3]["median_depths"])
    w = torch.randn(ref[0].shape, generator=gen).to(DEV)
    ga = _grads((ref[0] * w).sum() + ref[1].sum() + ref[2].sum(), A)
    gb = _grads((out[0] * w).sum() + out[1].sum() + out[2].sum(), B)
    for k in names:
        assert rel_l2(n(gb[k]), n(ga[k])) < 1e-4, f"lidar d/d{k}: {rel_l2(n(gb[k]), n(ga[k])):.2e}"


def _worker(rank, world, port, out_path):
    import torch.distributed as dist

    import splatad_b200
    from splatad_b200 import sharding
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device(f"cuda:{rank}")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    res = {}
    try:
        gen = torch.Generator().manual_seed(9)
        for kind, scene in (("camera", _camera_scene()), ("lidar", _lidar_scene())):
            g = _to(scene, dev)
            N = g["means"].shape[0]
            lo, hi = sharding.gaussian_slice(N, world, rank)
            feat = "colors" if kind == "camera" else "lidar_features"
            names = LEAVES + (feat,)
            cut = lambda k: g[k][:, lo:hi] if k == "lidar_features" else g[k][lo:hi]  # noqa: E731
            L = {k: cut(k).clone().requires_grad_(True) for k in names}
            F = {k: g[k].clone().requires_grad_(True) for k in names}
            kw = {k: v for k, v in g.items() if k not in names + ("packed",)}
            if kind == "camera":
                vel = kw.pop("velocities")
                stats = {}
                out = sharding.rasterization_gaussian_sharded(
                    **dict(kw, **L), velocities=vel[lo:hi], n_gaussians_total=N, gaussian_start=lo, stats=stats)
                ref = splatad_b200.rasterization(**dict(kw, **F), velocities=vel, packed=True)
                outs, refs, m, ref_m = out[:2], ref[:2], out[2], ref[2]
            else:
                stats = {}
                out = sharding.lidar_rasterization_gaussian_sharded(
                    **dict(kw, **L), n_gaussians_total=N, gaussian_start=lo, stats=stats)
                ref = splatad_b200.lidar_rasterization(**dict(kw, **F))
                outs, refs, m, ref_m = out[:3], ref[:3], out[3], ref[3]
            mine = m["sensor_ids"]
            res[kind + "_images"] = all(torch.equal(a, b[mine]) for a, b in zip(outs, refs))
            res[kind + "_isects"] = int(m["flatten_ids"].numel())
            res[kind + "_wire_bytes"] = int(stats["bytes_sent_off_rank"])
            # lists: the Gaussians of this rank's sensors' tiles in single-GPU order
            if kind == "camera":
                cam_of = ref_m["camera_ids"][ref_m["flatten_ids"].long()]
                keep = torch.isin(cam_of, torch.tensor(mine, device=dev))
                want = ref_m["gaussian_ids"][ref_m["flatten_ids"].long()][keep]
            else:
                flat = ref_m["flatten_ids"].long()
                keep = torch.isin(flat // N, torch.tensor(mine, device=dev))
                want = (flat % N)[keep]
            res[kind + "_lists"] = bool(torch.equal(m["gaussian_ids"][m["flatten_ids"].long()], want))
            # backward: every rank's loss covers its own sensors; the single-GPU loss covers all
            cots = [torch.randn(b.shape, generator=gen).to(dev) for b in refs]
            loss = sum((a * c[mine]).sum() for a, c in zip(outs, cots))
            loss.backward()                                   # mirrored all-to-all inside
            sum((b * c).sum() for b, c in zip(refs, cots)).backward()
            errs = {}
            for k in names:
                want_g = F[k].grad[:, lo:hi] if k == "lidar_features" else F[k].grad[lo:hi]
                errs[k] = rel_l2(n(L[k].grad), n(want_g))
            res[kind + "_grad_err"] = errs
        torch.save(res, f"{out_path}.{rank}")
    finally:
        dist.destroy_process_group()


def test_gaussian_sharded_render_two_gpus(tmp_path):
    """Two NCCL ranks (NVLS off), cameras and lidars: images and lists equal the single-GPU ones bit
    for bit on the owning rank; the gradients that come back through the mirrored all-to-all equal the
    single-GPU gradients of the rank's slice to 1e-4 relative L2."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = _free_port()
    out = str(tmp_path / "res")
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(f"{out}.{r}")
        print(f"rank {r}: {res}")
        for kind in ("camera", "lidar"):
            assert res[kind + "_isects"] > 10_000, res
            assert res[kind + "_wire_bytes"] > 0, res
            assert res[kind + "_lists"], f"rank {r}: {kind} tile lists differ from the single-GPU render"
            assert res[kind + "_images"], f"rank {r}: {kind} images differ from the single-GPU render"
            for k, e in res[kind + "_grad_err"].items():
                assert e < 1e-4, f"rank {r}: {kind} d/d{k} relative L2 {e:.2e}"
