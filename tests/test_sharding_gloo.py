"""Host-side logic of the two multi-GPU shardings, run as two gloo ranks on the CPU: sensor
assignment, Gaussian slices, and the record all-to-all (rows arrive in the single-GPU packed
order; gradients travel back through the mirrored all-to-all)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from splatad_b200 import sharding


def test_sensor_owners_and_slices():
    assert sharding.sensor_owners(7, 4) == [0, 1, 2, 3, 0, 1, 2]
    # six 2-Mpixel cameras and one 0.23-Mpoint lidar on four ranks: no rank gets two cameras and the lidar
    costs = [2.07] * 6 + [0.23]
    owners = sharding.sensor_owners(7, 4, costs)
    load = [sum(costs[c] for c in sharding.local_sensors(owners, r)) for r in range(4)]
    assert max(load) <= 2 * 2.07 + 1e-9 and sorted(sum(o == r for o in owners) for r in range(4)) == [1, 2, 2, 2]
    spans = [sharding.gaussian_slice(10, 4, r) for r in range(4)]
    assert spans == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert sharding.gaussian_slice(8_000_000, 8, 3) == (3_000_000, 4_000_000)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _fields(N, C, seed):
    g = torch.Generator().manual_seed(seed)
    f = dict(means2d=torch.randn(C, N, 2, generator=g, dtype=torch.float64).float(),
             conics=torch.randn(C, N, 3, generator=g), depths=torch.rand(C, N, generator=g),
             colors=torch.randn(C, N, 4, generator=g))
    vis = torch.rand(C, N, generator=g) > 0.4
    return f, vis


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        N, C = 101, 3
        full, vis = _fields(N, C, 0)
        owners = sharding.sensor_owners(C, world)
        lo, hi = sharding.gaussian_slice(N, world, rank)
        local = {k: v[:, lo:hi].clone().requires_grad_(True) for k, v in full.items()}
        recv, sens, gids = sharding.exchange_projected(local, vis[:, lo:hi], lo, N, owners)
        # expected: packed rows (sensor-major, Gaussian-minor) of the sensors this rank owns
        mine = sharding.local_sensors(owners, rank)
        exp_s, exp_g = [], []
        for c in mine:
            g = torch.nonzero(vis[c]).squeeze(-1)
            exp_s.append(torch.full_like(g, c))
            exp_g.append(g)
        exp_s, exp_g = torch.cat(exp_s), torch.cat(exp_g)
        assert torch.equal(sens, exp_s) and torch.equal(gids, exp_g)
        for k in full:
            assert torch.equal(recv[k], full[k][exp_s, exp_g]), k
        # backward: d(sum of received colours * w)/d(local colours) = w at the visible entries whatever the owner
        w = 1.0 + sens.float() + 0.01 * gids.float()
        loss = (recv["colors"] * w[:, None]).sum() + (recv["depths"] * 2.0).sum()
        loss.backward()
        want = torch.zeros(C, hi - lo, 4)
        for c in range(C):
            g = torch.arange(lo, hi)
            want[c] = (vis[c, lo:hi].float() * (1.0 + c + 0.01 * g.float()))[:, None]
        assert torch.allclose(local["colors"].grad, want, atol=1e-6)
        assert torch.allclose(local["depths"].grad, vis[:, lo:hi].float() * 2.0)
        assert local["conics"].grad is None or float(local["conics"].grad.abs().sum()) == 0.0
        # sensor-sharded training: gradient all-reduce of replicated parameters
        p = torch.ones(4, requires_grad=True)
        (p * (rank + 1)).sum().backward()
        sharding.all_reduce_gradients([p])
        assert torch.equal(p.grad, torch.full((4,), float(sum(range(1, world + 1)))))
        open(os.path.join(tmp, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_exchange_projected_two_ranks(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"ok{r}") for r in range(world))


def test_exchange_projected_single_process():
    f, vis = _fields(50, 2, 1)
    recv, sens, gids = sharding.exchange_projected(f, vis, 0, 50, [0, 0])
    cam, gau = torch.nonzero(vis, as_tuple=True)
    assert torch.equal(sens, cam) and torch.equal(gids, gau)
    assert torch.equal(recv["means2d"], f["means2d"][cam, gau])
