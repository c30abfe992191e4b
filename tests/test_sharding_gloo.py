"""Host-side logic of the two multi-GPU shardings, run as gloo ranks on the CPU: sensor assignment,
Gaussian slices, the exchange plan (split sizes and segment table from the count matrix), the
differentiable row all-to-all (rows arrive in the single-GPU packed order after the segment map;
gradients travel back through the mirrored all-to-all), gradient all-reduce, and what the
survivors see when a rank leaves between steps (an error within the process-group timeout, not a
hang). The packing / placing kernels themselves are CUDA and are covered by the GPU tests; here a
few lines of torch stand in for them."""

import datetime
import os
import socket
import time

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
    assert sharding.sensor_send_order([0, 1, 0, 2, 1]) == [0, 2, 1, 4, 3]


def test_plan_exchange_tables():
    owners = [0, 1, 0]
    order = sharding.sensor_send_order(owners)           # [0, 2, 1]
    counts = [[5, 2, 3], [1, 4, 6]]                       # rows per (source rank, sensor in send order)
    p0 = sharding.plan_exchange(counts, order, owners, 0)
    assert p0.send_splits == [7, 3] and p0.recv_splits == [7, 5] and p0.mine == [0, 2]
    assert p0.src_start == [0, 5, 7, 8, 12] and p0.dst_start == [0, 6, 5, 8] and p0.sensor_start == [0, 6, 12]
    p1 = sharding.plan_exchange(counts, order, owners, 1)
    assert p1.send_splits == [5, 6] and p1.recv_splits == [3, 6] and p1.mine == [1]
    assert p1.src_start == [0, 3, 9] and p1.dst_start == [0, 3] and p1.sensor_start == [0, 9]
    # what one rank sends to another is what the other expects from it
    assert p0.send_splits[1] == p1.recv_splits[0] and p1.send_splits[0] == p0.recv_splits[1]
    # a rank that owns nothing receives nothing
    idle = sharding.plan_exchange([[2, 3], [1, 1], [0, 4]], [0, 1], [0, 1], 2)
    assert idle.recv_splits == [0, 0, 0] and idle.mine == [] and idle.src_start == [0] and idle.dst_start == []


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _fields(N, C, seed):
    g = torch.Generator().manual_seed(seed)
    f = dict(means2d=torch.randn(C, N, 2, generator=g), conics=torch.randn(C, N, 3, generator=g),
             depths=torch.rand(C, N, 1, generator=g), colors=torch.randn(C, N, 4, generator=g))
    vis = torch.rand(C, N, generator=g) > 0.4
    return f, vis


def _exchange_on_cpu(local, vis, lo, owners, rank):
    """The exchange with torch stand-ins for the CUDA pack / place kernels. Sensors are taken in send
    order, as the sharded render functions do."""
    order = sharding.sensor_send_order(owners)
    names = sorted(local)
    C, n_local = vis.shape
    sel = torch.tensor(order)
    vis_o = vis[sel]
    pairs = torch.nonzero(vis_o.reshape(-1)).squeeze(-1)                 # c * n_local + n, (sensor, Gaussian) order
    ids = torch.stack([sel[pairs // n_local], pairs % n_local + lo], -1).float()
    rows = torch.cat([ids] + [local[k][sel].reshape(C * n_local, -1)[pairs] for k in names], dim=-1)
    counts_local = vis_o.sum(1)
    gathered = [torch.empty_like(counts_local) for _ in range(dist.get_world_size())]
    dist.all_gather(gathered, counts_local)
    plan = sharding.plan_exchange([g.tolist() for g in gathered], order, owners, rank)
    assert sum(plan.send_splits) == rows.shape[0]
    received = sharding.exchange_rows(rows, plan.send_splits, plan.recv_splits)
    # segment map: received row i of segment s lands at dst_start[s] + (i - src_start[s])
    row_map = torch.empty(received.shape[0], dtype=torch.int64)
    for s, dst in enumerate(plan.dst_start):
        a, b = plan.src_start[s], plan.src_start[s + 1]
        row_map[a:b] = torch.arange(dst, dst + b - a)
    placed = torch.zeros_like(received).index_add(0, row_map, received)
    out, col = {}, 2
    for k in names:
        w = local[k].shape[-1]
        out[k] = placed[:, col:col + w]
        col += w
    return out, placed[:, 0].long(), placed[:, 1].long(), plan


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        N, C = 101, 3
        full, vis = _fields(N, C, 0)
        owners = sharding.sensor_owners(C, world)
        lo, hi = sharding.gaussian_slice(N, world, rank)
        local = {k: v[:, lo:hi].clone().requires_grad_(True) for k, v in full.items()}
        recv, sens, gids, plan = _exchange_on_cpu(local, vis[:, lo:hi], lo, owners, rank)
        # expected: packed rows (sensor-major, Gaussian-minor) of the sensors this rank owns
        mine = sharding.local_sensors(owners, rank)
        assert plan.mine == mine
        exp_s, exp_g = [], []
        for c in mine:
            g = torch.nonzero(vis[c]).squeeze(-1)
            exp_s.append(torch.full_like(g, c))
            exp_g.append(g)
        exp_s, exp_g = torch.cat(exp_s), torch.cat(exp_g)
        assert torch.equal(sens, exp_s) and torch.equal(gids, exp_g)
        assert plan.sensor_start[-1] == exp_s.numel()
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
        assert torch.allclose(local["depths"].grad[..., 0], vis[:, lo:hi].float() * 2.0)
        assert local["conics"].grad is None or float(local["conics"].grad.abs().sum()) == 0.0
        # sensor-sharded training: gradient all-reduce of replicated parameters
        p = torch.ones(4, requires_grad=True)
        (p * (rank + 1)).sum().backward()
        sharding.all_reduce_gradients([p])
        assert torch.equal(p.grad, torch.full((4,), float(sum(range(1, world + 1)))))
        open(os.path.join(tmp, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_row_exchange_ranks(tmp_path, world):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"ok{r}") for r in range(world))


def _leaving_worker(rank, world, port, tmp):
    """Step 0: every rank exchanges. Then the last rank leaves (between steps, nothing of it in
    flight). Step 1: the others' exchange must come back with PeerLostError within the timeout."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    rows = torch.full((world * 2, 3), float(rank))
    splits = [2] * world
    got = sharding.exchange_rows(rows, splits, splits)
    assert torch.equal(got[:, 0], torch.arange(world).repeat_interleave(2).float())
    if rank == world - 1:
        open(os.path.join(tmp, f"left{rank}"), "w").write("left")
        os._exit(0)           # the rank is gone: no destroy, no goodbye
    t0 = time.time()
    try:
        sharding.exchange_rows(rows, splits, splits)
        outcome = "returned"
    except sharding.PeerLostError as e:
        outcome = f"lost after {time.time() - t0:.1f} s: {str(e)[:80]}"
    open(os.path.join(tmp, f"outcome{rank}"), "w").write(outcome)
    os._exit(0)               # the group is broken: do not wait in its destructor


def test_a_rank_leaving_between_steps_is_reported_not_waited_for(tmp_path):
    world = 3
    ctx = mp.spawn(_leaving_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=False)
    deadline = time.time() + 60
    while time.time() < deadline and not all(os.path.exists(tmp_path / f"outcome{r}") for r in range(world - 1)):
        time.sleep(0.2)
    for p in ctx.processes:
        p.join(timeout=5)
        if p.is_alive():
            p.kill()
    assert os.path.exists(tmp_path / f"left{world - 1}")
    for r in range(world - 1):
        path = tmp_path / f"outcome{r}"
        assert os.path.exists(path), f"rank {r} is still blocked in the exchange"
        assert open(path).read().startswith("lost after"), open(path).read()
