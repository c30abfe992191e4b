"""The checks that stand in for a memory checker (SPLATAD_DEBUG=1): list validation before the
compositing kernels follow an index, canary bytes behind every workspace verified after every
library call, a synchronisation and error check after every call. Nothing here makes a kernel
touch memory it does not own: the validation kernel never dereferences through the indices it
checks, and the deliberate overrun lands in the canary bytes of a buffer this test allocated."""

import os
import subprocess
import sys

import pytest
import torch

from gpu_util import DEV

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_validate_lists_reports_bad_indices_without_following_them():
    from splatad_b200 import ops
    flat = torch.tensor([0, 5, 9, 3, 7, 2], dtype=torch.int32, device=DEV)
    offs = torch.tensor([0, 2, 2, 5], dtype=torch.int32, device=DEV)
    assert ops.validate_lists(flat, 10, offs) == (0, 0, 0, 0)
    # the total behind the offsets: entries beyond it are not part of any tile's list
    offs_t = torch.tensor([0, 2, 2, 5, 6], dtype=torch.int32, device=DEV)
    assert ops.validate_lists(flat, 10, offs_t[:4], total_follows=True) == (0, 0, 0, 0)
    bad = flat.clone()
    bad[2] = 10                                        # one past the last row
    n, site, index, limit = ops.validate_lists(bad, 10, offs)
    assert (n, site, index, limit) == (1, 1, 10, 10)
    bad[4] = -3
    assert ops.validate_lists(bad, 10, offs)[0] == 2
    n, site, index, _ = ops.validate_lists(flat, 10, torch.tensor([0, 3, 2, 5], dtype=torch.int32, device=DEV))
    assert n == 1 and site == 2 and index == 1        # tile 1 starts behind the start of tile 2
    n, site, _, _ = ops.validate_lists(flat, 10, torch.tensor([0, 2, 4, 9], dtype=torch.int32, device=DEV))
    assert n == 2 and site in (2, 3)                   # a tile start beyond the list (and behind its end)
    gids = torch.tensor([0, 4, 99], device=DEV)
    cids = torch.tensor([0, 1, 2], device=DEV)
    n, site, index, limit = ops.validate_lists(flat, 10, offs, camera_ids=cids, gaussian_ids=gids, n_cameras=3,
                                               n_gaussians=50)
    assert (n, site, index, limit) == (1, 4, 99, 50)


_RENDERS = r"""
import sys, torch
sys.path.insert(0, %r)
import splatad_b200
from splatad_b200 import _lib, scenes, sharding
assert _lib.DEBUG
dev = "cuda:0"
to = lambda cfg: {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in cfg.items()}
for _ in range(2):            # the second frame of a shape takes the enqueue-ahead paths
    cfg = to(scenes.config2(N=20000))
    leaves = {k: cfg[k].clone().requires_grad_(True) for k in ("means", "quats", "scales", "opacities", "lidar_features")}
    out = splatad_b200.lidar_rasterization(**dict(cfg, **leaves))
    (out[0].square().mean() + out[1].mean()).backward()
    splatad_b200.lidar_rasterization(**cfg)            # the single-call frame
    cam = to(scenes.config1(N=20000))
    cam.update(width=640, height=360)
    leaves = {k: cam[k].clone().requires_grad_(True) for k in ("means", "quats", "scales", "opacities", "colors")}
    out = splatad_b200.rasterization(**dict(cam, **leaves))
    (out[0].square().mean() + out[1].mean()).backward()
    shard = scenes.config4_shard(0, 1, n_local=20000)
    sharding.rasterization_gaussian_sharded(**to(shard["camera"]))
    sharding.lidar_rasterization_gaussian_sharded(**to(shard["lidar"]))
torch.cuda.synchronize()
_lib.check_canaries("the end of the run")
print("debug renders ok", len(_lib._canaries), "workspaces watched")
"""

_OVERRUN = r"""
import sys, torch
sys.path.insert(0, %r)
from splatad_b200 import _lib
assert _lib.DEBUG
dev = torch.device("cuda:0")
lib = _lib.load()
C, N = 1, 400
radii = torch.ones(C, N, 2, device=dev)                               # every pair is visible
scratch = _lib.workspace("visible_rows", lib.splatad_visible_rows_workspace_bytes(C, N), dev)
indptr = torch.zeros(C + 1, dtype=torch.int32, device=dev)
stream = _lib.stream_ptr(dev)
_lib.call("splatad_visible_rows_count", C, N, _lib.ptr(radii), _lib.ptr(scratch), scratch.numel(), _lib.ptr(indptr),
          None, stream)
# the output of the fill is a watched buffer of 256 entries; the call claims it holds 300
rows = _lib.workspace("row_index_probe", 256 * 4, dev)
try:
    _lib.call("splatad_visible_rows_fill", C, N, _lib.ptr(radii), _lib.ptr(scratch), 300, _lib.ptr(rows), stream)
except RuntimeError as e:
    print("caught:", e)
else:
    print("not caught")
"""


def _run(script):
    env = dict(os.environ, SPLATAD_DEBUG="1")
    return subprocess.run([sys.executable, "-c", script % ROOT], env=env, capture_output=True, text=True, timeout=600)


def test_renders_pass_under_debug_mode():
    """Forward + backward lidar and camera frames, the single-call lidar frame and the sharded
    functions with every check on: no inconsistent list, no workspace overrun, no kernel error."""
    proc = _run(_RENDERS)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert "debug renders ok" in proc.stdout, proc.stdout[-2000:]


def test_a_write_past_a_workspace_is_caught_by_its_canary():
    proc = _run(_OVERRUN)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert "caught:" in proc.stdout and "row_index_probe" in proc.stdout and "past its end" in proc.stdout, proc.stdout
