"""Parity of the densification hooks (through the C ABI) against the oracle: the fused statistics
update on the reference strategy's own outputs (fixture) and on a rendered frame, and
compute_relocation against the float64 oracle (new opacities 1e-4 relative; new scales 1e-4 on 99 %
of the entries and 5e-4 on all: the kernel sums an alternating series in float32 in the reference's
order)."""

import math

import numpy as np
import pytest
import torch

from gpu_util import DEV, n, t

pytestmark = pytest.mark.gpu


def test_update_state_on_the_reference_fixture(golden):
    from splatad_b200 import densify
    g = golden("densify_state")
    C, N, W, H = (int(g[k]) for k in ("C", "N", "width", "height"))
    for tag, absgrad in (("grad", False), ("abs", True)):
        state = dict(grad2d=None, count=None)
        for frame in range(2):
            k = f"{tag}_f{frame}"
            means2d = torch.zeros(C, N, 2, device=DEV)
            means2d.grad = t(g[k + "_grads"]) if not absgrad else torch.full((C, N, 2), 7.0, device=DEV)
            means2d.absgrad = t(g[k + "_grads"]) if absgrad else None
            info = dict(width=W, height=H, n_cameras=C, radii=t(g[k + "_radii"], torch.int32), gaussian_ids=None,
                        means2d=means2d)
            densify.update_state(state, info, N, packed=False, absgrad=absgrad)
            np.testing.assert_allclose(n(state["grad2d"]), g[k + "_grad2d"], rtol=2e-6, atol=1e-9)
            assert np.array_equal(n(state["count"]), g[k + "_count"])
            assert "radii" not in state
    state = dict(grad2d=None, count=None, radii=None)
    for frame in range(2):
        k = f"packed_f{frame}"
        means2d = torch.zeros(g[k + "_grads"].shape, device=DEV)
        means2d.grad = t(g[k + "_grads"])
        info = dict(width=W, height=H, n_cameras=C, radii=t(g[k + "_radii"], torch.int32),
                    gaussian_ids=t(g[k + "_ids"], torch.int64), means2d=means2d)
        densify.update_state(state, info, N, packed=True, refine_scale2d=True)
        np.testing.assert_allclose(n(state["grad2d"]), g[k + "_grad2d"], rtol=2e-6, atol=1e-9)
        assert np.array_equal(n(state["count"]), g[k + "_count"])
        np.testing.assert_allclose(n(state["radii"]), g[k + "_state_radii"], rtol=1e-6)


@pytest.mark.parametrize("packed", [False, True])
def test_update_state_after_a_rendered_frame(packed):
    """The hook on the real ``meta`` of rasterization() after backward(), absgrad included."""
    import splatad_b200 as sp
    from oracle import densify as oracle
    from splatad_b200 import densify, scenes
    cfg = scenes.config3(device=DEV, N=20_000, seed=31)["camera"]
    cfg.update(width=480, height=270, packed=packed, absgrad=True)
    cfg["Ks"] = cfg["Ks"].clone()
    cfg["Ks"][:, :2] *= 0.25
    for k in ("means", "quats", "scales", "opacities", "colors"):
        cfg[k] = cfg[k].clone().requires_grad_(True)
    N = cfg["means"].shape[0]
    state = dict(grad2d=None, count=None, radii=None)
    ref = (np.zeros(N), np.zeros(N), np.zeros(N))
    for frame in range(2):
        colors, alphas, meta = sp.rasterization(**cfg)
        meta["means2d"].retain_grad()
        (colors.square().mean() + alphas.mean()).backward()
        for use_abs in (False, True):
            st = dict(grad2d=None, count=None, radii=None) if use_abs else state
            densify.update_state(st, meta, N, packed=packed, absgrad=use_abs, refine_scale2d=True)
            grads = meta["means2d"].absgrad if use_abs else meta["means2d"].grad
            base = (np.zeros(N), np.zeros(N), np.zeros(N)) if use_abs else ref
            want = oracle.update_state(n(grads), n(meta["radii"]), n(meta["gaussian_ids"]) if packed else None,
                                       meta["width"], meta["height"], meta["n_cameras"], *base)
            if not use_abs:
                ref = want
            np.testing.assert_allclose(n(st["grad2d"]), want[0], rtol=1e-5, atol=1e-12)
            assert np.array_equal(n(st["count"]), want[1])
            np.testing.assert_allclose(n(st["radii"]), want[2], rtol=1e-6)
        for k in ("means", "quats", "scales", "opacities", "colors"):
            cfg[k].grad = None
    assert ref[1].max() >= 2 and (ref[0] > 0).sum() > 1000 and ref[2].max() > 0


def test_compute_relocation():
    import splatad_b200 as sp
    from oracle import densify as oracle
    n_max = 51
    binoms = np.zeros((n_max, n_max), np.float32)
    for a in range(n_max):
        for b in range(a + 1):
            binoms[a, b] = math.comb(a, b)
    rng = np.random.default_rng(7)
    N = 3000
    op = (rng.random(N) * 0.985 + 0.005).astype(np.float32)
    sc = np.exp(rng.normal(-1.0, 0.7, (N, 3))).astype(np.float32)
    ratios = rng.integers(-2, 60, N)
    ratios[:n_max] = np.arange(1, n_max + 1)
    r_dev = t(ratios, torch.int64)
    got_o, got_s = sp.compute_relocation(t(op), t(sc), r_dev, t(binoms))
    # clamped in place, as the reference's wrapper does (gsplat/relocation.py:43)
    assert int(r_dev.min()) == 1 and int(r_dev.max()) == n_max
    want_o, want_s = oracle.compute_relocation(op, sc, ratios, binoms)
    np.testing.assert_allclose(n(got_o), want_o, rtol=1e-4, atol=1e-7)
    # the scale factor divides by an alternating float32 sum: a few entries lose another digit
    np.testing.assert_allclose(n(got_s), want_s, rtol=5e-4)
    assert (np.abs(n(got_s) - want_s) > 1e-4 * want_s).mean() < 0.01
    # one copy changes nothing
    same_o, same_s = sp.compute_relocation(t(op), t(sc), torch.ones(N, dtype=torch.int32, device=DEV), t(binoms))
    np.testing.assert_allclose(n(same_o), op, rtol=1e-6, atol=6e-8)   # 1 - (1 - o) rounds twice
    np.testing.assert_allclose(n(same_s), sc, rtol=1e-5)
    e_o, e_s = sp.compute_relocation(t(op[:0]), t(sc[:0]), r_dev[:0], t(binoms))
    assert e_o.shape == (0,) and e_s.shape == (0, 3)
