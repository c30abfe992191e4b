"""Pins of the oracle's densification hooks: the running statistics against the reference's own
``DefaultStrategy._update_state`` (pure torch, run on the CPU by tests/golden/make_golden.py), and
equation (9) of the MCMC paper against closed forms (the reference has no CPU twin of its
relocation kernel, gsplat/cuda/csrc/relocation.cu:4-31)."""

import math

import numpy as np

from oracle import densify


def test_update_state_against_the_reference_strategy(golden):
    g = golden("densify_state")
    C, N, W, H = (int(g[k]) for k in ("C", "N", "width", "height"))
    for tag in ("grad", "abs"):
        grad2d, count = np.zeros(N), np.zeros(N)
        for frame in range(2):
            k = f"{tag}_f{frame}"
            grad2d, count, _ = densify.update_state(g[k + "_grads"], g[k + "_radii"], None, W, H, C, grad2d, count)
            np.testing.assert_allclose(grad2d, g[k + "_grad2d"], rtol=2e-6, atol=1e-9)
            assert np.array_equal(count, g[k + "_count"])
        assert count.max() > C   # two frames really accumulated
    grad2d, count, radii = np.zeros(N), np.zeros(N), np.zeros(N)
    for frame in range(2):
        k = f"packed_f{frame}"
        grad2d, count, radii = densify.update_state(g[k + "_grads"], g[k + "_radii"], g[k + "_ids"], W, H, C,
                                                    grad2d, count, radii)
        np.testing.assert_allclose(grad2d, g[k + "_grad2d"], rtol=2e-6, atol=1e-9)
        assert np.array_equal(count, g[k + "_count"])
        np.testing.assert_allclose(radii, g[k + "_state_radii"], rtol=1e-6)


def _binoms(n_max=51):
    b = np.zeros((n_max, n_max))
    for n in range(n_max):
        for k in range(n + 1):
            b[n, k] = math.comb(n, k)
    return b


def test_compute_relocation_closed_forms():
    b = _binoms()
    op = np.array([0.05, 0.3, 0.6, 0.9, 0.99])
    sc = np.random.default_rng(0).random((5, 3)) + 0.1
    # one copy: nothing changes
    o1, s1 = densify.compute_relocation(op, sc, np.ones(5, np.int64), b)
    np.testing.assert_allclose(o1, op, rtol=1e-12)
    np.testing.assert_allclose(s1, sc, rtol=1e-12)
    # two copies: x = 1 - sqrt(1 - o), denominator x + (x - x^2 / sqrt 2)
    o2, s2 = densify.compute_relocation(op, sc, np.full(5, 2), b)
    x = 1 - np.sqrt(1 - op)
    np.testing.assert_allclose(o2, x, rtol=1e-12)
    np.testing.assert_allclose(s2, sc * (op / (2 * x - x * x / math.sqrt(2)))[:, None], rtol=1e-12)
    # the n copies together are as opaque as the original: 1 - (1 - x)^n = o
    for n_copies in (3, 7, 51):
        on, sn = densify.compute_relocation(op, sc, np.full(5, n_copies), b)
        np.testing.assert_allclose(1 - (1 - on) ** n_copies, op, rtol=1e-10)
        assert (sn < sc).all() and (sn > 0).all()   # each copy is smaller
    # ratios are clamped to 1..n_max
    lo, _ = densify.compute_relocation(op, sc, np.zeros(5, np.int64), b)
    hi, _ = densify.compute_relocation(op, sc, np.full(5, 1000), b)
    np.testing.assert_allclose(lo, o1)
    np.testing.assert_allclose(hi, densify.compute_relocation(op, sc, np.full(5, 51), b)[0])
    # float32 evaluation in the kernel's order stays close to float64
    o32, s32 = densify.compute_relocation(op, sc, np.array([1, 5, 20, 51, 51]), b, dtype=np.float32)
    o64, s64 = densify.compute_relocation(op, sc, np.array([1, 5, 20, 51, 51]), b)
    np.testing.assert_allclose(o32, o64, rtol=2e-5)
    np.testing.assert_allclose(s32, s64, rtol=2e-4)
