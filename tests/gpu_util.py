"""Helpers shared by the GPU parity tests."""

import numpy as np
import torch

DEV = "cuda:0"


def t(a, dtype=torch.float32, device=DEV):
    if a is None:
        return None
    return torch.as_tensor(np.asarray(a)).to(dtype).to(device)


def n(x):
    return None if x is None else x.detach().cpu().numpy()


def assert_close(name, got, want, rtol, atol, mask=None, max_bad_frac=0.0):
    """allclose with a readable report; ``max_bad_frac`` tolerates a stated fraction of outliers
    (used only where a discrete decision may legitimately flip, and said so at the call site)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (name, got.shape, want.shape)
    err = np.abs(got - want)
    tol = atol + rtol * np.abs(want)
    bad = err > tol
    if mask is not None:
        bad = bad & np.broadcast_to(mask, bad.shape)
        total = max(int(np.broadcast_to(mask, bad.shape).sum()), 1)
    else:
        total = max(bad.size, 1)
    frac = bad.sum() / total
    if frac > max_bad_frac:
        idx = np.unravel_index(np.argmax(np.where(bad, err / np.maximum(tol, 1e-30), 0)), err.shape)
        raise AssertionError(
            f"{name}: {int(bad.sum())}/{total} entries ({frac:.2e}) beyond rtol={rtol} atol={atol}; "
            f"worst at {idx}: got {got[idx]!r} want {want[idx]!r} (max abs err {err[bad].max():.3e})")


def rel_l2(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
