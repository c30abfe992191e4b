"""CPU restatement of the densification hooks. TEST INFRASTRUCTURE ONLY - see ``oracle/__init__.py``.

  update_state        gsplat/strategy/default.py:203-258
  compute_relocation  gsplat/cuda/csrc/relocation.cu:4-31 with the clamp of gsplat/relocation.py:43
"""

from __future__ import annotations

import numpy as np


def update_state(grads, radii, gaussian_ids, width, height, n_cameras, grad2d, count, radii_state=None):
    """grads [C,N,2] / [nnz,2], radii int [C,N,2] / [nnz,2], gaussian_ids None (unpacked) or [nnz].
    Returns the new (grad2d, count, radii_state); radii_state is a true per-Gaussian maximum (the
    reference's indexed assignment keeps one of the candidates when a Gaussian appears twice)."""
    g = np.asarray(grads, np.float32).copy()
    g[..., 0] *= np.float32(width / 2.0 * n_cameras)
    g[..., 1] *= np.float32(height / 2.0 * n_cameras)
    radii = np.asarray(radii)
    if gaussian_ids is None:
        sel = radii[..., 0] > 0
        ids = np.where(sel)[1]
        g = g[sel]
        r = radii[sel].max(-1)
    else:
        ids = np.asarray(gaussian_ids)
        r = radii.max(-1)
    grad2d = np.asarray(grad2d, np.float64).copy()
    count = np.asarray(count, np.float64).copy()
    np.add.at(grad2d, ids, np.sqrt(g[:, 0].astype(np.float64) ** 2 + g[:, 1].astype(np.float64) ** 2))
    np.add.at(count, ids, 1.0)
    if radii_state is not None:
        radii_state = np.asarray(radii_state, np.float64).copy()
        np.maximum.at(radii_state, ids, r / float(max(width, height)))
    return grad2d, count, radii_state


def compute_relocation(opacities, scales, ratios, binoms, dtype=np.float64):
    opacities = np.asarray(opacities, dtype)
    scales = np.asarray(scales, dtype)
    binoms = np.asarray(binoms, dtype)
    n_max = binoms.shape[0]
    ratios = np.clip(np.asarray(ratios), 1, n_max).astype(np.int64)
    new_op = np.zeros_like(opacities)
    new_sc = np.zeros_like(scales)
    one = dtype(1)
    for idx in range(opacities.shape[0]):
        n = int(ratios[idx])
        x = one - (one - opacities[idx]) ** (one / dtype(n))
        new_op[idx] = x
        denom = dtype(0)
        for i in range(1, n + 1):
            for k in range(i):
                term = (dtype((-1) ** k) / np.sqrt(dtype(k + 1))) * x ** dtype(k + 1)
                denom = denom + binoms[i - 1, k] * term
        new_sc[idx] = (opacities[idx] / denom) * scales[idx]
    return new_op, new_sc
