"""Densification hooks: the two places where the reference's training strategies touch device
code with the render path's outputs.

  update_state        gsplat/strategy/default.py:203-258 (``DefaultStrategy._update_state``), one
                      fused kernel instead of a chain of torch ops
  compute_relocation  gsplat/relocation.py:10-49 (kernel gsplat/cuda/csrc/relocation.cu:4-31)

Both run on the C-ABI CUDA library; there is no CPU fallback.
"""

from __future__ import annotations

from typing import Any, Dict, Tuple

import torch
from torch import Tensor

from . import _lib
from .ops import _call, _f


@torch.no_grad()
def update_state(
    state: Dict[str, Any],
    info: Dict[str, Any],
    n_gaussian: int,
    packed: bool = False,
    absgrad: bool = False,
    refine_scale2d: bool = False,
    key_for_gradient: str = "means2d",
) -> None:
    """Adds one rendered frame to the running densification statistics in ``state``: ``grad2d`` (sum
    of the screen-space gradient norms), ``count`` (number of sensors that saw the Gaussian) and,
    when ``refine_scale2d``, ``radii`` (largest normalised screen radius). ``info`` is the ``meta``
    of :func:`splatad_b200.rasterization` after ``backward()``; tensors that are still ``None`` in
    ``state`` are created, as the reference does on its first frame."""
    for key in ["width", "height", "n_cameras", "radii", "gaussian_ids", key_for_gradient]:
        assert key in info, f"{key} is required but missing."
    src = info[key_for_gradient]
    grads = src.absgrad if absgrad else src.grad
    assert grads is not None, "the gradient of the 2D means is missing: call retain_grad() and backward() first"
    grads = _f(grads)
    dev = grads.device
    for key in ("grad2d", "count") + (("radii",) if refine_scale2d else ()):
        if state.get(key) is None:
            state[key] = torch.zeros(n_gaussian, device=dev)
    radii = info["radii"].to(torch.int32).contiguous()
    if packed:
        gaussian_ids = info["gaussian_ids"].to(torch.int64).contiguous()
        total = gaussian_ids.numel()
        assert grads.shape == (total, 2) and radii.shape == (total, 2), (grads.shape, radii.shape)
    else:
        gaussian_ids = None
        C, N = radii.shape[:2]
        assert N == n_gaussian and grads.shape == (C, N, 2), (grads.shape, radii.shape, n_gaussian)
        total = C * N
    for key in ("grad2d", "count") + (("radii",) if refine_scale2d else ()):
        t = state[key]
        assert t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n_gaussian, key
    _call("splatad_densify_update_state", total, n_gaussian, _lib.ptr(grads), _lib.ptr(radii),
          _lib.ptr(gaussian_ids), int(info["width"]), int(info["height"]), int(info["n_cameras"]),
          _lib.ptr(state["grad2d"]), _lib.ptr(state["count"]),
          _lib.ptr(state["radii"]) if refine_scale2d else None, _lib.stream_ptr(dev))


@torch.no_grad()
def compute_relocation(
    opacities: Tensor,  # [N]
    scales: Tensor,  # [N, 3]
    ratios: Tensor,  # [N]
    binoms: Tensor,  # [n_max, n_max]
) -> Tuple[Tensor, Tensor]:
    """New opacities [N] and scales [N, 3] of Gaussians that are split ``ratios`` ways, equation (9) of
    "3D Gaussian Splatting as Markov Chain Monte Carlo". ``ratios`` is clamped to 1..n_max in place,
    like the reference's wrapper does."""
    N = opacities.shape[0]
    n_max, _ = binoms.shape
    assert scales.shape == (N, 3), scales.shape
    assert ratios.shape == (N,), ratios.shape
    opacities, scales, binoms = _f(opacities), _f(scales), _f(binoms)
    ratios.clamp_(min=1, max=n_max)
    ratios = ratios.int().contiguous()
    new_opacities = torch.empty_like(opacities)
    new_scales = torch.empty_like(scales)
    if N:
        _call("splatad_compute_relocation", N, _lib.ptr(opacities), _lib.ptr(scales), _lib.ptr(ratios),
              _lib.ptr(binoms), n_max, _lib.ptr(new_opacities), _lib.ptr(new_scales),
              _lib.stream_ptr(opacities.device))
    return new_opacities, new_scales
