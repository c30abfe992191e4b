"""CPU oracle of the SplatAD render hot path. TEST INFRASTRUCTURE ONLY.

This package restates, on the CPU, the algorithm of the reference (carlinds/splatad, a gsplat
fork) for projection, spherical harmonics, tile intersection and alpha compositing. It exists
to check the CUDA library of ``splatad_b200`` and to time a CPU baseline; nothing in
``splatad_b200`` imports it, and it must never be used as a product path or fallback.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU legs of ``bench.py`` may import it.

Parity status: pinned. Projection, SH, tile intersection and offsets are checked against the
reference's own PyTorch implementation (gsplat/cuda/_torch_impl.py, imported from the mounted
reference when the fixtures under ``tests/golden`` were generated); the per-pair compositing
arithmetic is checked against the reference's ``accumulate`` / ``accumulate_lidar``
(_torch_impl.py:610-820) run on explicit pair lists, with nerfacc's two published helpers
(``render_weight_from_alpha``, ``accumulate_along_rays``; nerfacc is an unpinned, un-vendored
dependency of the reference) restated in the fixture generator. The threshold / early-stop /
median rules of the CUDA kernels (gsplat/cuda/csrc/rasterization.cu:1466-1517, 2154-2218) have
no CPU counterpart in the reference and are pinned by hand-computed known-answer cases modelled
on tests/test_basic.py:1257-1281.
"""
