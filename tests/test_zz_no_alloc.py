"""The allocation-free packed count (``splatad_projection_packed_count_noalloc``) against the
regular, caller-workspace entry point, called straight through the C ABI.

Some hosts of this library are not allowed to allocate device memory once they are running: a
plugin inside an engine that owns the whole GPU through its own arena, or a loop whose rules ban
allocator calls after start-up. For them the per-(camera, block) counters sit in a fixed array
inside the library. The array is shared by every call and keeps whatever the previous call left,
so the check runs the entry point twice in a row - the second time on a smaller problem, where
stale counters of the first call would show up - and both results must equal the regular entry
point's exactly (they are integer counts: tolerance zero).

This file is named so that pytest collects it last.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _scene(N, C, seed):
    g = torch.Generator().manual_seed(seed)
    means = torch.empty(N, 3)
    means[:, 0] = torch.rand(N, generator=g) * 60 - 30
    means[:, 1] = torch.rand(N, generator=g) * 12 - 6
    means[:, 2] = torch.rand(N, generator=g) * 70 - 10
    quats = torch.randn(N, 4, generator=g)
    scales = torch.exp(torch.randn(N, 3, generator=g) * 0.7 - 1.5)
    vel = torch.randn(N, 3, generator=g)
    viewmats = torch.eye(4)[None].repeat(C, 1, 1)
    for c in range(C):
        viewmats[c, 0, 3] = 0.7 * c
    Ks = torch.tensor([[[400.0, 0.0, 320.0], [0.0, 400.0, 240.0], [0.0, 0.0, 1.0]]]).repeat(C, 1, 1)
    lin = torch.tensor([[8.0, 0.0, 0.0]]).repeat(C, 1)
    ang = torch.zeros(C, 3)
    rs = torch.full((C,), 0.02)
    return [t.to(DEV).contiguous() for t in (means, quats, scales, vel, viewmats, Ks, lin, ang, rs)]


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _count_both(lib, N, C, seed):
    from splatad_b200 import _lib
    means, quats, scales, vel, viewmats, Ks, lin, ang, rs = _scene(N, C, seed)
    stream = torch.cuda.current_stream().cuda_stream
    head = (C, N, _p(means), None, _p(quats), _p(scales), _p(vel), _p(viewmats), _p(Ks), 640, 480, _p(lin),
            _p(ang), _p(rs), 0.3, 0.01, 1e10, 0.0)
    # regular entry point: the caller brings the workspace
    ws = torch.empty(lib.splatad_projection_packed_workspace_bytes(C, N), dtype=torch.uint8, device=DEV)
    indptr_ref = torch.full((C + 1,), -1, dtype=torch.int32, device=DEV)
    nnz_ref = torch.full((1,), -1, dtype=torch.int64, device=DEV)
    _lib.check(lib.splatad_projection_packed_count(*head, _p(ws), ws.numel(), _p(indptr_ref), _p(nnz_ref), stream))
    # allocation-free entry point: inputs and outputs only
    indptr = torch.full((C + 1,), -2, dtype=torch.int32, device=DEV)
    nnz = torch.full((1,), -2, dtype=torch.int64, device=DEV)
    _lib.check(lib.splatad_projection_packed_count_noalloc(*head, _p(indptr), _p(nnz), stream))
    torch.cuda.synchronize()
    return indptr_ref.cpu(), int(nnz_ref), indptr.cpu(), int(nnz)


def test_noalloc_count_matches_workspace_count_twice_in_a_row():
    from splatad_b200 import _lib
    lib = _lib.load()
    # first call: larger problem (fills more of the shared array)
    ref_ptr, ref_nnz, ptr, nnz = _count_both(lib, 40_000, 3, seed=11)
    assert ref_nnz > 1000
    assert nnz == ref_nnz and torch.equal(ptr, ref_ptr)
    # second call right after it: smaller problem, different scene; stale counters must not leak in
    ref_ptr2, ref_nnz2, ptr2, nnz2 = _count_both(lib, 7_001, 2, seed=12)
    assert ref_nnz2 > 100 and ref_nnz2 != ref_nnz
    assert nnz2 == ref_nnz2 and torch.equal(ptr2, ref_ptr2)
    assert int(ptr2[0]) == 0 and int(ptr2[-1]) == nnz2


def test_noalloc_count_rejects_sizes_beyond_its_array():
    from splatad_b200 import _lib
    lib = _lib.load()
    # 300 cameras x ceil(60000 / 256) = 70500 block rows > 65536: refused before anything is launched
    C, N = 300, 60_000
    dummy = torch.zeros(16, device=DEV)
    indptr = torch.zeros(C + 1, dtype=torch.int32, device=DEV)
    nnz = torch.zeros(1, dtype=torch.int64, device=DEV)
    rc = lib.splatad_projection_packed_count_noalloc(
        C, N, _p(dummy), None, _p(dummy), _p(dummy), None, _p(dummy), _p(dummy), 640, 480, _p(dummy), _p(dummy),
        _p(dummy), 0.3, 0.01, 1e10, 0.0, _p(indptr), _p(nnz), None)
    assert rc == _lib.ERR_WORKSPACE
    assert "65536" in _lib.last_error()
    with pytest.raises(RuntimeError):
        _lib.check(rc)
