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


def _covars(quats, scales):
    """Upper triangles [N, 6] of (R S)(R S)^T: the input the entry points take instead of quats / scales."""
    q = torch.nn.functional.normalize(quats, dim=-1)
    w, x, y, z = q.unbind(-1)
    R = torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y),
                     2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x),
                     2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)], -1).reshape(-1, 3, 3)
    M = R * scales[:, None, :]
    cov = M @ M.transpose(1, 2)
    return torch.stack([cov[:, 0, 0], cov[:, 0, 1], cov[:, 0, 2], cov[:, 1, 1], cov[:, 1, 2], cov[:, 2, 2]],
                       -1).contiguous()


def _count_both(lib, N, C, seed, use_covars=False):
    from splatad_b200 import _lib
    means, quats, scales, vel, viewmats, Ks, lin, ang, rs = _scene(N, C, seed)
    stream = torch.cuda.current_stream().cuda_stream
    if use_covars:
        covars = _covars(quats, scales)
        shape = (_p(covars), None, None)
    else:
        shape = (None, _p(quats), _p(scales))
    head = (C, N, _p(means), *shape, _p(vel), _p(viewmats), _p(Ks), 640, 480, _p(lin),
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


def test_noalloc_count_takes_covariances_and_leaves_device_memory_alone():
    """The covariance input path (no quaternions / scales), and the claim in the name: once the
    first call on the device has happened, a call changes neither the free device memory the driver
    reports nor what torch's allocator holds. Inputs and outputs are made before the measurement."""
    from splatad_b200 import _lib
    lib = _lib.load()
    ref_ptr, ref_nnz, ptr, nnz = _count_both(lib, 9_000, 2, seed=13, use_covars=True)   # also the warm-up call
    assert ref_nnz > 100 and nnz == ref_nnz and torch.equal(ptr, ref_ptr)
    C, N = 2, 9_000
    means, quats, scales, vel, viewmats, Ks, lin, ang, rs = _scene(N, C, 14)
    covars = _covars(quats, scales)
    indptr = torch.zeros(C + 1, dtype=torch.int32, device=DEV)
    count = torch.zeros(1, dtype=torch.int64, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    held_before, reserved_before = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    _lib.check(lib.splatad_projection_packed_count_noalloc(
        C, N, _p(means), _p(covars), None, None, _p(vel), _p(viewmats), _p(Ks), 640, 480, _p(lin), _p(ang), _p(rs),
        0.3, 0.01, 1e10, 0.0, _p(indptr), _p(count), stream))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)
    assert torch.cuda.memory_allocated() == held_before and torch.cuda.memory_reserved() == reserved_before
    assert int(count) > 100 and int(indptr[-1]) == int(count)


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
