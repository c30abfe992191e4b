"""Loader for ``libsplatad_b200.so`` (the C-ABI CUDA library) and small helpers around it.

The argument types of every entry point are derived from ``include/splatad_b200.h`` so the
Python bindings cannot drift from the header. There is no CPU fallback: if the shared library
is missing, or an entry point is called with tensors that are not on a CUDA device, an
exception is raised.
"""

from __future__ import annotations

import ctypes
import os
import re
import subprocess
import time
from typing import Dict, List, Optional, Tuple

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_REPO_DIR = os.path.dirname(_PKG_DIR)
LIB_PATH = os.path.join(_PKG_DIR, "libsplatad_b200.so")
HEADER_PATH = os.path.join(_REPO_DIR, "include", "splatad_b200.h")
CSRC_DIR = os.path.join(_PKG_DIR, "csrc")

# SPLATAD_DEBUG=1: the stand-in for a memory checker. Every workspace gets a tail of canary bytes
# that is verified after each library call (a kernel that wrote past the size it was told shows up
# as an exception naming the workspace), every call is followed by a synchronisation and an error
# check, and ops.py validates the index lists before the compositing kernels follow them. Slow; for
# test runs, not for production frames.
DEBUG = os.environ.get("SPLATAD_DEBUG", "0") == "1"
CANARY_BYTES = 512
CANARY_VALUE = 0xA5

OK = 0
ERR_BAD_ARG = 1
ERR_CHANNELS = 2
ERR_KEY_BITS = 3
ERR_WORKSPACE = 4
ERR_CUDA = 5
ERR_OVERFLOW = 6
MAX_CHANNELS = 32

_SCALARS = {
    "int": ctypes.c_int,
    "int32_t": ctypes.c_int32,
    "uint32_t": ctypes.c_uint32,
    "int64_t": ctypes.c_int64,
    "uint64_t": ctypes.c_uint64,
    "size_t": ctypes.c_size_t,
    "float": ctypes.c_float,
}


def parse_header(path: str = HEADER_PATH) -> Dict[str, Tuple[object, List[object]]]:
    """Returns {symbol: (restype, [argtypes])} for every function declared in the header."""
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
    text = text.replace('extern "C" {', "")
    decls = {}
    for m in re.finditer(r"([\w\s\*]+?)\b(splatad_\w+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        if "*" in ret:
            restype = ctypes.c_char_p if "char" in ret else ctypes.c_void_p
        else:
            restype = _SCALARS[ret.replace("const", "").strip()]
        argtypes = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                if "*" in a:
                    argtypes.append(ctypes.c_void_p)
                else:
                    ty = a.replace("const", "").split()[0]
                    argtypes.append(_SCALARS[ty])
        decls[name] = (restype, argtypes)
    return decls


def build(verbose: bool = False) -> str:
    """Compiles the CUDA sources for sm_100a into ``libsplatad_b200.so`` (nvcc, in-tree)."""
    cmd = ["make", "-C", CSRC_DIR, "-j", str(os.cpu_count() or 4)]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or proc.returncode != 0:
        print(proc.stdout)
    if proc.returncode != 0:
        raise RuntimeError("building libsplatad_b200.so failed:\n" + proc.stdout[-4000:])
    return LIB_PATH


_lib: Optional[ctypes.CDLL] = None


def load() -> ctypes.CDLL:
    """Loads the shared library (once) and sets the ctypes signatures from the header."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA extension has not been built "
            "(run `python -c 'import __graft_entry__ as g; g.build()'` or `make -C splatad_b200/csrc`). "
            "splatad_b200 has no CPU fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in parse_header().items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    return load().splatad_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """Maps a status code to the exception type the reference raises for the same condition."""
    if status == OK:
        return
    msg = last_error() or f"splatad_b200 error {status}"
    if status in (ERR_BAD_ARG, ERR_CHANNELS):
        raise ValueError(msg)
    raise RuntimeError(msg)


class DevPtr(int):
    """A device address (or stream handle) that remembers which GPU it belongs to, so that
    :func:`call` can make that GPU current for the launch and refuse arguments from two GPUs."""

    def __new__(cls, value: int, device_index: int):
        obj = int.__new__(cls, value)
        obj.device_index = device_index
        return obj


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    """Device pointer of a contiguous CUDA tensor (None stays NULL)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError("splatad_b200 ops need CUDA tensors (there is no CPU fallback)")
    if not t.is_contiguous():
        raise RuntimeError("splatad_b200 ops need contiguous tensors")
    return DevPtr(t.data_ptr(), t.device.index)


def stream_ptr(device: torch.device) -> int:
    index = device.index if device.index is not None else torch.cuda.current_device()
    return DevPtr(torch.cuda.current_stream(device).cuda_stream, index)


def call(name: str, *args) -> None:
    """Calls entry point ``name`` with the GPU of its arguments current (the reference wraps every
    binding in a device guard, gsplat/cuda/csrc/*.cu ``DEVICE_GUARD``): the launch, the stream handle
    and the library's per-device state all refer to the device the tensors live on, whatever device
    the calling thread has selected. Arguments from two different GPUs raise ``ValueError`` before
    anything is launched."""
    dev = None
    for a in args:
        idx = getattr(a, "device_index", None)
        if idx is None:
            continue
        if dev is None:
            dev = idx
        elif idx != dev:
            raise ValueError(f"{name}: arguments live on cuda:{dev} and cuda:{idx}; every tensor of a call "
                             "must be on the same device")
    fn = getattr(load(), name)
    if dev is None or dev == torch.cuda.current_device():
        check(fn(*args))
    else:
        with torch.cuda.device(dev):
            check(fn(*args))
    if DEBUG and dev is not None:
        torch.cuda.synchronize(dev)     # raises here, with this call's name on the stack, if a kernel failed
        check_canaries(name)


# ---------------------------------------------------------------------------------------------
# Grow-only per-device workspaces and pinned host slots (the library itself never allocates).
# ---------------------------------------------------------------------------------------------
_workspaces: Dict[Tuple[str, int, int], torch.Tensor] = {}
_pinned: Dict[Tuple[str, int], torch.Tensor] = {}
_free_slots: Dict[Tuple[int, int], List[torch.Tensor]] = {}


def workspace(tag: str, nbytes: int, device: torch.device) -> torch.Tensor:
    """Scratch buffer for (tag, device, current stream of that device). Work enqueued on one stream
    is ordered, so consecutive calls may share a buffer; two streams never do."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (tag, index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        # grow with headroom so slowly growing scenes do not reallocate every frame
        size = max(int(nbytes * 1.25) + 1024, 1 << 16)
        if DEBUG:
            # exactly the bytes asked for, canary bytes right behind them; the library is told the
            # size without the canaries
            whole = torch.empty(nbytes + CANARY_BYTES, dtype=torch.uint8, device=device)
            whole[nbytes:].fill_(CANARY_VALUE)
            _canaries[key] = whole[nbytes:]
            buf = whole[:nbytes]
        else:
            buf = torch.empty(size, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


_canaries: Dict[Tuple[str, int, int], torch.Tensor] = {}


def check_canaries(after: str = "") -> None:
    """Debug mode: raises if any workspace's canary bytes were overwritten."""
    for key, tail in _canaries.items():
        if not bool((tail == CANARY_VALUE).all()):
            bad = int((tail != CANARY_VALUE).nonzero()[0])
            raise RuntimeError(f"workspace '{key[0]}' on cuda:{key[1]} was written {bad} bytes past its end "
                               f"(noticed after {after or 'a library call'})")


def pinned_counts(tag: str, device: torch.device, n: int = 4) -> torch.Tensor:
    """One pinned host slot per (tag, device) for calls that read their count before returning."""
    key = (tag, device.index if device.index is not None else torch.cuda.current_device())
    buf = _pinned.get(key)
    if buf is None or buf.numel() < n:
        buf = torch.zeros(n, dtype=torch.int64).pin_memory()
        _pinned[key] = buf
    return buf


def _stream_key(device: torch.device) -> Tuple[int, int]:
    index = device.index if device.index is not None else torch.cuda.current_device()
    return index, torch.cuda.current_stream(device).cuda_stream


def acquire_pinned_slot(device: torch.device) -> torch.Tensor:
    """A pinned 4 x int64 host slot owned by one outstanding call (its counts arrive there
    asynchronously); give it back with :func:`release_pinned_slot` once it has been read. Slots are
    recycled per (device, stream): a plan copies its counters twice (the count early, everything at
    its end), and only work enqueued later on the same stream is ordered behind the second copy."""
    free = _free_slots.get(_stream_key(device))
    slot = free.pop() if free else torch.zeros(8, dtype=torch.int64).pin_memory()
    slot._splatad_stream_key = _stream_key(device)
    return slot


_sequence = 0


def next_sequence() -> int:
    """A number no earlier early-count request has used (see splatad_isect_set_early_count)."""
    global _sequence
    _sequence += 1
    return _sequence


def wait_for_count(slot: torch.Tensor, sequence: int, event: torch.cuda.Event, patience_s: float = 0.02):
    """(n_isects, status) of a plan that was given ``slot`` (8 x int64 pinned: [0..3] the counters the
    plan copies at its end, [4..7] the early words {count, sequence, status, depth range}). Polls the triple for
    ``sequence`` - a kernel stores it there itself, long before the plan's own copy - and falls back to waiting for
    ``event`` (recorded behind the plan) when it does not show up within ``patience_s``."""
    view = slot.numpy()
    if sequence:
        deadline = time.perf_counter() + patience_s
        while view[5] != sequence:
            if time.perf_counter() > deadline:
                break
        else:
            return int(view[4]), int(view[6])
    event.synchronize()
    return int(view[0]), int(view[2])


def early_depth_range(slot: torch.Tensor, sequence: int):
    """(lo bits, hi bits) of the depth range a plan reported with its early count (slot[7], valid
    once slot[5] holds ``sequence``), or None when it reported none."""
    view = slot.numpy()
    if not sequence or view[5] != sequence or view[7] == 0:
        return None
    word = int(view[7]) & 0xFFFFFFFFFFFFFFFF
    return word & 0xFFFFFFFF, word >> 32


def release_pinned_slot(slot: torch.Tensor) -> None:
    free = _free_slots.setdefault(slot._splatad_stream_key, [])
    if len(free) < 16:
        free.append(slot)


def release_workspaces() -> None:
    _workspaces.clear()
    _canaries.clear()
    _pinned.clear()
    _free_slots.clear()
