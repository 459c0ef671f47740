"""ctypes binding of the in-tree native library ``libb200llm.so``.

The library is plain ``extern "C"``: tensors cross the boundary as raw device pointers plus the
current CUDA stream. On a machine with a GPU a missing or stale library is an error (nothing in
this package silently falls back to eager PyTorch on CUDA tensors); on a CPU-only machine the
library is only built, never loaded for execution.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

from . import build as _build

_lock = threading.Lock()
_lib = None
_status = {}

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_float = ctypes.c_float
c_long = ctypes.c_longlong


class NativeError(RuntimeError):
    pass


_launches = 0


def bump(n: int = 1) -> None:
    """Count kernels launched through this library (reported by the benchmark)."""
    global _launches
    _launches += n


def launch_count() -> int:
    return _launches


def available() -> bool:
    """True when CUDA tensors can be served by the native library."""
    return torch.cuda.is_available()


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        # The library is rebuilt whenever a source, a header or the flags changed since it was made (the
        # build is incremental: with nothing changed it only compares digests). A machine without nvcc
        # can only load a library whose stamps match the sources; a stale one is an error, never a
        # silent mismatch between the code that is read and the code that runs.
        path = _build.lib_path()
        try:
            path = _build.build(force=os.environ.get("B200_REBUILD") == "1")
        except RuntimeError as e:
            if "nvcc not found" not in str(e):
                raise NativeError(str(e)) from e
            if not _build.is_current():
                raise NativeError(f"{path} is missing or older than the sources under csrc/ and nvcc is not "
                                  f"available to rebuild it") from e
        try:
            _lib = ctypes.CDLL(str(path))
        except OSError as e:  # pragma: no cover
            raise NativeError(f"cannot load {path}: {e}") from e
        _lib.b200_abi_version.restype = c_int
        return _lib


def source_digest() -> str:
    """Digest of the sources the loaded library was built from (recorded by the benchmark)."""
    return _build.source_digest()


def status_tensor(device=None) -> torch.Tensor:
    """Per-device 4-int status block that kernels write when a bounded wait runs out."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    key = dev.index
    if key not in _status:
        t = torch.zeros(4, dtype=torch.int32, device=dev)
        _status[key] = t
        check(lib().b200_set_status_ptr(c_void_p(t.data_ptr())), "b200_set_status_ptr")
    return _status[key]


def read_status(clear: bool = True) -> tuple[int, int]:
    """Synchronising read of (error code, kernel id); 0 means no bounded wait ran out."""
    t = status_tensor()
    code, kid = (int(v) for v in t[:2].tolist())
    if clear and code != 0:
        t.zero_()
    return code, kid


def raise_on_status() -> None:
    code, kid = read_status()
    if code != 0:
        raise NativeError(f"native kernel {kid} reported error {code} (1: mbarrier wait timed out, "
                          f"2: peer flag wait timed out, 3: bad argument, 4: index out of range - kernel 401 / 402: "
                          f"token id >= vocabulary size in the embedding forward / backward)")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what} failed with CUDA error {rc}")


def stream_ptr() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())
