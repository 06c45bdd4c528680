"""ctypes bindings to the in-tree native libraries.

Every CUDA launcher is an ``extern "C" int ve_<name>(..., cudaStream_t)`` that returns a
``cudaError_t`` (0 = success).  Signatures are declared with a compact code string:
``p`` pointer, ``i`` int32, ``l`` int64, ``f`` float, ``d`` double.  The last stream argument is
appended automatically by :func:`call`.

On a machine with a GPU the kernel library is mandatory: a missing library raises instead of
falling back to eager PyTorch, so a silent fallback can never masquerade as the native path.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_CODES = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_int64, "f": ctypes.c_float,
          "d": ctypes.c_double, "s": ctypes.c_char_p}

_lock = threading.Lock()
_kernels = None
_host = None
_sigs: dict[str, str] = {}
launch_count = 0  # number of native kernel launchers invoked (bench.py reports it)


class NativeError(RuntimeError):
    pass


def _load(name: str, builder) -> ctypes.CDLL:
    path = Path(__file__).resolve().parent / "_native" / f"lib{name}.so"
    if not path.exists() or os.environ.get("VOLTA_REBUILD"):
        from . import _build
        getattr(_build, builder)()
    if not path.exists():
        raise NativeError(f"{path} is missing; run `python -m volta_engine_b200._build`")
    return ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)


def kernels() -> ctypes.CDLL:
    global _kernels
    if _kernels is None:
        with _lock:
            if _kernels is None:
                _kernels = _load("volta_kernels", "build_kernels")
    return _kernels


def host() -> ctypes.CDLL:
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                _host = _load("volta_host", "build_host")
    return _host


def have_kernels() -> bool:
    try:
        kernels()
        return True
    except Exception:
        return False


def _bind(lib: ctypes.CDLL, name: str, sig: str, restype=ctypes.c_int):
    fn = getattr(lib, name)
    fn.argtypes = [_CODES[c] for c in sig]
    fn.restype = restype
    return fn


_bound: dict[str, object] = {}


def ptr(t) -> int:
    """Device (or host) address of a tensor, or 0 for None."""
    if t is None:
        return 0
    return t.data_ptr()


def call(name: str, sig: str, *args) -> None:
    """Launch ``ve_<name>`` on the current CUDA stream; raises on a CUDA error code."""
    global launch_count
    fn = _bound.get(name)
    if fn is None:
        fn = _bind(kernels(), "ve_" + name, sig + "p")
        _bound[name] = fn
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(*args, stream)
    launch_count += 1
    if rc != 0:
        raise NativeError(f"ve_{name} failed with CUDA error {rc}")


def hcall(name: str, sig: str, *args, restype=ctypes.c_int):
    """Call a host-library function ``vh_<name>`` (no stream argument)."""
    key = "h:" + name
    fn = _bound.get(key)
    if fn is None:
        fn = _bind(host(), "vh_" + name, sig, restype)
        _bound[key] = fn
    return fn(*args)
