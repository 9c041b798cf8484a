"""ctypes loader for ``libmoonep_b200.so`` (plain C ABI, see ``_build.py``).

The reference binds its native code with pybind11 into ``moonep._C`` (csrc/bindings.cu:13-53).
Here every native entry point is an ``extern "C"`` function that takes raw pointers, sizes and
a ``cudaStream_t``; Python passes ``tensor.data_ptr()``.  Argument validation therefore lives
in the Python callers, which is also where the reference keeps its asserts.
"""
from __future__ import annotations

import ctypes
import os
import threading

from . import _build

_lock = threading.Lock()
_lib = None

P = ctypes.c_void_p
I = ctypes.c_int
L = ctypes.c_int64
F = ctypes.c_float

# name -> (restype, [argtypes]).  Filled by the modules that own the entry points.
_SIGNATURES: dict[str, tuple] = {}


def declare(name: str, restype, argtypes) -> None:
    _SIGNATURES[name] = (restype, list(argtypes))
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.restype = restype
        fn.argtypes = list(argtypes)


def lib() -> ctypes.CDLL:
    """Load (building first if the shared object is missing) and return the library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _build.LIB_PATH
        if not os.path.exists(path) or os.environ.get("MOONEP_B200_REBUILD") == "1":
            _build.build()
        handle = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
        for name, (restype, argtypes) in _SIGNATURES.items():
            if hasattr(handle, name):
                fn = getattr(handle, name)
                fn.restype = restype
                fn.argtypes = argtypes
        _lib = handle
    return _lib


# Number of native calls that launch at least one of this library's kernels (benchmarks read and
# reset it to report how many launches a step takes).
LAUNCHES = 0
_LAUNCH_PREFIXES = ("mep_launch_", "mep_gemm_launch", "mep_router_", "mep_swiglu_", "mep_sgd_")


def call(name: str, *args):
    """Call a declared entry point; raises if the symbol is missing (no silent fallback)."""
    global LAUNCHES
    if name.startswith(_LAUNCH_PREFIXES):
        LAUNCHES += 1
    handle = lib()
    try:
        fn = getattr(handle, name)
    except AttributeError as exc:  # pragma: no cover - build problem
        raise RuntimeError(f"native symbol {name} missing from {_build.LIB_PATH}") from exc
    if name in _SIGNATURES and fn.argtypes is None:
        fn.restype, fn.argtypes = _SIGNATURES[name][0], _SIGNATURES[name][1]
    return fn(*args)


def ptr(t) -> int:
    """``data_ptr`` of a tensor, or 0 for ``None``."""
    return 0 if t is None else t.data_ptr()


def last_error() -> str:
    handle = lib()
    handle.mep_last_error.restype = ctypes.c_char_p
    msg = handle.mep_last_error()
    return msg.decode() if msg else ""
