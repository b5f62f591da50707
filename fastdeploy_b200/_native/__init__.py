"""Loader for the in-tree native libraries (ctypes, plain C ABI).

``kernels()`` returns the CUDA kernel library and ``cpu()`` the host C++ library.
Both raise ``NativeLibraryError`` when the shared object is missing or cannot be
loaded - a GPU code path never silently falls back to eager PyTorch.
"""
from __future__ import annotations

import ctypes
import os
import threading

HERE = os.path.dirname(os.path.abspath(__file__))
KERNEL_LIB = os.path.join(HERE, "libfdb200_kernels.so")
CPU_LIB = os.path.join(HERE, "libfdb200_cpu.so")

# FDX_NATIVE_VARIANT=boundscheck swaps in the checked kernel library, =asan / tsan / ubsan the sanitised host
# library (both built by ``python -m fastdeploy_b200._native.build --mode <variant>``).
VARIANT = os.environ.get("FDX_NATIVE_VARIANT", "")
if VARIANT:
    _vdir = os.path.join(os.path.dirname(os.path.dirname(HERE)), "build", VARIANT)
    if VARIANT == "boundscheck":
        KERNEL_LIB = os.path.join(_vdir, "libfdb200_kernels.so")
    else:
        CPU_LIB = os.path.join(_vdir, "libfdb200_cpu.so")

_lock = threading.Lock()
_kernels = None
_cpu = None


class NativeLibraryError(RuntimeError):
    pass


def _load(path: str) -> ctypes.CDLL:
    if not os.path.exists(path):
        raise NativeLibraryError(
            f"{os.path.basename(path)} is not built; run `python -m fastdeploy_b200._native.build`")
    try:
        return ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    except OSError as e:  # pragma: no cover - depends on the machine
        raise NativeLibraryError(f"cannot load {path}: {e}") from e


def kernels() -> ctypes.CDLL:
    """CUDA kernel library (sm_100a)."""
    global _kernels
    with _lock:
        if _kernels is None:
            lib = _load(KERNEL_LIB)
            lib.fdb_last_error.restype = ctypes.c_char_p
            lib.fdb_plan_create.restype = ctypes.c_void_p
            lib.fdb_plan_add.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
            lib.fdb_plan_size.argtypes = [ctypes.c_void_p]
            lib.fdb_plan_launch_count.argtypes = [ctypes.c_void_p]
            lib.fdb_plan_launch_count.restype = ctypes.c_ulonglong
            lib.fdb_plan_run.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
            lib.fdb_plan_run_range.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
            lib.fdb_plan_destroy.argtypes = [ctypes.c_void_p]
            lib.fdb_op_launch.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
            lib.fdb_op_destroy.argtypes = [ctypes.c_void_p]
            _kernels = lib
        return _kernels


def cpu() -> ctypes.CDLL:
    """Host-side C++ library."""
    global _cpu
    with _lock:
        if _cpu is None:
            _cpu = _load(CPU_LIB)
        return _cpu


def kernels_available() -> bool:
    return os.path.exists(KERNEL_LIB)


def cpu_available() -> bool:
    return os.path.exists(CPU_LIB)


def last_error() -> str:
    msg = kernels().fdb_last_error()
    return msg.decode() if msg else ""


def bounds_report(reset: bool = True):
    """(count, text) of out-of-range data-dependent indices seen by the checked kernel library since the last
    reset; ``(0, "not a checked build")`` for the release library. Synchronises the device."""
    lib = kernels()
    if not lib.fdb_bounds_checked():
        return 0, "not a checked build"
    lib.fdb_bounds_report.restype = ctypes.c_longlong
    lib.fdb_bounds_report.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int]
    buf = ctypes.create_string_buffer(256)
    n = lib.fdb_bounds_report(buf, 256, 1 if reset else 0)
    if n < 0:
        raise NativeLibraryError(lib.fdb_last_error().decode())
    return int(n), buf.value.decode()
