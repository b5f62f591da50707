"""Caching memory pools (csrc/kernels/allocator.cu): device memory and page-locked host memory in power-of-two size
classes, reused only after the stream that last touched a block has passed the point of its release.

``pinned_tensor`` / ``device_tensor`` hand out torch tensors that view pool memory, so staging buffers of the serving
path (request batches, result read-backs) cost no ``cudaHostAlloc`` / ``cudaMalloc`` after warm-up. The reference's
allocators are fastdeploy/core/allocate.h:26-56 (plain malloc / cudaMalloc / cudaMallocHost wrappers)."""
from __future__ import annotations

import ctypes
from typing import Dict, Sequence

import numpy as np
import torch

from .. import _native

DEVICE, PINNED = 0, 1


def _lib():
    lib = _native.kernels()
    if not getattr(lib, "_pool_ready", False):
        lib.fdb_pool_alloc.restype = ctypes.c_void_p
        lib.fdb_pool_alloc.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_longlong]
        lib.fdb_pool_free.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        lib.fdb_pool_trim.restype = ctypes.c_longlong
        lib.fdb_pool_stats.argtypes = [ctypes.POINTER(ctypes.c_longlong)]
        lib._pool_ready = True
    return lib


class _Block:
    """Keeps a pool block alive while a tensor views it; returns it to the pool when the last view dies."""

    def __init__(self, ptr: int, nbytes: int, kind: int, device: int):
        self.ptr, self.nbytes, self.kind, self.device = ptr, nbytes, kind, device

    def release(self, stream: int = None) -> None:
        if self.ptr:
            _lib().fdb_pool_free(ctypes.c_void_p(self.ptr), ctypes.c_void_p(stream or 0), 1 if stream is not None else 0)
            self.ptr = 0

    def __del__(self):
        try:
            if self.ptr:
                stream = None
                if torch.cuda.is_available():
                    dev = self.device if self.kind == DEVICE else torch.cuda.current_device()
                    stream = torch.cuda.current_stream(dev).cuda_stream
                self.release(stream)
        except Exception:
            pass


def _alloc(kind: int, device: int, nbytes: int) -> _Block:
    ptr = _lib().fdb_pool_alloc(kind, device, max(int(nbytes), 1))
    if not ptr:
        raise MemoryError(f"memory pool: {_native.last_error()}")
    return _Block(ptr, nbytes, kind, device)


def pinned_tensor(shape: Sequence[int], dtype: torch.dtype = torch.uint8) -> torch.Tensor:
    """A page-locked host tensor backed by the pool (``is_pinned()`` is true; copies to the device are asynchronous)."""
    n = int(np.prod(shape)) if len(shape) else 1
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    blk = _alloc(PINNED, -1, nbytes)
    buf = (ctypes.c_uint8 * max(nbytes, 1)).from_address(blk.ptr)
    buf._fdb_block = blk                       # the ctypes array owns the block; numpy and torch keep the array alive
    arr = np.frombuffer(buf, dtype=np.uint8, count=nbytes)
    return torch.from_numpy(arr).view(dtype).reshape(list(shape))


class _CudaArray:
    """``__cuda_array_interface__`` view of a pool block, so that torch can wrap device memory it did not allocate."""

    def __init__(self, blk: _Block, nbytes: int):
        self._blk = blk
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (blk.ptr, False), "version": 3,
                                         "strides": None}


def device_tensor(shape: Sequence[int], dtype: torch.dtype = torch.uint8, device: int = 0) -> torch.Tensor:
    """A device tensor backed by the pool (uninitialised)."""
    n = int(np.prod(shape)) if len(shape) else 1
    nbytes = max(n * torch.empty((), dtype=dtype).element_size(), 1)
    blk = _alloc(DEVICE, device, nbytes)
    t = torch.as_tensor(_CudaArray(blk, nbytes), device=torch.device("cuda", device))
    return t[:n * torch.empty((), dtype=dtype).element_size()].view(dtype).reshape(list(shape))


def trim() -> int:
    """Gives idle cached blocks back to the driver; returns the bytes released."""
    return int(_lib().fdb_pool_trim())


def stats() -> Dict[str, Dict[str, int]]:
    out = (ctypes.c_longlong * 10)()
    _lib().fdb_pool_stats(out)
    keys = ("allocated", "cached", "high_water", "driver_calls", "cache_hits")
    return {"device": dict(zip(keys, out[0:5])), "pinned": dict(zip(keys, out[5:10]))}
