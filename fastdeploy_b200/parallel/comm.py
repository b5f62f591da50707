"""Peer-memory communicator: one process per GPU, buffers shared through CUDA IPC.

``Communicator`` sits on top of a ``torch.distributed`` process group (NCCL on GPUs; the group is
only used to exchange IPC handles and as the baseline the fused kernels are compared against). Every
rank allocates a *symmetric heap* through csrc/kernels/comm.cu, publishes its IPC handle, opens the
peers' handles and from then on addresses any peer's heap by ``(rank, offset)``. Kernels get raw
peer pointers; no library kernel is ever handed one.

The reference has no communication layer (it scales by independent model instances,
serving/src/fastdeploy_runtime.cc:162-271), so nothing here has a counterpart there.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import _native
from ..ops.base import StatusWord, current_stream_ptr, dtype_code

ALIGN = 1024        # heap allocations are aligned for 128B-swizzled TMA tiles
FLAG_BYTES = 4096   # signal area at the start of the heap: barrier slots + scratch counters


def _lib():
    lib = _native.kernels()
    if not getattr(lib, "_comm_ready", False):
        lib.fdb_comm_alloc.restype = ctypes.c_void_p
        lib.fdb_comm_alloc.argtypes = [ctypes.c_longlong]
        lib.fdb_comm_free.argtypes = [ctypes.c_void_p]
        lib.fdb_comm_ipc_handle.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        lib.fdb_comm_ipc_open.restype = ctypes.c_void_p
        lib.fdb_comm_ipc_open.argtypes = [ctypes.c_void_p]
        lib.fdb_comm_ipc_close.argtypes = [ctypes.c_void_p]
        lib.fdb_comm_barrier.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int, ctypes.c_uint,
                                         ctypes.c_void_p, ctypes.c_void_p]
        lib.fdb_comm_allgather.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_longlong,
                                           ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        lib.fdb_comm_reduce.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_longlong,
                                        ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        lib.fdb_comm_slot_reduce.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p,
                                             ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                             ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        lib.fdb_comm_slot_reduce_res.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p,
                                                 ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                                 ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                 ctypes.c_void_p, ctypes.c_void_p]
        lib.fdb_comm_slot_reduce_ln.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p,
                                                ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float,
                                                ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                                ctypes.c_float]
        lib.fdb_comm_slot_reduce_ln_pull.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p,
                                                     ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                     ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                     ctypes.c_float, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                                     ctypes.c_int, ctypes.c_float]
        lib._comm_ready = True
    return lib


@dataclass
class HeapBlock:
    """A same-offset allocation on every rank's heap."""
    offset: int
    nbytes: int


class HeapLayout:
    """Bump allocator over the symmetric heap; identical call sequences on all ranks give identical
    offsets, which is what makes the heap symmetric. Pure bookkeeping, usable without a GPU."""

    def __init__(self, capacity: int, reserved: int = FLAG_BYTES):
        self.capacity = capacity
        self.top = (reserved + ALIGN - 1) // ALIGN * ALIGN
        self.blocks: Dict[str, HeapBlock] = {}

    def alloc(self, name: str, nbytes: int) -> HeapBlock:
        if name in self.blocks:
            b = self.blocks[name]
            if b.nbytes < nbytes:
                raise ValueError(f"heap block {name!r} exists with {b.nbytes} bytes, {nbytes} requested")
            return b
        size = (nbytes + ALIGN - 1) // ALIGN * ALIGN
        if self.top + size > self.capacity:
            raise MemoryError(f"symmetric heap exhausted: {self.top + size} > {self.capacity}")
        b = HeapBlock(self.top, nbytes)
        self.top += size
        self.blocks[name] = b
        return b


def shard_rows(total_rows: int, world: int, multiple: int = 128) -> int:
    """Rows per rank of an evenly sharded, tile-aligned row dimension."""
    if total_rows % world != 0 or (total_rows // world) % multiple != 0:
        raise ValueError(f"{total_rows} rows do not split into {world} shards of a multiple of {multiple}")
    return total_rows // world


class Communicator:
    def __init__(self, group=None, heap_bytes: int = 1 << 30, device: Optional[torch.device] = None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if self.world > 8:
            raise ValueError("at most 8 ranks (one NVSwitch domain)")
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.layout = HeapLayout(heap_bytes)
        self.status = StatusWord(self.device)
        lib = _lib()
        with torch.cuda.device(self.device):
            self.base = lib.fdb_comm_alloc(heap_bytes)
            if not self.base:
                raise RuntimeError("comm: " + _native.last_error())
            handle = ctypes.create_string_buffer(64)
            if lib.fdb_comm_ipc_handle(self.base, handle) != 0:
                raise RuntimeError("comm: " + _native.last_error())
            handles: List[Optional[bytes]] = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(handles, handle.raw, group=group)
            else:
                handles[0] = handle.raw
            self.peer_base: List[int] = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.peer_base.append(self.base)
                else:
                    p = lib.fdb_comm_ipc_open(ctypes.create_string_buffer(h, 64))
                    if not p:
                        raise RuntimeError(f"comm: cannot open rank {r}'s heap: " + _native.last_error())
                    self.peer_base.append(p)
        self.heap_bytes = heap_bytes
        self.epoch = 0
        self._closed = False
        if self.world > 1:
            dist.barrier(group=group)     # every heap is mapped (and zeroed) before anyone signals

    # ------------------------------------------------------------------ addressing
    def ptr(self, rank: int, block: HeapBlock, byte_offset: int = 0) -> int:
        return self.peer_base[rank] + block.offset + byte_offset

    def ptrs(self, block: HeapBlock, byte_offset: int = 0):
        arr = (ctypes.c_void_p * 8)()
        for r in range(self.world):
            arr[r] = self.ptr(r, block, byte_offset)
        return arr

    def alloc(self, name: str, nbytes: int) -> HeapBlock:
        return self.layout.alloc(name, nbytes)

    def tensor(self, block: HeapBlock, shape: Sequence[int], dtype: torch.dtype, byte_offset: int = 0) -> torch.Tensor:
        """This rank's part of ``block`` as a tensor (no copy)."""
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        assert byte_offset + nbytes <= block.nbytes
        cai = {"shape": (nbytes,), "typestr": "|u1", "data": (self.base + block.offset + byte_offset, False),
               "version": 2}
        holder = type("_Heap", (), {"__cuda_array_interface__": cai})()
        t = torch.as_tensor(holder, device=self.device)
        return t.view(dtype).view(*shape)

    # ------------------------------------------------------------------ collectives on peer memory
    def barrier(self, stream: Optional[int] = None) -> None:
        """Device-side barrier: returns once it is queued; kernels queued after it on the same
        stream run after every rank's barrier kernel has seen all arrivals (bounded wait)."""
        self.epoch += 1
        flags = (ctypes.c_void_p * 8)()
        for r in range(self.world):
            flags[r] = self.peer_base[r]          # barrier slots live at heap offset 0
        rc = _lib().fdb_comm_barrier(flags, self.world, self.rank, self.epoch, self.status.ptr,
                                     ctypes.c_void_p(stream if stream is not None else current_stream_ptr()))
        if rc != 0:
            raise RuntimeError("comm: " + _native.last_error())

    def all_gather(self, block: HeapBlock, nbytes_per_rank: int, out: torch.Tensor, byte_offset: int = 0) -> None:
        """``out[r] = rank r's block``; the caller places barriers around it."""
        rc = _lib().fdb_comm_allgather(self.ptrs(block, byte_offset), ctypes.c_void_p(out.data_ptr()), nbytes_per_rank,
                                       self.world, self.rank, ctypes.c_void_p(current_stream_ptr()))
        if rc != 0:
            raise RuntimeError("comm: " + _native.last_error())

    def reduce(self, block: HeapBlock, out: torch.Tensor, offset_elems: int, count: int, byte_offset: int = 0) -> None:
        """``out[i] = sum_r block_r[offset + i]`` (fp32 accumulation). ``offset = rank * count`` makes
        it a reduce-scatter, ``offset = 0`` with the full count an all-reduce."""
        rc = _lib().fdb_comm_reduce(self.ptrs(block, byte_offset), ctypes.c_void_p(out.data_ptr()), offset_elems, count,
                                    dtype_code(out.dtype), self.world, self.rank, ctypes.c_void_p(current_stream_ptr()))
        if rc != 0:
            raise RuntimeError("comm: " + _native.last_error())

    def all_reduce(self, x: torch.Tensor, name: str = "allreduce") -> torch.Tensor:
        """One-shot all-reduce through the heap: copy in, barrier, pull + sum, barrier."""
        blk = self.alloc(name, x.numel() * x.element_size())
        mine = self.tensor(blk, x.shape, x.dtype)
        mine.copy_(x)
        self.barrier()
        out = torch.empty_like(x)
        self.reduce(blk, out, 0, x.numel())
        self.barrier()
        return out

    def reduce_scatter(self, x: torch.Tensor, name: str = "reducescatter") -> torch.Tensor:
        assert x.shape[0] % self.world == 0
        blk = self.alloc(name, x.numel() * x.element_size())
        self.tensor(blk, x.shape, x.dtype).copy_(x)
        self.barrier()
        rows = x.shape[0] // self.world
        out = torch.empty((rows,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        self.reduce(blk, out, self.rank * out.numel(), out.numel())
        self.barrier()
        return out

    def all_gather_tensor(self, x: torch.Tensor, name: str = "allgather") -> torch.Tensor:
        blk = self.alloc(name, x.numel() * x.element_size())
        self.tensor(blk, x.shape, x.dtype).copy_(x)
        self.barrier()
        out = torch.empty((self.world,) + tuple(x.shape), dtype=x.dtype, device=x.device)
        self.all_gather(blk, x.numel() * x.element_size(), out)
        self.barrier()
        return out.view((self.world * x.shape[0],) + tuple(x.shape[1:]))

    def check(self, what: str = "comm") -> None:
        self.status.check(what)

    def close(self) -> None:
        """Unmaps the peers' heaps and frees this rank's. Call between steps with nothing in flight."""
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            self.dist.barrier(group=self.group)
        lib = _lib()
        for r, p in enumerate(self.peer_base):
            if r != self.rank:
                lib.fdb_comm_ipc_close(p)
        lib.fdb_comm_free(self.base)
