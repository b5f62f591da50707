"""Serialised launch plans: a built plan written to one file that a C program replays without Python.

A plan is a list of native ops, each made by a ``fdb_*_create(descriptor)`` call of the kernel library; the
descriptors hold device addresses. ``export_plan`` writes

* the device buffers the plan touches (the caching allocator's blocks that contain any address the plan uses),
  with their bytes when they are constants (weights, tables: the bytes that do not change between two runs on
  different inputs) and as zero-filled space otherwise;
* every op's creation function, ``kind`` argument and descriptor bytes, plus the byte offsets inside the
  descriptor that hold device addresses, each as (buffer, offset);
* device arrays of device pointers (the embedding op's id / table lists), element by element;
* the plan's inputs and outputs (buffer, offset, dtype, dims, strides).

``csrc/runner/plan_runner.cu`` (``libfdb200_runner.so``, tool ``fdplan_run``) allocates the buffers, patches
the addresses, re-creates the ops through the same kernel library and launches them (as one CUDA graph).
The reference's counterpart is the serialised TensorRT engine that its C++ runtime loads without Python
(fastdeploy/runtime/backends/tensorrt/trt_backend.cc:61-114).

File layout (little endian): ``"FDPLAN1\\0"``; u32 buffers {u64 size, u8 has_data, data}; u32 ops {u16 len, name,
i32 kind, u32 desc_size, desc, u32 relocs {u32 desc_offset, u32 buffer, u64 offset}}; u32 tables {u32 buffer,
u64 offset, u32 count {i32 buffer, u64 offset}}; u32 io {u8 is_output, u16 len, name, u32 buffer, u64 offset,
u8 dtype, u8 ndim, i64 dims, i64 strides}.
"""
from __future__ import annotations

import ctypes
import hashlib
import struct
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _native
from ..ops.base import dtype_code

MAGIC = b"FDPLAN1\0"
_CHUNK = 64 << 20


class PlanExportError(RuntimeError):
    pass


def _pointer_slots(desc: ctypes.Structure) -> List[int]:
    """Byte offsets of every ``void*`` field (or element of a ``void*`` array) of a descriptor."""
    slots: List[int] = []
    for name, ctype in desc._fields_:
        off = getattr(type(desc), name).offset
        if ctype is ctypes.c_void_p:
            slots.append(off)
        elif isinstance(ctype, type) and issubclass(ctype, ctypes.Array) and ctype._type_ is ctypes.c_void_p:
            slots += [off + k * ctypes.sizeof(ctypes.c_void_p) for k in range(ctype._length_)]
    return slots


def _active_blocks(device: torch.device) -> List[Tuple[int, int]]:
    """(address, size) of every live block of the caching allocator on ``device``."""
    out = []
    for seg in torch.cuda.memory_snapshot():
        if seg.get("device") != device.index:
            continue
        addr = seg["address"]
        for b in seg["blocks"]:
            if b["state"] == "active_allocated":
                out.append((addr, b["size"]))
            addr += b["size"]
    return sorted(out)


class _Buffers:
    def __init__(self, device: torch.device):
        self.blocks = _active_blocks(device)
        self.addrs = [a for a, _ in self.blocks]
        self.used: Dict[int, int] = {}             # block index -> buffer id

    def locate(self, ptr: int, what: str) -> Tuple[int, int]:
        import bisect
        k = bisect.bisect_right(self.addrs, ptr) - 1
        if k < 0 or ptr >= self.blocks[k][0] + self.blocks[k][1]:
            raise PlanExportError(f"{what}: address {ptr:#x} is not inside a live device allocation of this process")
        if k not in self.used:
            self.used[k] = len(self.used)
        return self.used[k], ptr - self.blocks[k][0]

    def ordered(self) -> List[Tuple[int, int]]:
        inv = {v: k for k, v in self.used.items()}
        return [self.blocks[inv[i]] for i in range(len(inv))]


def _digest(lib, addr: int, size: int, host: np.ndarray) -> bytes:
    h = hashlib.blake2b(digest_size=16)
    for off in range(0, size, _CHUNK):
        n = min(_CHUNK, size - off)
        if lib.fdb_copy_to_host(host.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(addr + off),
                                ctypes.c_ulonglong(n)) != 0:
            raise PlanExportError(_native.last_error())
        h.update(host[:n].tobytes())
    return h.digest()


def _randomise_inputs(plan, seed: int) -> None:
    g = torch.Generator(device="cpu").manual_seed(seed)
    for v in plan.inputs.values():
        t = v.t
        if t.is_floating_point():
            t.copy_(torch.rand(t.shape, generator=g).to(t.dtype))
        else:
            t.copy_(torch.randint(0, 2, t.shape, generator=g).to(t.dtype))


def export_plan(plan, path: str) -> Dict[str, Any]:
    """Writes ``plan`` (every step must be a native op) to ``path``; returns a summary."""
    dev = plan.device
    lib = _native.kernels()
    lib.fdb_copy_to_host.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_ulonglong]
    ops = []
    for s in plan.steps:
        if s.native is None or getattr(s.native, "create", None) is None:
            raise PlanExportError(f"step {s.name!r} has no creation record: it cannot be replayed without Python")
        ops.append(s.native)
    with torch.cuda.device(dev):
        torch.cuda.synchronize(dev)
        bufs = _Buffers(dev)
        op_recs = []
        for op in ops:
            fn, kind, desc = op.create
            raw = bytes(desc)
            relocs = []
            for off in _pointer_slots(desc):
                ptr = struct.unpack_from("<Q", raw, off)[0]
                if ptr:
                    b, o = bufs.locate(ptr, f"{op.name}.{fn}+{off}")
                    relocs.append((off, b, o))
            op_recs.append((fn, -1 if kind is None else int(kind), raw, relocs))
        tables = []
        for op in ops:
            for t in getattr(op, "pointer_tables", []):
                b, o = bufs.locate(t.data_ptr(), f"{op.name} pointer table")
                elems = []
                for ptr in t.cpu().tolist():
                    elems.append(bufs.locate(int(ptr), f"{op.name} pointer table element") if ptr else (-1, 0))
                tables.append((b, o, elems))
        io = []
        for is_out, group in ((0, plan.inputs), (1, plan.outputs)):
            for name, v in group.items():
                t = v.t
                b, o = bufs.locate(t.data_ptr(), f"plan {'output' if is_out else 'input'} {name}")
                io.append((is_out, name, b, o, dtype_code(t.dtype), list(t.shape), list(t.stride())))
        # which buffers are constants: the bytes that two runs on different inputs leave alone
        blocks = bufs.ordered()
        host = np.empty(min(_CHUNK, max(sz for _, sz in blocks)), np.uint8)
        digests = []
        for seed in (1, 2):
            _randomise_inputs(plan, seed)
            plan.run()
            torch.cuda.synchronize(dev)
            digests.append([_digest(lib, a, sz, host) for a, sz in blocks])
        constant = [x == y for x, y in zip(*digests)]
        table_bufs = {b for b, _, _ in tables}
        with open(path, "wb") as f:
            f.write(MAGIC)
            f.write(struct.pack("<I", len(blocks)))
            saved = 0
            for k, (addr, size) in enumerate(blocks):
                keep = constant[k] and k not in table_bufs
                f.write(struct.pack("<QB", size, 1 if keep else 0))
                if keep:
                    for off in range(0, size, _CHUNK):
                        n = min(_CHUNK, size - off)
                        lib.fdb_copy_to_host(host.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(addr + off),
                                             ctypes.c_ulonglong(n))
                        f.write(host[:n].tobytes())
                    saved += size
            f.write(struct.pack("<I", len(op_recs)))
            for fn, kind, raw, relocs in op_recs:
                name = fn.encode()
                f.write(struct.pack("<H", len(name)) + name)
                f.write(struct.pack("<iI", kind, len(raw)) + raw)
                f.write(struct.pack("<I", len(relocs)))
                for off, b, o in relocs:
                    f.write(struct.pack("<IIQ", off, b, o))
            f.write(struct.pack("<I", len(tables)))
            for b, o, elems in tables:
                f.write(struct.pack("<IQI", b, o, len(elems)))
                for eb, eo in elems:
                    f.write(struct.pack("<iQ", eb, eo))
            f.write(struct.pack("<I", len(io)))
            for is_out, name, b, o, dt, dims, strides in io:
                nm = name.encode()
                f.write(struct.pack("<BH", is_out, len(nm)) + nm)
                f.write(struct.pack("<IQBB", b, o, dt, len(dims)))
                f.write(struct.pack(f"<{len(dims)}q", *dims) + struct.pack(f"<{len(dims)}q", *strides))
    return {"ops": len(op_recs), "buffers": len(blocks), "buffer_bytes": int(sum(sz for _, sz in blocks)),
            "constant_bytes": int(saved), "pointer_tables": len(tables),
            "inputs": [r[1] for r in io if not r[0]], "outputs": [r[1] for r in io if r[0]]}
