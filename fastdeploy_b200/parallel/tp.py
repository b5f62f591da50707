"""Tensor-parallel linear layers built on the fused GEMM + collective kernels.

* :class:`ColumnParallelLinear` — *all-gather -> GEMM* in one kernel: activations are row-sharded
  across the ranks' heaps. A few CTAs of the GEMM grid act as copiers: they pull the remote shards
  over NVLink into this rank's gathered buffer, 128 rows at a time, and publish a flag per block;
  the other CTAs run the tcgen05 GEMM, local rows first, and their TMA producers wait (bounded) for
  the flag of a row block before reading it. Every remote row crosses NVLink once and the transfer
  overlaps the tensor-core work. Output: all M rows x this rank's N / world columns.
* :class:`RowParallelLinear` — *GEMM -> reduce-scatter*: every rank multiplies its K / world slice;
  the epilogue TMA-stores each 128-row block into the heap of the rank that owns those rows and bumps
  that rank's counter; a slot-reduction kernel on the owner waits per block (bounded) and sums the
  world partial blocks. Output: this rank's M / world rows x all N columns.

Both are compared in the tests and in ``bench_tp`` against the unfused baseline (NCCL collective +
local GEMM). The reference has no tensor parallelism.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native
from ..ops.base import current_stream_ptr, dtype_code
from ..ops.conv_gemm import ConvGemm, pack_linear_weight
from .comm import Communicator, _lib, shard_rows


def _round8(n: int) -> int:
    return (n + 7) // 8 * 8


class ColumnParallelLinear:
    """``y[:, cols of this rank] = act(gather(x) @ w_shard.T + b_shard)``.

    ``x_block`` is the heap block every rank writes its ``[rows_per_rank, K]`` activations into
    (see :meth:`input_tensor`).
    """

    def __init__(self, comm: Communicator, m_total: int, k: int, w_shard: torch.Tensor,
                 bias: Optional[torch.Tensor] = None, act: Optional[str] = None, dtype: torch.dtype = torch.bfloat16,
                 name: str = "col_linear", copiers: int = 0):
        self.comm, self.name = comm, name
        self.rows = shard_rows(m_total, comm.world)
        n_local = w_shard.shape[0]
        assert w_shard.shape[1] == k and k % 8 == 0
        # Gathered buffer [M, K] at the same heap offset on every rank; rank r writes its shard at rows
        # r * rows of its own buffer, the copier CTAs of the GEMM fill in the rest from the peers.
        self.x_block = comm.alloc(name + ".x", m_total * k * 2)
        self.gathered = comm.tensor(self.x_block, (m_total, k), dtype)
        self.x = self.gathered[comm.rank * self.rows:(comm.rank + 1) * self.rows]
        self.ready = torch.zeros(m_total // 128, dtype=torch.int32, device=comm.device)
        self.w = pack_linear_weight(w_shard.to(comm.device), dtype)
        self.y = torch.empty(m_total, _round8(n_local), dtype=dtype, device=comm.device)
        self.bias = bias.float().contiguous().to(comm.device) if bias is not None else None
        ptrs = [comm.ptr(r, self.x_block) for r in range(comm.world)]
        self.op = ConvGemm(self.gathered, self.w, self.y, in_shape=(1, 1, m_total, k), out_hw=(1, m_total),
                           cout=n_local, bias=self.bias, act=act, x_ld=k, y_ld=self.y.stride(0), status=comm.status,
                           name=name, peer_mode=1, peer_rows=self.rows, peer_rank=comm.rank, peer_world=comm.world,
                           peer_ptrs=ptrs, peer_ready=self.ready, peer_copiers=copiers)
        self.n_local = n_local

    def input_tensor(self) -> torch.Tensor:
        return self.x

    def forward(self) -> torch.Tensor:
        """Call after every rank has written its ``input_tensor()``; the leading barrier makes the
        peers' writes visible and ordered, the trailing one keeps them from overwriting rows that a
        slower rank is still reading."""
        self.comm.barrier()
        self.op.launch()
        self.comm.barrier()
        return self.y[:, :self.n_local]


class RowParallelLinear:
    """``y[rows of this rank] = sum_r x_r @ w_r.T (+ b)`` where ``x_r [M, K / world]``."""

    def __init__(self, comm: Communicator, m_total: int, k_local: int, n: int, w_shard: torch.Tensor,
                 bias: Optional[torch.Tensor] = None, dtype: torch.dtype = torch.bfloat16, name: str = "row_linear",
                 x: Optional[torch.Tensor] = None):
        self.comm, self.name = comm, name
        self.rows = shard_rows(m_total, comm.world)
        assert w_shard.shape == (n, k_local) and k_local % 8 == 0 and n % 8 == 0
        self.n, self.m_total, self.dtype = n, m_total, dtype
        # Two slot buffers and counter sets, used by even and odd calls. A rank can only reach call
        # i + 2 after its call i + 1 reduction saw every rank's call i + 1 stores, and those follow
        # (in stream order) that rank's call i reduction: so nobody overwrites slots that are still
        # being read, and no barrier is needed between calls.
        slot_bytes = comm.world * self.rows * n * 2
        self.blocks = (self.rows + 127) // 128
        cnt_bytes = (self.blocks * 4 + 1023) // 1024 * 1024
        self.slots_block = comm.alloc(name + ".slots", 2 * slot_bytes)
        self.cnt_block = comm.alloc(name + ".cnt", 2 * cnt_bytes)
        self.x = x if x is not None else torch.empty(m_total, k_local, dtype=dtype, device=comm.device)
        assert self.x.shape == (m_total, k_local) and self.x.stride(1) == 1
        self.w = pack_linear_weight(w_shard.to(comm.device), dtype)
        self.y = torch.empty(self.rows, n, dtype=dtype, device=comm.device)
        self.bias = bias.float().contiguous().to(comm.device) if bias is not None else None
        self.slots, self.counters, self.ops = [], [], []
        for par in range(2):
            slots = comm.tensor(self.slots_block, (comm.world, self.rows, n), dtype, byte_offset=par * slot_bytes)
            cnt = comm.tensor(self.cnt_block, (self.blocks,), torch.int32, byte_offset=par * cnt_bytes)
            slot_ptrs = [comm.ptr(r, self.slots_block, par * slot_bytes) for r in range(comm.world)]
            cnt_ptrs = [comm.ptr(r, self.cnt_block, par * cnt_bytes) for r in range(comm.world)]
            # the slot buffer doubles as the op's nominal output (it fixes dtype, alignment and row pitch)
            op = ConvGemm(self.x, self.w, slots.view(comm.world * self.rows, n), in_shape=(1, 1, m_total, k_local),
                          out_hw=(1, m_total), cout=n, x_ld=self.x.stride(0), y_ld=n, status=comm.status, name=name,
                          peer_mode=2, peer_rows=self.rows, peer_rank=comm.rank, peer_world=comm.world,
                          peer_ptrs=slot_ptrs, peer_counters=cnt_ptrs)
            self.slots.append(slots)
            self.counters.append(cnt)
            self.ops.append(op)
        self.op = self.ops[0]
        info = self.op.info()
        n_tiles = (n + info["block_n"] - 1) // info["block_n"]
        blks_per_tile = [(min(n, (t + 1) * info["block_n"]) - t * info["block_n"] + 31) // 32 for t in range(n_tiles)]
        self.stores_per_block = sum(blks_per_tile)      # TMA stores one source rank makes per 128-row block
        self.calls = 0

    def input_tensor(self) -> torch.Tensor:
        return self.x

    def forward(self) -> torch.Tensor:
        par = self.calls & 1
        self.calls += 1
        self.ops[par].launch()
        target = ((self.calls + 1) // 2) * self.comm.world * self.stores_per_block
        rc = _lib().fdb_comm_slot_reduce(
            ctypes.c_void_p(self.slots[par].data_ptr()), ctypes.c_void_p(self.counters[par].data_ptr()), target,
            ctypes.c_void_p(self.y.data_ptr()), ctypes.c_void_p(self.bias.data_ptr()) if self.bias is not None else None,
            self.rows, self.n, self.n, self.n, self.comm.world, dtype_code(self.dtype), self.comm.status.ptr,
            ctypes.c_void_p(current_stream_ptr()))
        if rc != 0:
            raise RuntimeError(self.name + ": " + _native.last_error())
        return self.y


class TensorParallelMLP:
    """Transformer feed-forward block over ``world`` ranks: rows of the activations are sharded,
    ``fc1`` is column-parallel behind a fused all-gather, ``fc2`` row-parallel in front of a fused
    reduce-scatter, so the block takes row shards in and gives row shards out with the GELU
    intermediate never leaving its rank.

    ``w1 [ffn, hidden]``, ``w2 [hidden, ffn]`` are the full weights; each rank keeps its slice.
    """

    def __init__(self, comm: Communicator, m_total: int, hidden: int, ffn: int, w1: torch.Tensor, b1: torch.Tensor,
                 w2: torch.Tensor, b2: torch.Tensor, dtype: torch.dtype = torch.bfloat16, act: str = "gelu",
                 name: str = "tp_mlp"):
        ws, r = comm.world, comm.rank
        assert ffn % ws == 0 and (ffn // ws) % 8 == 0
        fl = ffn // ws
        self.fc1 = ColumnParallelLinear(comm, m_total, hidden, w1[r * fl:(r + 1) * fl], b1[r * fl:(r + 1) * fl], act=act,
                                        dtype=dtype, name=name + ".fc1")
        self.fc2 = RowParallelLinear(comm, m_total, fl, hidden, w2[:, r * fl:(r + 1) * fl], b2, dtype=dtype,
                                     name=name + ".fc2", x=self.fc1.y[:, :fl])
        self.comm = comm

    def input_tensor(self) -> torch.Tensor:
        return self.fc1.input_tensor()

    def forward(self) -> torch.Tensor:
        self.fc1.forward()
        return self.fc2.forward()
