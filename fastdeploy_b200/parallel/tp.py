"""Tensor-parallel linear layers built on the fused GEMM + collective kernels.

* :class:`ColumnParallelLinear` — *all-gather -> GEMM*: activations are row-sharded across the ranks'
  heaps; the GEMM's TMA producer reads every 128-row tile straight from the heap of the rank that
  owns it (NVLink for remote tiles, HBM for local ones), so there is no gathered copy of A and the
  transfer overlaps the tensor-core work tile by tile. Output: all M rows x this rank's N / world
  columns.
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
                 name: str = "col_linear"):
        self.comm, self.name = comm, name
        self.rows = shard_rows(m_total, comm.world)
        n_local = w_shard.shape[0]
        assert w_shard.shape[1] == k and k % 8 == 0
        self.x_block = comm.alloc(name + ".x", self.rows * k * 2)
        self.x = comm.tensor(self.x_block, (self.rows, k), dtype)
        self.w = pack_linear_weight(w_shard.to(comm.device), dtype)
        self.y = torch.empty(m_total, _round8(n_local), dtype=dtype, device=comm.device)
        self.bias = bias.float().contiguous().to(comm.device) if bias is not None else None
        ptrs = [comm.ptr(r, self.x_block) for r in range(comm.world)]
        self.op = ConvGemm(self.x, self.w, self.y, in_shape=(1, 1, m_total, k), out_hw=(1, m_total), cout=n_local,
                           bias=self.bias, act=act, x_ld=k, y_ld=self.y.stride(0), status=comm.status,
                           name=name, peer_mode=1, peer_rows=self.rows, peer_rank=comm.rank, peer_world=comm.world,
                           peer_ptrs=ptrs)
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
                 bias: Optional[torch.Tensor] = None, dtype: torch.dtype = torch.bfloat16, name: str = "row_linear"):
        self.comm, self.name = comm, name
        self.rows = shard_rows(m_total, comm.world)
        assert w_shard.shape == (n, k_local) and k_local % 8 == 0 and n % 8 == 0
        self.n, self.m_total, self.dtype = n, m_total, dtype
        self.slots_block = comm.alloc(name + ".slots", comm.world * self.rows * n * 2)
        self.blocks = (self.rows + 127) // 128
        self.cnt_block = comm.alloc(name + ".cnt", max(self.blocks * 4, 16))
        self.slots = comm.tensor(self.slots_block, (comm.world, self.rows, n), dtype)
        self.counters = comm.tensor(self.cnt_block, (self.blocks,), torch.int32)
        self.x = torch.empty(m_total, k_local, dtype=dtype, device=comm.device)
        self.w = pack_linear_weight(w_shard.to(comm.device), dtype)
        self.y = torch.empty(self.rows, n, dtype=dtype, device=comm.device)
        self.bias = bias.float().contiguous().to(comm.device) if bias is not None else None
        slot_ptrs = [comm.ptr(r, self.slots_block) for r in range(comm.world)]
        cnt_ptrs = [comm.ptr(r, self.cnt_block) for r in range(comm.world)]
        # the slot buffer doubles as the op's nominal output (it fixes dtype, alignment and row pitch)
        self.op = ConvGemm(self.x, self.w, self.slots.view(comm.world * self.rows, n), in_shape=(1, 1, m_total, k_local),
                           out_hw=(1, m_total), cout=n, x_ld=k_local, y_ld=n, status=comm.status, name=name,
                           peer_mode=2, peer_rows=self.rows, peer_rank=comm.rank, peer_world=comm.world,
                           peer_ptrs=slot_ptrs, peer_counters=cnt_ptrs)
        info = self.op.info()
        n_tiles = (n + info["block_n"] - 1) // info["block_n"]
        blks_per_tile = [(min(n, (t + 1) * info["block_n"]) - t * info["block_n"] + 63) // 64 for t in range(n_tiles)]
        self.stores_per_block = sum(blks_per_tile)      # TMA stores one source rank makes per 128-row block
        self.calls = 0

    def input_tensor(self) -> torch.Tensor:
        return self.x

    def forward(self) -> torch.Tensor:
        self.calls += 1
        self.op.launch()
        target = self.calls * self.comm.world * self.stores_per_block
        rc = _lib().fdb_comm_slot_reduce(
            ctypes.c_void_p(self.slots.data_ptr()), ctypes.c_void_p(self.counters.data_ptr()), target,
            ctypes.c_void_p(self.y.data_ptr()), ctypes.c_void_p(self.bias.data_ptr()) if self.bias is not None else None,
            self.rows, self.n, self.n, self.n, self.comm.world, dtype_code(self.dtype), self.comm.status.ptr,
            ctypes.c_void_p(current_stream_ptr()))
        if rc != 0:
            raise RuntimeError(self.name + ": " + _native.last_error())
        # the next call's stores must not land before every rank has read this call's slots
        self.comm.barrier()
        return self.y
