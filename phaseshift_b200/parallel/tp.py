"""Tensor parallelism over one node: process group plumbing, symmetric (peer-mapped) buffers and the
row-parallel combine.

One process per GPU (torchrun); every rank runs the same step on the same batch, weights are sliced
Megatron-style (models/qwen35/weights.py) and the only collective is the sum of a ``[rows, hidden]``
activation after each row-parallel projection (out_proj / o_proj / down_proj): two per layer, the
same communication shape as the reference (docs/developer/tensor_parallel_execution.md:137-156) but
for ``tp_size`` in {1, 2, 4, 8} and without its per-collective host rendezvous.

Two transports implement the combine:

* ``fused`` (decode / verify, rows <= 8): the projection kernel itself pushes its fp32 partials into
  every peer's receive buffer over NVLink, signals per-CTA flags and adds the partials in rank order
  (``TpCombine`` in csrc/kernels/gemv_core.cuh).  No separate collective launch exists.
* ``nccl`` (baseline, and prefill-sized activations): ``all_reduce`` on the partial projection, then a
  residual-add kernel.  Also the path used on CPU (gloo) by the host-logic tests.

Transport selection mirrors ``create_tp_transport`` + ``verify()`` in the reference
(src/phaseshift/runtime/tp/tp_transports.cpp:81-110, hip_peer_tp_transport.hip:200-312): the fused
transport is used only after a self-test round against the NCCL sum passes on every rank; otherwise
the engine falls back to NCCL loudly.
"""
from __future__ import annotations

import ctypes
import os
import sys
from typing import Dict, Optional

import torch
import torch.distributed as dist

MAX_RANKS = 8
MAX_ROWS = 8
GRID_MAX = 256


class TpCombineStruct(ctypes.Structure):
    _fields_ = [("size", ctypes.c_int), ("rank", ctypes.c_int),
                ("recv", ctypes.c_void_p * MAX_RANKS), ("flags", ctypes.c_void_p * MAX_RANKS),
                ("counter", ctypes.c_void_p), ("max_rows", ctypes.c_int), ("n_pad", ctypes.c_int)]


class TensorParallel:
    def __init__(self, group, device, transport: str = "auto"):
        self.group = group
        self.device = torch.device(device)
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.transport = "nccl"
        self.combines: Dict[int, TpCombineStruct] = {}
        self._keep = []
        self.stats = {"fused": 0, "nccl": 0}
        want = os.environ.get("PS_TP_TRANSPORT", transport)
        if self.size > 1 and self.device.type == "cuda" and want in ("auto", "fused"):
            try:
                self._symm = __import__("torch.distributed._symmetric_memory", fromlist=["x"])
                self.transport = "fused"
            except Exception as e:  # pragma: no cover
                print(f"[tp] symmetric memory unavailable ({e}); using NCCL transport", file=sys.stderr)
        if self.size > MAX_RANKS:
            raise ValueError(f"tp_size {self.size} > {MAX_RANKS}")

    # ------------------------------------------------------------------ symmetric buffers
    def _symm_alloc(self, nbytes: int):
        sm = self._symm
        t = sm.empty(nbytes, dtype=torch.uint8, device=self.device)
        t.zero_()
        hdl = sm.rendezvous(t, self.group.group_name)
        self._keep.append((t, hdl))
        return t, [int(p) for p in hdl.buffer_ptrs]

    def combine_for(self, n: int) -> Optional[TpCombineStruct]:
        """Fused-combine descriptor for projections with `n` output features (allocated on first use;
        collective: every rank must ask for the same `n` in the same order)."""
        if self.transport != "fused":
            return None
        c = self.combines.get(n)
        if c is None:
            n_pad = -(-n // 4) * 4
            recv_bytes = 2 * self.size * MAX_ROWS * n_pad * 4
            _, recv_ptrs = self._symm_alloc(recv_bytes)
            _, flag_ptrs = self._symm_alloc(GRID_MAX * self.size * 4)
            counter = torch.zeros(GRID_MAX, dtype=torch.int32, device=self.device)
            self._keep.append(counter)
            c = TpCombineStruct()
            c.size, c.rank, c.max_rows, c.n_pad = self.size, self.rank, MAX_ROWS, n_pad
            for r in range(self.size):
                c.recv[r] = recv_ptrs[r]
                c.flags[r] = flag_ptrs[r]
            c.counter = counter.data_ptr()
            torch.cuda.synchronize()
            dist.barrier(self.group)
            self.combines[n] = c
        return c

    # ------------------------------------------------------------------ baseline combine
    def all_reduce_residual(self, partial: torch.Tensor, residual: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out = sum_over_ranks(partial) + residual with the library collective (baseline / large rows)."""
        self.stats["nccl"] += 1
        if self.size > 1:
            dist.all_reduce(partial, group=self.group)
        torch.add(partial, residual, out=out)
        return out

    def disable_fused(self, why: str) -> None:
        if self.transport == "fused":
            print(f"[tp] rank {self.rank}: fused transport disabled: {why}; falling back to NCCL", file=sys.stderr)
        self.transport = "nccl"
