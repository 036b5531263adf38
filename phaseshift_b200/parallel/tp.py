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
* prefill-sized activations (rows > 8) under the fused transport: the stand-alone peer-memory
  all-reduce kernel (csrc/kernels/allreduce.cu; peer one-shot by default, ``PS_TP_MULTIMEM=1`` selects
  the NVSwitch ``multimem`` two-shot) with the residual add fused.
* ``nccl`` (baseline): ``all_reduce`` on the partial projection, then a residual-add kernel.  Also the
  path used on CPU (gloo) by the host-logic tests.

Transport selection mirrors ``create_tp_transport`` + ``verify()`` in the reference
(src/phaseshift/runtime/tp/tp_transports.cpp:81-110, hip_peer_tp_transport.hip:200-312): the engine runs
``TensorParallel.verify`` at construction -- a self-test round against the NCCL sum on every rank -- and falls back
to NCCL loudly if any rank fails it.
"""
from __future__ import annotations

import ctypes
import os
import sys
from typing import Dict, Optional

import torch
import torch.distributed as dist

MAX_RANKS = 8
MAX_ROWS = 32          # rows the fused combine's receive buffers are sized for
GRID_MAX = 256


class TpCombineStruct(ctypes.Structure):
    _fields_ = [("size", ctypes.c_int), ("rank", ctypes.c_int),
                ("recv", ctypes.c_void_p * MAX_RANKS), ("flags", ctypes.c_void_p * MAX_RANKS),
                ("counter", ctypes.c_void_p), ("max_rows", ctypes.c_int), ("n_pad", ctypes.c_int)]


class ArStruct(ctypes.Structure):
    """Host twin of ps::ArArgs (csrc/kernels/allreduce.cu)."""
    _fields_ = [("size", ctypes.c_int), ("rank", ctypes.c_int),
                ("inp", ctypes.c_void_p * MAX_RANKS), ("mc_in", ctypes.c_void_p), ("mc_res", ctypes.c_void_p),
                ("res_local", ctypes.c_void_p), ("flags", ctypes.c_void_p * MAX_RANKS), ("counter", ctypes.c_void_p),
                ("residual", ctypes.c_void_p), ("ld_res", ctypes.c_int), ("out", ctypes.c_void_p), ("ldo", ctypes.c_int),
                ("rows", ctypes.c_int), ("n", ctypes.c_int), ("status", ctypes.c_void_p)]


class TpScatterStruct(ctypes.Structure):
    """Host twin of ps::TpScatter (csrc/kernels/gemm_bs.cu)."""
    _fields_ = [("size", ctypes.c_int), ("rank", ctypes.c_int), ("rpr", ctypes.c_int), ("ld", ctypes.c_int),
                ("recv", ctypes.c_void_p * MAX_RANKS)]


class RgStruct(ctypes.Structure):
    """Host twin of ps::RgArgs (csrc/kernels/allreduce.cu)."""
    _fields_ = [("size", ctypes.c_int), ("rank", ctypes.c_int), ("rows", ctypes.c_int), ("n", ctypes.c_int), ("rpr", ctypes.c_int),
                ("src", ctypes.c_void_p * MAX_RANKS), ("src_row0", ctypes.c_int), ("ld", ctypes.c_int),
                ("partial", ctypes.c_void_p), ("ld_partial", ctypes.c_int), ("recv", ctypes.c_void_p * MAX_RANKS),
                ("flags", ctypes.c_void_p * MAX_RANKS), ("counter", ctypes.c_void_p),
                ("residual", ctypes.c_void_p), ("ld_res", ctypes.c_int),
                ("out", ctypes.c_void_p * MAX_RANKS), ("ldo", ctypes.c_int), ("status", ctypes.c_void_p)]


AR_GRID = 128
RG_GRID = 296


class TensorParallel:
    def __init__(self, group, device, transport: str = "auto"):
        self.group = group
        self.device = torch.device(device)
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.transport = "nccl"
        self.combines: Dict[int, TpCombineStruct] = {}
        self._keep = []
        self.stats = {"fused": 0, "nccl": 0, "peer_allreduce": 0}
        self._ar = None                      # stand-alone all-reduce state (symmetric buffers), built on first use
        self.use_multimem = os.environ.get("PS_TP_MULTIMEM", "0") == "1"
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
        self._last_hdl = hdl
        return t, [int(p) for p in hdl.buffer_ptrs]

    # ------------------------------------------------------------------ stand-alone all-reduce (rows > 8)
    def _ar_state(self, nbytes: int):
        """Symmetric input (two parities) / result buffers and flags for the all-reduce kernel; grown
        collectively (every rank sees the same sequence of sizes)."""
        st = self._ar
        if st is not None and st["cap"] >= nbytes:
            return st
        cap = max(nbytes, 1 << 20)
        cap = 1 << (cap - 1).bit_length()
        inp, in_ptrs = self._symm_alloc(2 * cap)
        mc_in = int(getattr(self._last_hdl, "multicast_ptr", 0) or 0)
        res, res_ptrs = self._symm_alloc(cap)
        mc_res = int(getattr(self._last_hdl, "multicast_ptr", 0) or 0)
        _, flag_ptrs = self._symm_alloc(2 * AR_GRID * self.size * 4)
        counter = torch.zeros(AR_GRID, dtype=torch.int32, device=self.device)
        status = torch.zeros(1, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize()
        dist.barrier(self.group)
        self._ar = dict(cap=cap, inp=inp, in_ptrs=in_ptrs, mc_in=mc_in, res=res, res_ptrs=res_ptrs, mc_res=mc_res,
                        flag_ptrs=flag_ptrs, counter=counter, status=status, parity=0)
        return self._ar

    def peer_all_reduce(self, partial: torch.Tensor, residual: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
        """out = sum over ranks of `partial` (+ residual) with the one-shot peer / multimem kernels (benchmarks and
        tests; the engine's collectives are `combine_for`, `scatter_for` + `reduce_gather`).  The input double buffer
        is selected by a parity kept on the HOST, so calls must not be captured into a CUDA graph."""
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("peer_all_reduce keeps its buffer parity on the host and cannot be graph-captured")
        from ..ops import _lib
        rows, n = partial.shape
        nbytes = rows * n * 2
        st = self._ar_state(nbytes)
        par = st["parity"]
        st["inp"][par * st["cap"]: par * st["cap"] + nbytes].view(torch.bfloat16).copy_(partial.reshape(-1))
        a = ArStruct()
        a.size, a.rank, a.rows, a.n = self.size, self.rank, rows, n
        for r in range(self.size):
            a.inp[r] = st["in_ptrs"][r] + par * st["cap"]
            a.flags[r] = st["flag_ptrs"][r]
        multimem = self.use_multimem and st["mc_in"] != 0 and st["mc_res"] != 0
        a.mc_in = (st["mc_in"] + par * st["cap"]) if multimem else None
        a.mc_res = st["mc_res"] if multimem else None
        a.res_local = st["res"].data_ptr()
        a.counter = st["counter"].data_ptr()
        a.residual = residual.data_ptr() if residual is not None else None
        a.ld_res = residual.stride(0) if residual is not None else 0
        a.out, a.ldo = out.data_ptr(), out.stride(0)
        # bounded-wait failures go to the engine's status word when one is attached (Engine sets `status_word`),
        # so a timed-out all-reduce poisons the step like any other device failure
        word = getattr(self, "status_word", None)
        a.status = (word if word is not None else st["status"]).data_ptr()
        _lib.call("ps_allreduce", ctypes.byref(a), ctypes.c_int(1 if multimem else 0), ctypes.c_int(AR_GRID))
        st["parity"] ^= 1
        self.stats["peer_allreduce"] += 1
        return out

    # ------------------------------------------------------------------ fused projection -> reduce-scatter -> all-gather
    def _rs_state(self, rows: int, n: int):
        """Symmetric receive buffer ([source][rows per rank][n] bf16), barrier flags and the per-name output buffers of
        the scatter path; grown collectively (every rank sees the same sequence of shapes)."""
        st = getattr(self, "_rs", None)
        need = (rows + self.size) * n * 2
        if st is None or st["cap"] < need or st["n"] != n:
            cap = 1 << (max(need, 1 << 20) - 1).bit_length()
            recv, recv_ptrs = self._symm_alloc(cap)
            _, flag_ptrs = self._symm_alloc(2 * RG_GRID * self.size * 4)
            counter = torch.zeros(RG_GRID, dtype=torch.int32, device=self.device)
            torch.cuda.synchronize()
            dist.barrier(self.group)
            st = dict(cap=cap, n=n, recv=recv, recv_ptrs=recv_ptrs, flag_ptrs=flag_ptrs, counter=counter, outs={})
            self._rs = st
        return st

    def _rs_out(self, st, name: str, rows: int, n: int):
        """Output buffer `name` in symmetric memory (peers store finished rows into it)."""
        o = st["outs"].get(name)
        if o is None or o[0].shape[0] < rows or o[0].shape[1] != n:
            cap_rows = 1 << (max(rows, 64) - 1).bit_length()
            t, ptrs = self._symm_alloc(cap_rows * n * 2)
            torch.cuda.synchronize()
            dist.barrier(self.group)
            o = (t.view(torch.bfloat16).view(cap_rows, n), ptrs)
            st["outs"][name] = o
        return o

    def scatter_for(self, rows: int, n: int) -> TpScatterStruct:
        """Descriptor that makes the block-scaled projection kernel push its bf16 output rows to their owner ranks."""
        st = self._rs_state(rows, n)
        c = TpScatterStruct()
        c.size, c.rank, c.rpr, c.ld = self.size, self.rank, -(-rows // self.size), n
        for r in range(self.size):
            c.recv[r] = st["recv_ptrs"][r]
        return c

    def reduce_gather(self, rows: int, n: int, residual: Optional[torch.Tensor], name: str,
                      partial: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum of the ranks' partials of this rank's rows + residual, finished rows stored to every rank.  Returns this
        rank's (complete) output [rows, n].  The partials were pushed into the receive buffers by the projection kernel
        (``scatter_for``), or -- ``partial`` given: this rank's whole partial product [rows, n] bf16, any local
        memory -- are dealt to their owners by the same kernel first (a two-shot all-reduce with remote stores only)."""
        from ..ops import _lib
        st = self._rs_state(rows, n)
        out, out_ptrs = self._rs_out(st, name, rows, n)
        a = RgStruct()
        a.size, a.rank, a.rows, a.n, a.rpr = self.size, self.rank, rows, n, -(-rows // self.size)
        a.ld = n
        a.src_row0 = a.rank * a.rpr
        for r in range(self.size):
            a.src[r] = st["recv"].data_ptr() + r * a.rpr * n * 2
            a.recv[r] = st["recv_ptrs"][r]
        if partial is not None:
            assert partial.dtype == torch.bfloat16 and partial.stride(1) == 1 and partial.stride(0) % 8 == 0
            a.partial, a.ld_partial = partial.data_ptr(), partial.stride(0)
        else:
            a.partial, a.ld_partial = None, 0
        for r in range(self.size):
            a.flags[r] = st["flag_ptrs"][r]
            a.out[r] = out_ptrs[r]
        a.counter = st["counter"].data_ptr()
        a.residual = residual.data_ptr() if residual is not None else None
        a.ld_res = residual.stride(0) if residual is not None else 0
        a.ldo = n
        word = getattr(self, "status_word", None)
        if word is None:
            word = st.setdefault("status", torch.zeros(1, dtype=torch.int32, device=self.device))
        a.status = word.data_ptr()
        _lib.call("ps_tp_reduce_gather", ctypes.byref(a), ctypes.c_int(RG_GRID))
        key = "two_shot" if partial is not None else "scatter"
        self.stats[key] = self.stats.get(key, 0) + 1
        return out[:rows]

    def max_fused_rows(self, W) -> int:
        """Rows up to which a row-parallel projection over `W` combines inside its own kernel: 16 on the block-scaled
        tensor-core path (its one-shot push of fp32 partials to every rank stops paying beyond that; the receive
        buffers hold 32 rows), 8 on the streaming kernel."""
        return 16 if getattr(W, "sf_atoms", None) is not None else 8

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
        if (self.transport == "fused" and self.size > 1 and partial.dtype == torch.bfloat16 and partial.stride(1) == 1
                and partial.shape[1] % 8 == 0 and partial.stride(0) % 8 == 0 and out.dtype == torch.bfloat16):
            # two-shot kernel with device-side collective counters (safe inside captured graphs, unlike
            # `peer_all_reduce`, whose input parity is tracked on the host)
            out.copy_(self.reduce_gather(partial.shape[0], partial.shape[1], residual, "__ar_out__", partial=partial))
            return out
        self.stats["nccl"] += 1
        if self.size > 1:
            dist.all_reduce(partial, group=self.group)
        torch.add(partial, residual, out=out)
        return out

    # ------------------------------------------------------------------ liveness
    def start_monitor(self, store=None, interval_s: float = 0.2, timeout_s: float = 2.0):
        """Start the host-side heartbeat (parallel/health.py); `assert_alive()` is then cheap to call between
        steps and raises RankLostError before a launch that would wait for a dead peer."""
        from .health import PeerMonitor
        if store is None:
            from torch.distributed.distributed_c10d import _get_default_store
            store = _get_default_store()
        self.monitor = PeerMonitor(store, self.rank, self.size, interval_s, timeout_s).start()
        return self.monitor

    def assert_alive(self) -> None:
        m = getattr(self, "monitor", None)
        if m is not None:
            m.assert_alive()

    # ------------------------------------------------------------------ transport self-test
    def verify(self, ops=None) -> bool:
        """Self-test of the peer-memory transport against the library collective, run once by every rank at engine
        construction (the reference's transport does the same before it is used,
        src/phaseshift/runtime/tp/hip_peer_tp_transport.hip:200-312): the two-shot reduce/gather kernel on two payload
        sizes and -- when an op set is given -- one projection with the in-kernel combine.  Any rank that sees a wrong
        sum, a disagreement with its peers or a device wait that ran out makes EVERY rank fall back to the library
        transport (the verdict is itself all-reduced).  Also performs, collectively and up front, the symmetric-memory
        allocations the first real steps would otherwise do lazily."""
        if self.transport != "fused" or self.size <= 1:
            return True
        dev = self.device
        ok = True
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        saved = getattr(self, "status_word", None)
        self.status_word = status
        try:
            g = torch.Generator(device=dev).manual_seed(4321 + self.rank)
            shared = torch.Generator(device=dev).manual_seed(99)
            for rows, n in ((3, 256), (200, 512)):
                part = (torch.randn(rows, n, device=dev, generator=g) * 0.5).to(torch.bfloat16)
                res = torch.randn(rows, n, device=dev, generator=shared).to(torch.bfloat16)
                got = self.reduce_gather(rows, n, res, "__verify__", partial=part).clone()
                ref = part.float()
                dist.all_reduce(ref, group=self.group)
                ref = ref.to(torch.bfloat16).float() + res.float()
                ok = ok and bool(((got.float() - ref).abs().max() <= 0.06).item())
                low = got.float().clone()
                high = got.float().clone()
                dist.all_reduce(low, op=dist.ReduceOp.MIN, group=self.group)
                dist.all_reduce(high, op=dist.ReduceOp.MAX, group=self.group)
                ok = ok and bool(torch.equal(low, high))              # every rank holds the same bits
            if ops is not None and hasattr(ops, "linear_bs"):
                from ..models.qwen35.weights import LinearW
                from ..quant.formats import quantize, to_kernel_format
                W = LinearW(to_kernel_format(quantize(torch.randn(256, 128, device=dev, generator=g) * 0.05, "bf16")))
                x = torch.randn(2, 128, device=dev, generator=g).to(torch.bfloat16)
                res = torch.randn(2, 256, device=dev, generator=shared).to(torch.bfloat16)
                got = ops.linear(x, W, name="__verify_lin__", residual=res, tp_combine=self.combine_for(256)).float().clone()
                ref = x.float() @ W.dense().to(dev).T
                dist.all_reduce(ref, group=self.group)
                ok = ok and bool(((got - (ref + res.float())).abs().max() <= 0.06).item())
            torch.cuda.synchronize(dev)
            ok = ok and int(status[0]) == 0
            if ops is not None and getattr(ops, "status", None) is not None:
                ok = ok and int(ops.status[0]) == 0
        except Exception as e:      # pragma: no cover - a broken transport must not take the engine down
            print(f"[tp] rank {self.rank}: transport self-test raised {e!r}", file=sys.stderr)
            ok = False
        finally:
            self.status_word = saved
        verdict = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN, group=self.group)
        self.verified = bool(verdict.item())
        if not self.verified:
            self.disable_fused("transport self-test failed on at least one rank")
        return self.verified

    def disable_fused(self, why: str) -> None:
        if self.transport == "fused":
            print(f"[tp] rank {self.rank}: fused transport disabled: {why}; falling back to NCCL", file=sys.stderr)
        self.transport = "nccl"
