"""CUDA op set: thin Python wrappers over the sm_100a kernels in ``libps_kernels.so``.

Each method validates shapes/dtypes (the role of the reference's ``resolve_*_args`` functions, e.g.
src/phaseshift/models/qwen35/runtime/paged_attention_dispatch.hip:274-436), picks the kernel variant
(small-M fused GEMV vs tensor-core GEMM -- the job of the reference's linear selector,
src/.../runtime/linear_selector.cpp:202-308) and launches on the current stream.  Output buffers come
from a per-instance workspace keyed by (name, rows) so pointers are stable across steps, which is
what lets a whole step be captured in a CUDA graph.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from .trace import OpTrace
from ..models.qwen35.config import Qwen35Config
from ..models.qwen35.weights import AttnW, GdnW, LinearW
from ..runtime.batch import StepBatch
from ..runtime.state import GdnLayerState, KVLayer, ModelState
from . import _lib
from ._lib import c_float, c_int, c_ll, ptr

WFMT = {"bf16": 0, "nvfp4": 1, "mxfp8": 2}
PRO_NONE, PRO_RMSNORM, PRO_SIGMOID_GATE = 0, 1, 2
EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2
SMALL_M_MAX = 8


class CudaOps(OpTrace):
    act_dtype = torch.bfloat16
    name = "cuda"
    GDN_CHUNKED_MIN_ROWS = 16      # steps with more rows than this use the chunked GDN kernels
    ATTN_PREFILL_MIN_ROWS = 16     # ... and the tiled tensor-core attention kernel

    def __init__(self, cfg: Qwen35Config, device, attn_split_tokens: int = 64, attn_max_splits: int = 0,
                 max_seq_len: int = 4096):
        if device.type != "cuda":
            raise ValueError("CudaOps needs a CUDA device")
        _lib.lib()      # fail loudly when the native library is missing
        self.cfg, self.device = cfg, device
        self.ws: Dict[Tuple[str, int], torch.Tensor] = {}
        self.checked = _lib.checked_build()          # PS_CHECKED=1: descriptor assertions in the kernels + workspace canaries
        self._guarded: Dict[Tuple[str, int], torch.Tensor] = {}
        half = cfg.rotary_dim // 2
        inv = cfg.rope_theta ** (-np.arange(half, dtype=np.float64) * 2.0 / cfg.rotary_dim)
        self.inv_freq = torch.from_numpy(inv).to(device)
        # the split length is fixed per engine for steps of up to 8 rows and for Exact mode, so attention results there do not
        # depend on the batch; larger Fast-mode batches lengthen it (see paged_attention).  PS_ATTN_SPLIT_TOKENS overrides the
        # base length (a multiple of 32).
        self.split_tokens = int(os.environ.get("PS_ATTN_SPLIT_TOKENS", attn_split_tokens))
        if self.split_tokens < 32 or self.split_tokens % 32:
            raise ValueError("the attention split length must be a positive multiple of 32")
        while -(-(max_seq_len + 1) // self.split_tokens) > 512:
            self.split_tokens *= 2
        self.max_splits = attn_max_splits or -(-(max_seq_len + 1) // self.split_tokens)
        self.launches = 0
        self.use_tc_gemm = True
        self.exact_rows = False     # verify steps: keep every projection on the batch-invariant small-M kernel
        self.attn_decode_tc = os.environ.get("PS_ATTN_DECODE", "tc") != "legacy"
        self.wscratch = None
        self.status = torch.zeros(1, dtype=torch.int32, device=device)   # kernels' own bounded-wait status word
        # block-scaled tensor-core projections: stream-K partials + flags (flags must read 0 between launches)
        self.bs_ws: Optional[torch.Tensor] = None
        self.bs_flags: Optional[torch.Tensor] = None
        self.bs_grid_override = 0
        self.force_tc = os.environ.get("PS_FORCE_TC", "0") == "1"   # single-row steps on the tensor-core kernel too
        self.bs_prefetch = os.environ.get("PS_BS_PREFETCH", "1") != "0"
        self._bs_plan_cache: Dict[tuple, bool] = {}
        self.sel_counts: Dict[str, int] = {"tc_resident": 0, "tc_streamed": 0, "stream": 0, "gemm": 0}   # projection calls per kernel
        self.fallbacks: Dict[str, int] = {}

    # ------------------------------------------------------------------ workspace
    CANARY = 0xA5
    CANARY_BYTES = 256

    def buf(self, name: str, rows: int, cols: int, dtype=torch.bfloat16) -> torch.Tensor:
        key = (name, rows)
        t = self.ws.get(key)
        if t is None or t.shape[1] != cols or t.dtype != dtype:
            if self.checked:
                # checked build: every workspace sits between two guard regions that `check_canaries` inspects
                n = rows * cols * torch.empty(0, dtype=dtype).element_size()
                raw = torch.full((n + 2 * self.CANARY_BYTES,), self.CANARY, dtype=torch.uint8, device=self.device)
                t = raw[self.CANARY_BYTES:self.CANARY_BYTES + n].view(dtype).view(rows, cols)
                self._guarded[key] = raw
            else:
                t = torch.empty(rows, cols, dtype=dtype, device=self.device)
            self.ws[key] = t
        return t

    def check_canaries(self):
        """Checked build: names of the workspaces whose guard bytes were overwritten (an out-of-bounds write by some
        kernel).  Synchronises; the engine calls it after every step when the checked library is loaded."""
        bad = []
        g = self.CANARY_BYTES
        for key, raw in self._guarded.items():
            if bool((raw[:g] != self.CANARY).any()) or bool((raw[-g:] != self.CANARY).any()):
                bad.append(key[0])
        return bad

    # ------------------------------------------------------------------ ops
    SSQ_LD = 64          # partial sums of squares per row: one per 128-feature tile of the producing projection

    def ssq_buf(self, name: str, rows: int) -> torch.Tensor:
        return self.buf("ssq_" + name, rows, self.SSQ_LD, torch.float32)

    def embed(self, b: StepBatch, rows: int, table: LinearW, status, ssq_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        H = table.K
        out = self.buf("x_embed", rows, H)
        ld = ssq_out.stride(0) if ssq_out is not None else 0
        if table.fmt == "bf16":
            _lib.call("ps_embedding", ptr(b.ids), ptr(table.q.codes), c_int(rows), c_int(table.N), c_int(H),
                      ptr(out), c_int(H), ptr(status), ptr(ssq_out), c_int(ld))
        elif table.fmt == "mxfp8":
            _lib.call("ps_embedding_mxfp8", ptr(b.ids), ptr(table.q.codes), ptr(table.q.scales), c_int(rows),
                      c_int(table.N), c_int(H), ptr(out), c_int(H), ptr(status), ptr(ssq_out), c_int(ld))
        else:
            raise ValueError("embedding table must be bf16 or mxfp8")
        self.launches += 1
        return out

    def linear(self, x: torch.Tensor, W: LinearW, *, name: str, norm_w: Optional[torch.Tensor] = None,
               eps: float = 0.0, residual: Optional[torch.Tensor] = None, swiglu: bool = False,
               out_f32: bool = False, out: Optional[torch.Tensor] = None,
               xn_out: Optional[torch.Tensor] = None, tp_combine=None, ssq_in=None,
               ssq_out: Optional[torch.Tensor] = None, prefetch: Optional[LinearW] = None, tp_scatter=None) -> torch.Tensor:
        """``tp_combine`` (a parallel.tp.TpCombineStruct): the projection is row-parallel and the kernel sums
        the ranks' partial results over NVLink before the residual epilogue.
        ``ssq_in`` = (tensor [rows, SSQ_LD] fp32, n): n partial sums of squares per row of ``x`` left by the kernel
        that produced it, consumed by the fused RMSNorm; ``ssq_out``: receives the partial sums of the rows this
        projection stores (block-scaled tensor-core path, <= 32 rows; ignored elsewhere).
        ``prefetch``: the projection that will run next on the same rows; the tensor-core kernel warms L2 with the first
        bytes of its weights while it drains.
        ``tp_scatter`` (a parallel.tp.TpScatterStruct; tensor-core path with streamed activations only): instead of
        storing to ``out`` the kernel pushes each bf16 output row to the receive buffer of the rank that owns it."""
        M, K = x.shape
        assert K == W.K and x.dtype == torch.bfloat16 and x.stride(1) == 1, (x.shape, W.K, x.dtype)
        n_out = W.N // 2 if swiglu else W.N
        if out is None:
            out = self.buf(name, M, n_out, torch.float32 if out_f32 else torch.bfloat16)
        assert out.shape[0] == M and out.shape[1] == n_out and out.stride(1) == 1
        if W.K % 32 and W.sf_atoms is None:
            raise ValueError(f"K={W.K} must be a multiple of 32 for the streaming / bf16 tensor-core kernels")
        sel = self.select_linear(W, M)
        if sel == "tc":
            # block-quantised codes straight into the tensor cores (any number of rows)
            return self.linear_bs(x, W, name=name, norm_w=norm_w, eps=eps, residual=residual, swiglu=swiglu,
                                  out_f32=out_f32, out=out, xn_out=xn_out, tp_combine=tp_combine, ssq_in=ssq_in,
                                  ssq_out=ssq_out, prefetch=prefetch, tp_scatter=tp_scatter)
        if tp_scatter is not None:
            raise ValueError("tp_scatter needs the block-scaled tensor-core path")
        if tp_combine is not None and M > SMALL_M_MAX:
            raise ValueError("the fused tensor-parallel combine handles at most 8 rows")
        # bf16 tensor-core GEMM: prefill-sized steps, and batched steps (>= 2 rows) of bf16 weights whose row-major form
        # is resident (Fast mode only: Exact verification stays on the batch-invariant streaming kernel)
        batched = (M >= 2 and W.rowmajor_bf16 is not None and tp_combine is None and xn_out is None and self.use_tc_gemm
                   and not self.exact_rows)
        self.sel_counts["gemm" if (sel == "gemm" or batched) else "stream"] += 1
        if sel == "gemm" or batched:
            return self.linear_large(x, W, name=name, norm_w=norm_w, eps=eps, residual=residual, swiglu=swiglu,
                                     out_f32=out_f32, out=out)
        pro = PRO_RMSNORM if norm_w is not None else PRO_NONE
        epi = EPI_SWIGLU if swiglu else (EPI_RESIDUAL if residual is not None else EPI_STORE)
        if W.tiled is None:
            W.make_tiled()
        L = _lib.lib()
        L.ps_linear_stream_max_rows.restype = ctypes.c_int
        mmax = L.ps_linear_stream_max_rows(c_int(WFMT[W.fmt]), c_int(W.k_padded))
        if mmax < 1:
            raise ValueError(f"K={W.K} is too large for the streaming small-M linear kernel")
        for m0 in range(0, M, mmax):
            m = min(mmax, M - m0)
            rs = residual[m0:m0 + m] if residual is not None else None
            _lib.call("ps_linear_stream", c_int(WFMT[W.fmt]), ptr(x[m0:m0 + m]), c_int(m), c_int(W.N),
                      c_int(W.k_padded), c_int(x.stride(0)), ptr(W.tiled), c_float(W.tensor_scale), c_int(pro),
                      ptr(norm_w), c_float(eps), ptr(None), c_int(0), c_int(epi), ptr(rs),
                      c_int(residual.stride(0) if residual is not None else 0), ptr(out[m0:m0 + m]),
                      c_int(out.stride(0)), c_int(1 if out_f32 else 0),
                      ptr(xn_out[m0:m0 + m] if xn_out is not None else None),
                      ctypes.byref(tp_combine) if tp_combine is not None else ptr(None), ptr(self.status))
            self.launches += 1
        return out

    def can_fuse_argmax(self, W: LinearW, M: int) -> bool:
        """True when ``linear_argmax`` can serve these rows: the streaming kernel would be chosen and holds them in one launch."""
        if M < 1 or M > SMALL_M_MAX or self.exact_rows or W.K % 32 or self.select_linear(W, M) != "stream":
            return False
        if M >= 2 and W.rowmajor_bf16 is not None and self.use_tc_gemm:
            return False
        L = _lib.lib()
        L.ps_linear_stream_max_rows.restype = ctypes.c_int
        return M <= L.ps_linear_stream_max_rows(c_int(WFMT[W.fmt]), c_int(W.k_padded))

    def linear_argmax(self, x: torch.Tensor, W: LinearW, *, norm_w=None, eps: float = 1e-6) -> torch.Tensor:
        """Greedy sampling fused into the projection (lm_head of a decode step): int32 [M] indices of each row's largest
        output, ties to the lower index; the logits are never written.  One launch."""
        M = x.shape[0]
        if W.tiled is None:
            W.make_tiled()
        if getattr(self, "_amax_state", None) is None:
            self._amax_state = torch.zeros(10, dtype=torch.int64, device=self.device)       # 8 keys + control words, kept zero by the kernel
        tokens = self.buf("sampled", max(M, 1), 1, torch.int32)
        _lib.call("ps_linear_stream_argmax", c_int(WFMT[W.fmt]), ptr(x), c_int(M), c_int(W.N), c_int(W.k_padded), c_int(x.stride(0)),
                  ptr(W.tiled), c_float(W.tensor_scale), c_int(PRO_RMSNORM if norm_w is not None else PRO_NONE), ptr(norm_w),
                  c_float(eps), ptr(None), c_int(0), ptr(self._amax_state), ptr(tokens), ptr(self.status))
        self.launches += 1
        self.sel_counts["stream"] += 1
        return tokens.view(-1)[:M]

    def linear_large(self, x: torch.Tensor, W: LinearW, *, name: str, norm_w, eps, residual, swiglu, out_f32, out):
        """Prefill-sized projection: (RMSNorm kernel) -> weight expansion to a bf16 scratch matrix -> tcgen05
        GEMM with the residual / SwiGLU / dtype epilogue fused."""
        M, K = x.shape
        a = x if norm_w is None else self.rmsnorm(x, norm_w, eps, "gemm_norm_in")
        if W.tiled is None:
            W.make_tiled()
        kp = W.k_padded
        if W.rowmajor_bf16 is not None:
            wd = W.rowmajor_bf16
        else:
            need = W.N * kp
            if self.wscratch is None or self.wscratch.numel() < need:
                self.wscratch = torch.empty(need, dtype=torch.bfloat16, device=self.device)
            wd = self.wscratch[:need].view(W.N, kp)
            _lib.call("ps_dequant_tiled", c_int(WFMT[W.fmt]), ptr(W.tiled), c_int(W.N), c_int(kp),
                      c_float(W.tensor_scale), ptr(wd), c_int(kp))
            self.launches += 1
        epi = EPI_SWIGLU if swiglu else (EPI_RESIDUAL if residual is not None else EPI_STORE)
        if W.rowmajor_bf16 is not None and M <= 64 and W.N % 2 == 0:
            # batched decode: swap-AB split-K weight-streaming GEMM (gemm_smallm.cu)
            L = _lib.lib()
            L.ps_gemm_smallm_splits.restype = ctypes.c_int
            splits = L.ps_gemm_smallm_splits(c_int(W.N), c_int(kp))
            need = splits * M * W.N
            part = self.ws.get(("smallm_partial", 0))
            if part is None or part.numel() < need:
                part = torch.empty(max(need, 1 << 22), dtype=torch.float32, device=self.device)
                self.ws[("smallm_partial", 0)] = part
            _lib.call("ps_gemm_smallm", ptr(a), c_int(a.stride(0)), ptr(wd), c_int(kp), c_int(M), c_int(W.N), c_int(kp), c_int(epi),
                      ptr(residual), c_int(residual.stride(0) if residual is not None else 0), ptr(out), c_int(out.stride(0)),
                      c_int(1 if out_f32 else 0), ptr(part), ptr(self.status))
            self.launches += 2
            return out
        _lib.call("ps_gemm_bf16_tc", ptr(a), c_int(a.stride(0)), ptr(wd), c_int(kp), c_int(M), c_int(W.N), c_int(kp),
                  c_int(epi), ptr(residual), c_int(residual.stride(0) if residual is not None else 0), ptr(out),
                  c_int(out.stride(0)), c_int(1 if out_f32 else 0), ptr(self.status))
        self.launches += 1
        return out

    # ------------------------------------------------------------------ kernel selection
    def select_linear(self, W: LinearW, M: int) -> str:
        """Which projection kernel serves `M` rows of `W` -- the job of the reference's linear selector
        (src/phaseshift/models/qwen35/runtime/linear_selector.cpp:202-308), here a pure function of the weight's
        resident layouts, the row count and two switches:

        * ``"tc"``     block-scaled tcgen05 kernel (needs ``W.sf_atoms``): every multi-row step, and single-row steps
                       when only that layout is resident or ``force_tc`` is set (speculative decoding: verification
                       and plain steps must share one arithmetic);
        * ``"stream"`` CUDA-core streaming kernel over ``W.tiled`` (bf16 activations): single rows, bf16 weights up to
                       8 rows, and Exact verification of weights that have no tensor-core layout;
        * ``"gemm"``   bf16 tcgen05 GEMM after a weight expansion: more than 8 rows of weights without ``sf_atoms``."""
        if W.sf_atoms is not None:
            if M > 1 or W.tiled is None or self.force_tc:
                return "tc"
            return "stream"
        if M > SMALL_M_MAX and self.use_tc_gemm and not self.exact_rows:
            return "gemm"
        return "stream"

    # ------------------------------------------------------------------ block-scaled tensor-core projection
    # Rows up to which the activations are quantised inside the projection kernel and kept resident (every CTA repeats that
    # prologue for the K-panels it needs, which pays for a handful of rows: 27B decode batches measured 13.1 vs 14.6 ms per
    # step at 12 rows and 18.6 vs 23.6 ms at 32 rows in favour of one `ps_act_quant` launch + the streamed kernel); the
    # kernel itself supports 32.
    BS_RESIDENT_MAX_ROWS = 8

    def _bs_workspace(self):
        if self.bs_ws is None:
            L = _lib.lib()
            L.ps_gemm_bs_workspace_bytes.restype = ctypes.c_longlong
            L.ps_gemm_bs_flag_words.restype = ctypes.c_int
            with torch.cuda.device(self.device):
                nbytes, nflags = int(L.ps_gemm_bs_workspace_bytes()), int(L.ps_gemm_bs_flag_words())
            self.bs_ws = torch.empty(nbytes // 4, dtype=torch.float32, device=self.device)
            self.bs_flags = torch.zeros(nflags, dtype=torch.int32, device=self.device)
        return self.bs_ws, self.bs_flags

    def reset_after_error(self) -> None:
        """A kernel gave up on a bounded wait: stream-K flags may be left raised; clear them."""
        if self.bs_flags is not None:
            self.bs_flags.zero_()
        if getattr(self, "_amax_state", None) is not None:
            self._amax_state.zero_()              # a fused arg-max launch that did not finish leaves its keys and counter
        self.status.zero_()

    def leaves_row_stats(self, W: LinearW, M: int) -> bool:
        """Whether a residual projection of `M` rows through `W` hands the next fused RMSNorm its rows' sums of squares."""
        return M <= 32 and getattr(W, "sf_atoms", None) is not None and self.select_linear(W, M) == "tc" and self.bs_resident_ok(W, M)

    def bs_resident_ok(self, W: LinearW, M: int) -> bool:
        """Whether `M` rows of this projection fit the kernel's resident-activation path (pure host arithmetic)."""
        if M > self.BS_RESIDENT_MAX_ROWS:
            return False
        key = (W.fmt, 16 if M <= 16 else 32, W.N, W.K)
        ok = self._bs_plan_cache.get(key)
        if ok is None:
            out = (ctypes.c_int * 8)()
            L = _lib.lib()
            L.ps_gemm_bs_plan.restype = ctypes.c_int
            with torch.cuda.device(self.device):
                ok = bool(L.ps_gemm_bs_plan(c_int(WFMT[W.fmt]), c_int(M), c_int(W.N), c_int(W.K), c_int(1),
                                            c_int(self.bs_grid_override), out))
            self._bs_plan_cache[key] = ok
        return ok

    def act_quant(self, x: torch.Tensor, W: LinearW, norm_w, eps: float):
        """Quantise `x` (after the optional fused RMSNorm) to the block format of `W` for the streamed path.
        Returns (codes uint8 [M, panels * 128], scale atoms uint8, row scale fp32 [M] = 1/rms)."""
        from ..quant.act_quant import ATOMS_PER_PANEL, PANEL_K
        M, K = x.shape
        P = -(-K // PANEL_K[W.fmt])
        # one buffer per (K, format): a preset mixes formats at the same K, and a shared name would re-allocate the
        # buffer at every change of format (inside a graph capture too)
        codes = self.buf(f"bs_xq{K}_{W.fmt}", M, P * 128, torch.uint8)
        mblk = -(-M // 256) * 2
        sf = self.buf(f"bs_xsf{K}_{W.fmt}", mblk, P * ATOMS_PER_PANEL[W.fmt] * 512, torch.uint8)
        rs = self.buf("bs_xrs", M, 1, torch.float32)
        _lib.call("ps_act_quant", c_int(WFMT[W.fmt]), ptr(x), c_int(x.stride(0)), c_int(M), c_int(K), ptr(norm_w),
                  c_float(eps), c_float(W.act_scale), ptr(codes), ptr(sf), ptr(rs))
        self.launches += 1
        return codes, sf, rs

    def linear_bs(self, x: torch.Tensor, W: LinearW, *, name: str, norm_w, eps, residual, swiglu, out_f32, out,
                  xn_out=None, tp_combine=None, ssq_in=None, ssq_out=None, prefetch=None, tp_scatter=None) -> torch.Tensor:
        M, K = x.shape
        if K % 8 or x.stride(0) % 8:
            raise ValueError("block-scaled projections need K and the row pitch to be multiples of 8")
        ws, flags = self._bs_workspace()
        epi = EPI_SWIGLU if swiglu else (EPI_RESIDUAL if residual is not None else EPI_STORE)
        resident = self.bs_resident_ok(W, M)
        self.sel_counts["tc_resident" if resident else "tc_streamed"] += 1
        if M <= self.BS_RESIDENT_MAX_ROWS and not resident:
            self.fallbacks["tc_resident_to_streamed"] = self.fallbacks.get("tc_resident_to_streamed", 0) + 1
        if tp_combine is not None and M > tp_combine.max_rows:
            raise ValueError("the fused tensor-parallel combine is sized for %d rows" % tp_combine.max_rows)
        codes = W.codes
        if resident:
            xq = sf = rs = None
        else:
            if xn_out is not None:
                raise ValueError("xn_out is produced by the resident path only")
            xq, sf, rs = self.act_quant(x, W, norm_w, eps)
        ssq_t, ssq_n = ssq_in if (ssq_in is not None and resident and norm_w is not None) else (None, 0)
        if M > 32 or swiglu or (not resident and not out_f32 and tp_combine is None):
            ssq_out = None          # the streamed kernel's staged bf16 epilogue leaves no row statistics
        nxt = prefetch if (prefetch is not None and prefetch.sf_atoms is not None and self.bs_prefetch) else None
        err = _lib.lib().ps_gemm_bs
        err.restype = ctypes.c_int
        rc = err(c_int(WFMT[W.fmt]), ptr(codes), c_ll(codes.shape[1]), c_ll(codes.stride(0)), ptr(W.sf_atoms),
                 c_float(W.tensor_scale), c_int(M), c_int(W.N), c_int(K), ptr(x if resident else None),
                 c_int(x.stride(0)), ptr(norm_w if resident else None), c_float(eps), c_float(W.act_scale),
                 ptr(xn_out), ptr(ssq_t), c_int(ssq_n), c_int(ssq_t.stride(0) if ssq_t is not None else 0),
                 ptr(ssq_out), c_int(ssq_out.stride(0) if ssq_out is not None else 0), ptr(xq), ptr(sf), ptr(rs),
                 c_int(epi), ptr(residual),
                 c_int(residual.stride(0) if residual is not None else 0), ptr(out), c_int(out.stride(0)),
                 c_int(1 if out_f32 else 0), ptr(ws), ptr(flags),
                 ctypes.byref(tp_combine) if tp_combine is not None else ptr(None), ptr(self.status),
                 c_int(self.bs_grid_override), c_int(WFMT[nxt.fmt] if nxt is not None else 0),
                 ptr(nxt.codes if nxt is not None else None), c_ll(nxt.codes.shape[1] if nxt is not None else 0),
                 c_ll(nxt.codes.stride(0) if nxt is not None else 0), ptr(nxt.sf_atoms if nxt is not None else None),
                 c_int(nxt.N if nxt is not None else 0), c_int(nxt.K if nxt is not None else 0),
                 ctypes.byref(tp_scatter) if tp_scatter is not None else ptr(None), _lib.stream())
        _lib.check(rc, "ps_gemm_bs")
        self.launches += 1
        return out

    def attn_prep(self, qkv: torch.Tensor, aw: AttnW, hq: int, hkv: int, b: StepBatch, kv: KVLayer,
                  st: ModelState) -> torch.Tensor:
        cfg = self.cfg
        rows, D = qkv.shape[0], cfg.head_dim
        q = self.buf("attn_q", rows, hq * D)
        _lib.call("ps_attn_prep", ptr(qkv), c_int(qkv.stride(0)), c_int(rows), c_int(hq), c_int(hkv), c_int(D),
                  c_int(cfg.rotary_dim), ptr(aw.q_norm), ptr(aw.k_norm), c_float(cfg.rms_norm_eps),
                  ptr(self.inv_freq), ptr(b.row_slot), ptr(b.row_pos), ptr(q), ptr(kv.k), ptr(kv.v),
                  ptr(kv.k_scale), ptr(kv.v_scale), ptr(st.block_table), c_int(st.max_blocks),
                  c_int(st.sc.page_tokens), c_int(st.num_pages), c_int(st.kv_fmt), ptr(st.status))
        self.launches += 1
        return q

    def paged_attention(self, q: torch.Tensor, qkv: torch.Tensor, hq: int, hkv: int, b: StepBatch, kv: KVLayer,
                        st: ModelState, max_visible: int) -> torch.Tensor:
        cfg = self.cfg
        rows, D = q.shape[0], cfg.head_dim
        out = self.buf("attn_ctx", rows, hq * D)
        # the tiled kernel pays off when some sequence brings a long run of rows (a prefill chunk); steps made of
        # many sequences with a row or two each (batched decode) keep the per-row split-KV kernel
        tiled = (not self.exact_rows and not b.graph_static and D in (64, 128, 256)
                 and any(len(sq.token_ids) > self.ATTN_PREFILL_MIN_ROWS for sq in b.seqs))
        row_pos = b.row_pos
        if tiled:
            # prefill-sized step: the long sequences' query tiles on the tensor cores (tcgen05 for head dim 256 and pages of
            # 16 / 32 / 64 tokens, FP8 pools through a bf16 scratch copy of the step's pages; mma.sync otherwise); sequences
            # with a row or two (decode rows of other requests in the same step) stay on the per-row kernel below
            T = self.ATTN_PREFILL_MIN_ROWS
            pt = st.sc.page_tokens
            any_short = T == StepBatch.SHORT_SEQ_ROWS and any(len(sq.token_ids) <= T for sq in b.seqs)
            min_rows = T if any_short else 0
            deq = (None, None, 0, None, None)
            src = (kv.k, kv.v, kv.k_scale, kv.v_scale, st.block_table, st.num_pages, b.seq_desc, 1 if st.kv_fp8 else 0)
            n_long_pages = lambda: sum(-(-(sq.pos_start + len(sq.token_ids)) // pt) for sq in b.seqs if len(sq.token_ids) > min_rows)
            if st.kv_fmt == 2:
                # NVFP4 pages: the step's pages are widened into the bf16 scratch pool, which then IS the pool of the tiled
                # kernels (with its own block table and sequence descriptors), whatever the head size
                dk, dv, n_pg, dbt, dsq = self._attn_scratch(n_long_pages(), hkv, pt, D, b.max_seqs, st.max_blocks)
                _lib.call("ps_kv_fp4_dequant", ptr(kv.k), ptr(kv.v), ptr(kv.k_scale), ptr(kv.v_scale), ptr(st.block_table),
                          c_int(st.max_blocks), c_int(st.num_pages), c_int(pt), c_int(hkv), c_int(D), ptr(b.seq_desc),
                          c_int(b.n_seqs), c_int(min_rows), ptr(dk), ptr(dv), c_int(n_pg), ptr(dbt), ptr(dsq), ptr(st.status))
                self.launches += 1
                src = (dk, dv, None, None, dbt, dk.shape[0], dsq, 0)
            elif st.kv_fp8 and D == 256 and pt in (16, 32, 64):
                deq = self._attn_scratch(n_long_pages(), hkv, pt, D, b.max_seqs, st.max_blocks)
            _lib.call("ps_attn_prefill", ptr(q), ptr(src[0]), ptr(src[1]), ptr(src[2]), ptr(src[3]),
                      ptr(src[4]), c_int(st.max_blocks), c_int(pt), c_int(src[5]),
                      ptr(src[6]), c_int(b.n_seqs), c_int(rows), c_int(q.shape[0]), c_int(min_rows), c_int(hq), c_int(hkv), c_int(D),
                      c_float(D ** -0.5), c_int(src[7]), ptr(qkv), c_int(qkv.stride(0)), c_int(2 * D), c_int(D),
                      ptr(deq[0]), ptr(deq[1]), c_int(deq[2]), ptr(deq[3]), ptr(deq[4]), ptr(out), ptr(st.status))
            self.launches += 2 if deq[0] is not None else 1
            if not any_short:
                return out
            row_pos = b.row_pos_short
        # Split length: 64 tokens give a single row enough CTAs to fill the GPU; a batch of many rows already does, and its
        # CTAs should rather amortise their set-up over a longer run of tokens (about four CTAs per SM in total).  Exact mode
        # and small batches keep the fixed length, so a row's summation order does not depend on its neighbours there.
        split_tokens = self.split_tokens
        if rows > SMALL_M_MAX and not self.exact_rows:
            want = max(1, (4 * 148) // (rows * hkv))
            split_tokens = max(split_tokens, -(-(-(-max_visible // want)) // 32) * 32)
        pacc = self.buf("attn_part_acc", rows, hq * self.max_splits * D, torch.float32)
        pml = self.buf("attn_part_ml", rows, hq * self.max_splits * 2, torch.float32)
        # Decode / verify rows on the tensor cores: bf16 pages, head dim 256, every sequence handled here has at most 16 rows
        # (the query heads that share a KV head are packed into one MMA tile).  A row's result does not depend on the other
        # rows of its tile (every tile row has its own scores, reference maximum and accumulator lane), so Exact mode -- whose
        # verified rows must reproduce single-row decoding bit for bit -- uses it as well.  FP8 pages and other shapes keep the
        # per-row kernel.  PS_ATTN_DECODE=legacy switches it off.
        if (self.attn_decode_tc and D == 256 and st.kv_fmt == 0 and st.sc.page_tokens in (16, 32, 64) and hq // hkv <= 8
                and (b.graph_static or row_pos is b.row_pos_short or all(len(sq.token_ids) <= 16 for sq in b.seqs))):
            st_tok = -(-split_tokens // 64) * 64
            n_seqs = b.max_seqs if b.graph_static else b.n_seqs
            _lib.call("ps_attn_decode_tc", ptr(q), c_int(q.shape[0]), ptr(kv.k), ptr(kv.v), ptr(st.block_table),
                      c_int(st.max_blocks), c_int(st.sc.page_tokens), c_int(st.num_pages), ptr(b.seq_desc), c_int(n_seqs),
                      c_int(16), c_int(hq), c_int(hkv), c_int(D), c_float(D ** -0.5), c_int(st_tok), c_int(self.max_splits),
                      c_int(max_visible), ptr(pacc), ptr(pml), ptr(st.status))
            _lib.call("ps_paged_attention_merge", ptr(pacc), ptr(pml), ptr(row_pos), c_int(rows), c_int(hq), c_int(D),
                      c_int(st_tok), c_int(self.max_splits), ptr(qkv), c_int(qkv.stride(0)), c_int(2 * D), c_int(D), ptr(out))
            self.launches += 2
            return out
        if st.kv_fmt == 2:
            _lib.call("ps_paged_attention_fp4", ptr(q), ptr(kv.k), ptr(kv.v), ptr(kv.k_scale), ptr(kv.v_scale),
                      ptr(st.block_table), c_int(st.max_blocks), c_int(st.sc.page_tokens), c_int(st.num_pages),
                      ptr(b.row_slot), ptr(row_pos), c_int(rows), c_int(hq), c_int(hkv), c_int(D), c_float(D ** -0.5),
                      c_int(split_tokens), c_int(self.max_splits), c_int(max_visible), ptr(pacc), ptr(pml), ptr(st.status))
            _lib.call("ps_paged_attention_merge", ptr(pacc), ptr(pml), ptr(row_pos), c_int(rows), c_int(hq), c_int(D),
                      c_int(split_tokens), c_int(self.max_splits), ptr(qkv), c_int(qkv.stride(0)), c_int(2 * D), c_int(D), ptr(out))
            self.launches += 2
            return out
        _lib.call("ps_paged_attention", ptr(q), ptr(kv.k), ptr(kv.v), ptr(kv.k_scale), ptr(kv.v_scale),
                  ptr(st.block_table), c_int(st.max_blocks), c_int(st.sc.page_tokens), c_int(st.num_pages),
                  ptr(b.row_slot), ptr(row_pos), c_int(rows), c_int(hq), c_int(hkv), c_int(D),
                  c_float(D ** -0.5), c_int(1 if st.kv_fp8 else 0), c_int(split_tokens),
                  c_int(self.max_splits), c_int(max_visible), ptr(pacc), ptr(pml), ptr(qkv), c_int(qkv.stride(0)),
                  c_int(2 * D), c_int(D), ptr(out), ptr(st.status))
        self.launches += 2
        return out

    def _attn_scratch(self, pages: int, hkv: int, pt: int, D: int, max_seqs: int, max_blocks: int):
        """bf16 scratch pool for the tiled attention over FP8 pages: (k, v, pages, block table, sequence descriptors).  One
        allocation that grows to the largest step seen (by doubling)."""
        cap = getattr(self, "_deq_cap", 0)
        if pages > cap or getattr(self, "_deq_geom", None) != (hkv, pt, D, max_seqs, max_blocks):
            cap = max(pages, 2 * cap, 64)
            self._deq_k = torch.empty(cap, hkv, pt, D, dtype=torch.bfloat16, device=self.device)
            self._deq_v = torch.empty_like(self._deq_k)
            self._deq_bt = torch.zeros(max_seqs, max_blocks, dtype=torch.int32, device=self.device)
            self._deq_seqs = torch.zeros(max_seqs, 4, dtype=torch.int32, device=self.device)
            self._deq_cap, self._deq_geom = cap, (hkv, pt, D, max_seqs, max_blocks)
        return self._deq_k, self._deq_v, pages, self._deq_bt, self._deq_seqs

    def gdn(self, proj: torch.Tensor, gw: GdnW, hk: int, hv: int, b: StepBatch, gs: GdnLayerState,
            st: ModelState, log=None, to_alt: bool = False, xn: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``xn`` given: the kernel projects beta/decay inputs itself from the normalised rows (bf16
        ``ba_proj`` weights); otherwise they are read from the last 2*hv columns of ``proj``."""
        cfg = self.cfg
        rows = proj.shape[0]
        Dk, Dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        out = self.buf("gdn_o", rows, hv * Dv)
        state_out = gs.rec_alt if to_alt else gs.rec
        n_seqs = b.max_seqs if b.graph_static else b.n_seqs
        # Sequences with many rows in this step (prefill chunks) take the chunked kernels, sequences with few rows
        # (decode / verify rows of other requests in the same step) the row-sequential kernel; both can be present.
        T = self.GDN_CHUNKED_MIN_ROWS
        plain = log is None and not to_alt and not self.exact_rows and not b.graph_static
        seq_rows = [len(sq.token_ids) for sq in b.seqs] if plain else []
        any_long = any(n > T for n in seq_rows)
        any_short = (not any_long) or any(n <= T for n in seq_rows)
        if any_long:
            f32 = torch.float32
            long_rows = sum(n for n in seq_rows if n > T)
            chunks = sum((n + 63) // 64 for n in seq_rows if n > T)
            scr = self.buf("gdn_scratch", 1, chunks * hv * 64 * (3 * Dk + Dv + 64), f32)
            dc = self.buf("gdn_dc", 1, chunks * hv, f32)
            o = self.buf("gdn_of", rows, hv * Dv, f32)
            if xn is not None:
                raise ValueError("the chunked GDN path reads the b/a projections from `proj`")
            _lib.call("ps_gdn_chunked", ptr(proj), c_int(proj.stride(0)), c_int(rows), c_int(hk), c_int(hv), c_int(Dk),
                      c_int(Dv), ptr(gw.conv_w), ptr(gw.A_log), ptr(gw.dt_bias), ptr(gw.norm_w),
                      c_float(cfg.rms_norm_eps), ptr(gs.conv), c_int(st.sc.conv_ring), ptr(gs.rec), ptr(b.seq_desc),
                      c_int(n_seqs), ptr(b.row_slot), ptr(b.row_pos), c_int(T), ptr(scr), ptr(dc), ptr(o), ptr(out))
            self.launches += 4
            del long_rows
        if any_short:
            lk = ld = ldd = None
            if log is not None:
                lk, ld, ldd = log
            _lib.call("ps_gdn_rows", ptr(proj), c_int(proj.stride(0)), c_int(hk), c_int(hv), c_int(Dk), c_int(Dv),
                      ptr(gw.conv_w), ptr(gw.A_log), ptr(gw.dt_bias), ptr(gw.norm_w), c_float(cfg.rms_norm_eps),
                      ptr(gs.conv), c_int(st.sc.conv_ring), ptr(gs.rec), ptr(state_out), ptr(b.seq_desc),
                      c_int(n_seqs), ptr(out), ptr(lk), ptr(ld), ptr(ldd),
                      ptr(gw.ba_proj.q.codes if xn is not None else None), ptr(xn), c_int(gw.ba_proj.K),
                      c_int(T if any_long else 0))
            self.launches += 1
        return out

    def gdn_replay(self, gs: GdnLayerState, hv: int, seq_desc: torch.Tensor, n_seqs: int, log) -> None:
        cfg = self.cfg
        lk, ld, ldd = log
        _lib.call("ps_gdn_replay", ptr(gs.rec), c_int(hv), c_int(cfg.linear_key_head_dim),
                  c_int(cfg.linear_value_head_dim), ptr(seq_desc), c_int(n_seqs), ptr(lk), ptr(ld), ptr(ldd))
        self.launches += 1

    def gather_rows(self, x: torch.Tensor, rows_idx: torch.Tensor, n: int, name: str, status) -> torch.Tensor:
        out = self.buf(name, n, x.shape[1], x.dtype)
        rb = x.shape[1] * x.element_size()
        _lib.call("ps_gather_rows", ptr(x), c_ll(x.stride(0) * x.element_size()), ptr(rows_idx), c_int(n), ptr(out),
                  c_ll(rb), c_int(rb), c_int(x.shape[0]), ptr(status))
        self.launches += 1
        return out

    def sample(self, logits: torch.Tensor, b: StepBatch, n: int, mask=None, mask_active=None,
               status=None) -> torch.Tensor:
        out = self.buf("sampled", max(n, 1), 1, torch.int32)
        _lib.call("ps_sample", ptr(logits), c_int(logits.stride(0)), c_int(logits.shape[1]), c_int(n), ptr(b.d_samp),
                  ptr(mask), c_int(mask.shape[1] if mask is not None else 0), ptr(mask_active), ptr(out), ptr(status))
        self.launches += 1
        return out.view(-1)[:n]

    def topk(self, logits: torch.Tensor, k: int, mask: Optional[torch.Tensor] = None):
        """Exact top-k (k <= 128) per row of fp32 logits, sorted descending, ties to the lower id.
        Returns (ids int32 [rows, k], values fp32 [rows, k]); `mask` is an optional allowed-token bitmask."""
        rows, vocab = logits.shape
        ids = self.buf("topk_ids", rows, k, torch.int32)
        vals = self.buf("topk_vals", rows, k, torch.float32)
        L = _lib.lib()
        L.ps_topk_workspace_bytes.restype = ctypes.c_longlong
        need = int(L.ps_topk_workspace_bytes(c_int(vocab), c_int(rows), c_int(k)))
        ws = self.buf("topk_ws", rows * k, need // (rows * k * 8), torch.int64)
        _lib.call("ps_topk", ptr(logits), c_ll(logits.stride(0)), c_int(vocab), c_int(rows), c_int(k), ptr(mask),
                  c_int(mask.shape[1] if mask is not None else 0), ptr(ids), ptr(vals), ptr(ws), c_ll(need))
        self.launches += 2
        return ids, vals

    def rmsnorm(self, x: torch.Tensor, w: torch.Tensor, eps: float, name: str, one_plus: bool = True,
                add: Optional[torch.Tensor] = None, sum_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        rows, H = x.shape
        out = self.buf(name, rows, H)
        _lib.call("ps_rmsnorm", ptr(x), c_int(x.stride(0)), ptr(add), c_int(add.stride(0) if add is not None else 0),
                  ptr(sum_out), c_int(sum_out.stride(0) if sum_out is not None else 0), ptr(w), c_float(eps),
                  c_int(rows), c_int(H), ptr(out), c_int(out.stride(0)), c_int(1 if one_plus else 0))
        self.launches += 1
        return out
