"""Qwen3.5 hybrid decoder forward over an op set (CUDA kernels or the PyTorch reference ops).

One call = one scheduled step over a mixed batch of rows (decode rows, prefill chunks, speculative
verify rows): the public contract is phase-agnostic like the reference executor's
(AGENTS.md:133-157).  A decode layer is 5 launches (GDN) or 7 (full attention): the norms, gates,
residual adds and SwiGLU live in the projection kernels' prologues/epilogues, versus ~26 dispatches
per layer in the reference's lowering (src/phaseshift/models/qwen35/model/lower_to_primitives.cpp:694-960).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ...runtime.batch import StepBatch
from ...runtime.state import ModelState
from .config import Qwen35Config
from .weights import EngineWeights


FUSED_BA_MAX_ROWS = 8


class StepOutput:
    __slots__ = ("tokens", "logits", "hidden", "taps", "taps_cat", "read_back")

    def __init__(self, tokens, logits, hidden, taps, taps_cat=None):
        self.tokens, self.logits, self.hidden, self.taps = tokens, logits, hidden, taps
        self.taps_cat = taps_cat        # the tapped hidden states side by side, [rows, taps * H] (taps are views of it)
        self.read_back = None


class Qwen35Runner:
    def __init__(self, weights: EngineWeights, state: ModelState, ops, tp=None):
        self.w, self.state, self.ops, self.tp = weights, state, ops, tp
        self.cfg: Qwen35Config = weights.cfg
        geo = state.geo
        self.hq, self.hkv = len(geo.q_heads), len(geo.kv_heads)
        self.hk, self.hv = len(geo.gdn_k_heads), len(geo.gdn_v_heads)
        # optional callable(tag, activations[rows, K]): importance-matrix collection at projection inputs
        self.imatrix_collector = None
        # optional callable(tag, values[rows, K]): what the tensor-core projections quantise at each input site,
        # i.e. x (1 + norm weight) before the row factor 1/rms (activation-scale calibration)
        self.act_collector = None
        self.use_ssq = hasattr(ops, "ssq_buf")

    def _tap(self, tag: str, x: torch.Tensor, n_rows: int, norm_w=None) -> None:
        if self.act_collector is not None:
            v = x[:n_rows].float()
            self.act_collector(tag, v * (1.0 + norm_w.float()) if norm_w is not None else v)
        if self.imatrix_collector is None:
            return
        if norm_w is not None:
            x = self.ops.rmsnorm(x, norm_w, self.cfg.rms_norm_eps, "imatrix_norm")
        self.imatrix_collector(tag, x[:n_rows])

    def _first_proj(self, li: int):
        """The first projection of layer `li` (the lm_head after the last layer): what runs after layer li-1's down."""
        if li >= len(self.w.layers):
            return self.w.lm_head
        L = self.w.layers[li]
        return L.mixer.in_proj if L.kind == 0 else L.mixer.qkv_proj

    def _row_parallel(self, inp: torch.Tensor, W, residual: torch.Tensor, name: str, rows: int, nxt=None):
        """Row-parallel projection + residual.  Single rank: residual fused in the projection epilogue.
        Tensor parallel, few rows: the projection kernel also performs the cross-rank sum (fused one-shot
        all-reduce over NVLink); otherwise the partial goes through the all-reduce kernel / library.
        Returns (output, ssq): ssq = (tensor, n) partial sums of squares of the output rows when the kernel left
        them for the next fused RMSNorm, else None."""
        ops, tp = self.ops, self.tp
        ssq_out, ssq = None, None
        if self.use_ssq and rows <= 32 and getattr(W, "sf_atoms", None) is not None and \
                (not hasattr(ops, "leaves_row_stats") or ops.leaves_row_stats(W, rows)):
            ssq_out = ops.ssq_buf(name, rows)
            ssq = (ssq_out, -(-W.N // 128))
        kw = {"prefetch": nxt} if self.use_ssq else {}
        if tp is None or tp.size <= 1:
            return ops.linear(inp, W, name=name, residual=residual, ssq_out=ssq_out, **kw), ssq
        comb = tp.combine_for(W.N) if (rows <= tp.max_fused_rows(W) and hasattr(ops, "buf")) else None
        if comb is not None:
            tp.stats["fused"] += 1
            return ops.linear(inp, W, name=name, residual=residual, tp_combine=comb, ssq_out=ssq_out, **kw), ssq
        if (tp.transport == "fused" and hasattr(ops, "select_linear") and ops.select_linear(W, rows) == "tc"
                and not ops.bs_resident_ok(W, rows) and W.N % 8 == 0 and getattr(tp, "use_scatter", True)):
            # many rows: the projection's epilogue pushes its partial rows to their owner ranks while later tiles
            # are still being multiplied; the owners reduce, add the residual and hand the rows to everybody
            ops.linear(inp, W, name="tp_partial", tp_scatter=tp.scatter_for(rows, W.N))
            return tp.reduce_gather(rows, W.N, residual, name), None
        if (tp.transport == "fused" and hasattr(ops, "buf") and W.N % 8 == 0 and rows >= tp.size
                and getattr(tp, "use_scatter", True)):
            # projection kernels that cannot push: the collective kernel deals the partial to the owners itself
            part = ops.linear(inp, W, name="tp_partial")
            return tp.reduce_gather(rows, W.N, residual, name, partial=part), None
        part = ops.linear(inp, W, name="tp_partial")
        out = ops.buf(name, rows, W.N) if hasattr(ops, "buf") else torch.empty_like(part)
        return tp.all_reduce_residual(part, residual, out), None

    def forward(self, b: StepBatch, rows: int, n_out: int, *, tap_layers: Sequence[int] = (),
                gdn_log: Optional[Dict[int, tuple]] = None, gdn_to_alt: bool = False,
                mask=None, mask_active=None, sample: bool = True, greedy_only: bool = False) -> StepOutput:
        """``greedy_only``: every output row is sampled greedily, without a mask, and nobody reads the logits: the lm_head
        may then produce the token ids itself (fused arg-max) and ``StepOutput.logits`` is None."""
        cfg, ops, st, w = self.cfg, self.ops, self.state, self.w
        eps = cfg.rms_norm_eps
        x_ssq = None
        with ops.range("embed"):
            if self.use_ssq and rows <= 32:
                e_ssq = ops.ssq_buf("embed", rows)
                x = ops.embed(b, rows, w.embed, st.status, ssq_out=e_ssq)
                x_ssq = (e_ssq, 1)
            else:
                x = ops.embed(b, rows, w.embed, st.status)
        taps = {}
        taps_cat = None
        if tap_layers and hasattr(ops, "buf"):
            # one buffer for all taps: a block drafter reads them side by side as its fc input
            taps_cat = ops.buf("taps_cat", rows, len(tap_layers) * cfg.hidden_size)
        tap_order = {li: j for j, li in enumerate(tap_layers)}
        from .weights import P as _P
        for li, L in enumerate(w.layers):
            m = L.mixer
            lp = f"{_P}layers.{li}."
            if L.kind == 0:
                self._tap(lp + "linear_attn.in_proj_qkv.weight", x, b.n_rows, L.input_norm)
                n_main = m.in_proj.N
                rng = ops.range("gdn.in_proj")
                rng.__enter__()
                if hasattr(ops, "buf"):
                    proj = ops.buf("gdn_proj", rows, n_main + m.ba_proj.N)
                    batched = rows >= 2 and m.in_proj.rowmajor_bf16 is not None and not ops.exact_rows
                    if rows <= FUSED_BA_MAX_ROWS and not batched:
                        # decode / verify: the GDN kernel projects beta/decay inputs itself from the
                        # normalised row that in_proj leaves behind -> one launch fewer per layer
                        xn = ops.buf("gdn_xn", rows, x.shape[1])
                        ops.linear(x, m.in_proj, name="gdn_in", norm_w=L.input_norm, eps=eps, out=proj[:, :n_main],
                                   xn_out=xn, ssq_in=x_ssq, prefetch=m.out_proj)
                    else:
                        xn = None
                        ops.linear(x, m.in_proj, name="gdn_in", norm_w=L.input_norm, eps=eps, out=proj[:, :n_main],
                                   ssq_in=x_ssq, prefetch=m.out_proj)
                        ops.linear(x, m.ba_proj, name="gdn_ba", norm_w=L.input_norm, eps=eps, out=proj[:, n_main:])
                    rng.__exit__(None, None, None)
                    with ops.range("gdn.mixer"):
                        o = ops.gdn(proj, m, self.hk, self.hv, b, st.gdn[li], st,
                                    log=None if gdn_log is None else gdn_log[li], to_alt=gdn_to_alt, xn=xn)
                else:
                    proj = torch.cat([ops.linear(x, m.in_proj, name="gdn_in", norm_w=L.input_norm, eps=eps),
                                      ops.linear(x, m.ba_proj, name="gdn_ba", norm_w=L.input_norm, eps=eps)], 1)
                    rng.__exit__(None, None, None)
                    with ops.range("gdn.mixer"):
                        o = ops.gdn(proj, m, self.hk, self.hv, b, st.gdn[li], st,
                                    log=None if gdn_log is None else gdn_log[li], to_alt=gdn_to_alt)
                self._tap(lp + "linear_attn.out_proj.weight", o, b.n_rows)
                with ops.range("gdn.out_proj"):
                    r, r_ssq = self._row_parallel(o, m.out_proj, x, "r", rows, L.gate_up)
            else:
                self._tap(lp + "self_attn.q_proj.weight", x, b.n_rows, L.input_norm)
                with ops.range("attn.qkv_proj"):
                    qkv = ops.linear(x, m.qkv_proj, name="attn_qkv", norm_w=L.input_norm, eps=eps,
                                     **({"ssq_in": x_ssq, "prefetch": m.o_proj} if self.use_ssq else {}))
                with ops.range("attn.prep"):
                    q = ops.attn_prep(qkv, m, self.hq, self.hkv, b, st.kv[li], st)
                with ops.range("attn.core"):
                    ctx = ops.paged_attention(q, qkv, self.hq, self.hkv, b, st.kv[li], st, b.max_visible_launch)
                self._tap(lp + "self_attn.o_proj.weight", ctx, b.n_rows)
                with ops.range("attn.o_proj"):
                    r, r_ssq = self._row_parallel(ctx, m.o_proj, x, "r", rows, L.gate_up)
            self._tap(lp + "mlp.gate_proj.weight", r, b.n_rows, L.post_norm)
            with ops.range("mlp.gate_up"):
                act = ops.linear(r, L.gate_up, name="mlp_act", norm_w=L.post_norm, eps=eps, swiglu=True,
                                 **({"ssq_in": r_ssq, "prefetch": L.down} if self.use_ssq else {}))
            self._tap(lp + "mlp.down_proj.weight", act, b.n_rows)
            # ping-pong the residual stream so a layer never writes the buffer it still reads
            xname = "x_a" if (li & 1) == 0 else "x_b"
            with ops.range("mlp.down"):
                x, x_ssq = self._row_parallel(act, L.down, r, xname, rows, self._first_proj(li + 1))
            if li in tap_layers:
                if taps_cat is None:
                    taps[li] = x
                else:
                    H = x.shape[1]
                    taps[li] = taps_cat[:, tap_order[li] * H:(tap_order[li] + 1) * H].copy_(x)
        tokens = logits = hidden = None
        if n_out > 0:
            if b.identity_out and self.use_ssq:
                hidden, h_ssq = x[:n_out], x_ssq          # pure decode batch: no gather, and the row statistics carry over
            else:
                hidden, h_ssq = ops.gather_rows(x, b.out_rows, n_out, "out_hidden", st.status), None
            self._tap(_P + "lm_head.weight", hidden, n_out, w.final_norm)
            if (greedy_only and sample and mask is None and self.tp is None and hasattr(ops, "can_fuse_argmax")
                    and ops.can_fuse_argmax(w.lm_head, n_out)):
                with ops.range("head.lm_head"):
                    tokens = ops.linear_argmax(hidden, w.lm_head, norm_w=w.final_norm, eps=eps)
                return StepOutput(tokens, None, hidden, taps, taps_cat)
            with ops.range("head.lm_head"):
                logits = ops.linear(hidden, w.lm_head, name="logits", norm_w=w.final_norm, eps=eps, out_f32=True,
                                    **({"ssq_in": h_ssq} if self.use_ssq else {}))
            if sample:
                with ops.range("head.sample"):
                    tokens = ops.sample(logits, b, n_out, mask=mask, mask_active=mask_active, status=st.status)
        return StepOutput(tokens, logits, hidden, taps, taps_cat)
