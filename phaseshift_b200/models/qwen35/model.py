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
    __slots__ = ("tokens", "logits", "hidden", "taps")

    def __init__(self, tokens, logits, hidden, taps):
        self.tokens, self.logits, self.hidden, self.taps = tokens, logits, hidden, taps


class Qwen35Runner:
    def __init__(self, weights: EngineWeights, state: ModelState, ops, tp=None):
        self.w, self.state, self.ops, self.tp = weights, state, ops, tp
        self.cfg: Qwen35Config = weights.cfg
        geo = state.geo
        self.hq, self.hkv = len(geo.q_heads), len(geo.kv_heads)
        self.hk, self.hv = len(geo.gdn_k_heads), len(geo.gdn_v_heads)
        # optional callable(tag, activations[rows, K]): importance-matrix collection at projection inputs
        self.imatrix_collector = None

    def _tap(self, tag: str, x: torch.Tensor, n_rows: int, norm_w=None) -> None:
        if self.imatrix_collector is None:
            return
        if norm_w is not None:
            x = self.ops.rmsnorm(x, norm_w, self.cfg.rms_norm_eps, "imatrix_norm")
        self.imatrix_collector(tag, x[:n_rows])

    def _row_parallel(self, inp: torch.Tensor, W, residual: torch.Tensor, name: str, rows: int) -> torch.Tensor:
        """Row-parallel projection + residual.  Single rank: residual fused in the projection epilogue.
        Tensor parallel, <= 8 rows: the projection kernel also performs the cross-rank sum (fused
        one-shot all-reduce over NVLink); otherwise the partial goes through the library all-reduce."""
        ops, tp = self.ops, self.tp
        if tp is None or tp.size <= 1:
            return ops.linear(inp, W, name=name, residual=residual)
        comb = tp.combine_for(W.N) if (rows <= 8 and hasattr(ops, "buf")) else None
        if comb is not None:
            tp.stats["fused"] += 1
            return ops.linear(inp, W, name=name, residual=residual, tp_combine=comb)
        part = ops.linear(inp, W, name="tp_partial")
        out = ops.buf(name, rows, W.N) if hasattr(ops, "buf") else torch.empty_like(part)
        return tp.all_reduce_residual(part, residual, out)

    def forward(self, b: StepBatch, rows: int, n_out: int, *, tap_layers: Sequence[int] = (),
                gdn_log: Optional[Dict[int, tuple]] = None, gdn_to_alt: bool = False,
                mask=None, mask_active=None, sample: bool = True) -> StepOutput:
        cfg, ops, st, w = self.cfg, self.ops, self.state, self.w
        eps = cfg.rms_norm_eps
        x = ops.embed(b, rows, w.embed, st.status)
        taps = {}
        from .weights import P as _P
        for li, L in enumerate(w.layers):
            m = L.mixer
            lp = f"{_P}layers.{li}."
            if L.kind == 0:
                self._tap(lp + "linear_attn.in_proj_qkv.weight", x, b.n_rows, L.input_norm)
                n_main = m.in_proj.N
                if hasattr(ops, "buf"):
                    proj = ops.buf("gdn_proj", rows, n_main + m.ba_proj.N)
                    batched = rows >= 2 and m.in_proj.shadow is not None and not ops.exact_rows
                    if rows <= FUSED_BA_MAX_ROWS and not batched:
                        # decode / verify: the GDN kernel projects beta/decay inputs itself from the
                        # normalised row that in_proj leaves behind -> one launch fewer per layer
                        xn = ops.buf("gdn_xn", rows, x.shape[1])
                        ops.linear(x, m.in_proj, name="gdn_in", norm_w=L.input_norm, eps=eps, out=proj[:, :n_main],
                                   xn_out=xn)
                    else:
                        xn = None
                        ops.linear(x, m.in_proj, name="gdn_in", norm_w=L.input_norm, eps=eps, out=proj[:, :n_main])
                        ops.linear(x, m.ba_proj, name="gdn_ba", norm_w=L.input_norm, eps=eps, out=proj[:, n_main:])
                    o = ops.gdn(proj, m, self.hk, self.hv, b, st.gdn[li], st,
                                log=None if gdn_log is None else gdn_log[li], to_alt=gdn_to_alt, xn=xn)
                else:
                    proj = torch.cat([ops.linear(x, m.in_proj, name="gdn_in", norm_w=L.input_norm, eps=eps),
                                      ops.linear(x, m.ba_proj, name="gdn_ba", norm_w=L.input_norm, eps=eps)], 1)
                    o = ops.gdn(proj, m, self.hk, self.hv, b, st.gdn[li], st,
                                log=None if gdn_log is None else gdn_log[li], to_alt=gdn_to_alt)
                self._tap(lp + "linear_attn.out_proj.weight", o, b.n_rows)
                r = self._row_parallel(o, m.out_proj, x, "r", rows)
            else:
                self._tap(lp + "self_attn.q_proj.weight", x, b.n_rows, L.input_norm)
                qkv = ops.linear(x, m.qkv_proj, name="attn_qkv", norm_w=L.input_norm, eps=eps)
                q = ops.attn_prep(qkv, m, self.hq, self.hkv, b, st.kv[li], st)
                ctx = ops.paged_attention(q, qkv, self.hq, self.hkv, b, st.kv[li], st, b.max_visible_launch)
                self._tap(lp + "self_attn.o_proj.weight", ctx, b.n_rows)
                r = self._row_parallel(ctx, m.o_proj, x, "r", rows)
            self._tap(lp + "mlp.gate_proj.weight", r, b.n_rows, L.post_norm)
            act = ops.linear(r, L.gate_up, name="mlp_act", norm_w=L.post_norm, eps=eps, swiglu=True)
            self._tap(lp + "mlp.down_proj.weight", act, b.n_rows)
            # ping-pong the residual stream so a layer never writes the buffer it still reads
            xname = "x_a" if (li & 1) == 0 else "x_b"
            x = self._row_parallel(act, L.down, r, xname, rows)
            if li in tap_layers:
                taps[li] = x if not hasattr(ops, "buf") else ops.buf(f"tap{li}", rows, x.shape[1]).copy_(x)
        tokens = logits = hidden = None
        if n_out > 0:
            hidden = ops.gather_rows(x, b.out_rows, n_out, "out_hidden", st.status)
            self._tap(_P + "lm_head.weight", hidden, n_out, w.final_norm)
            logits = ops.linear(hidden, w.lm_head, name="logits", norm_w=w.final_norm, eps=eps, out_f32=True)
            if sample:
                tokens = ops.sample(logits, b, n_out, mask=mask, mask_active=mask_active, status=st.status)
        return StepOutput(tokens, logits, hidden, taps)
