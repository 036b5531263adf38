"""Multi-token-prediction (MTP) head of the Qwen3.5 family used as a built-in one-layer drafter.

Forward contract (reference: docs/developer/mtp.md:100-143, lowering in
src/phaseshift/models/qwen35/model/lower_to_primitives.cpp:1017-1271, executor
src/phaseshift/models/qwen35/runtime/mtp_executor.hip, KV state mtp_kv_state.cpp):

    e = RMSNorm(embed(token));  h = RMSNorm(hidden)                (pre_fc_norm_embedding / pre_fc_norm_hidden)
    x = fc([e, h])                                                  (2H -> H, embedding half first)
    one gated full-attention decoder layer over the head's own KV state (q/gate interleaved per head, per-head
    q/k RMSNorm, partial NeoX RoPE, sigmoid gate before o_proj, residual = x), then the SwiGLU MLP
    hidden_out = layer output (before the final norm);  logits = lm_head(RMSNorm(hidden_out))   (mtp.norm, tied head)

Every RMSNorm is the (1 + w) form.  Row j of the head's KV state pairs the target's hidden state of position j
with the token of position j + 1 and predicts the token of position j + 2.  A proposal of k tokens chains the head
on its own output: the first row uses the target's hidden state of the last committed position, every further row
uses the previous row's ``hidden_out`` (``chain="pre"``) or its normed form (``chain="post"``); chained rows are
speculative and leave the KV state again.  The committed rows are recomputed from the target's true hidden states
when the verified tokens come back (``append_context``).

The class implements the drafter interface of the speculative decoder (``DFlash2SpecDecoder``): ``cfg.
target_layer_ids`` (here: the last layer, i.e. the hidden state in front of the final norm), ``reset``,
``append_context`` and ``propose``; the decoder verifies in Exact numeric mode, so the emitted stream equals plain
greedy decoding whatever the head proposes.  As upstream, the head is a bench / test component and is not wired
into the serving path.
"""
from __future__ import annotations

import zlib
from types import SimpleNamespace
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from .config import Qwen35Config

MP = "mtp."
LP = "mtp.layers.0."


def mtp_tensor_shapes(c: Qwen35Config) -> Dict[str, tuple]:
    h, i, D = c.hidden_size, c.intermediate_size, c.head_dim
    q, kv = c.num_attention_heads * D, c.num_key_value_heads * D
    return {MP + "fc.weight": (h, 2 * h), MP + "pre_fc_norm_embedding.weight": (h,), MP + "pre_fc_norm_hidden.weight": (h,),
            MP + "norm.weight": (h,),
            LP + "input_layernorm.weight": (h,), LP + "post_attention_layernorm.weight": (h,),
            LP + "self_attn.q_proj.weight": (2 * q, h), LP + "self_attn.k_proj.weight": (kv, h),
            LP + "self_attn.v_proj.weight": (kv, h), LP + "self_attn.o_proj.weight": (h, q),
            LP + "self_attn.q_norm.weight": (D,), LP + "self_attn.k_norm.weight": (D,),
            LP + "mlp.gate_proj.weight": (i, h), LP + "mlp.up_proj.weight": (i, h), LP + "mlp.down_proj.weight": (h, i)}


def validate_mtp_geometry(c: Qwen35Config, shapes: Dict[str, tuple]) -> None:
    """Shape contract of the head's tensors against the target configuration."""
    for n, want in mtp_tensor_shapes(c).items():
        if n not in shapes:
            raise ValueError(f"MTP head: tensor {n} is missing")
        if tuple(shapes[n]) != tuple(want):
            raise ValueError(f"MTP head: {n} has shape {tuple(shapes[n])}, expected {tuple(want)}")


def random_mtp_weights(c: Qwen35Config, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
    out = {}
    for n, shp in mtp_tensor_shapes(c).items():
        g = torch.Generator(device=device)
        g.manual_seed((seed * 104729 + zlib.crc32(n.encode())) & 0x7FFFFFFF)
        if n.endswith("norm.weight") or n.endswith("norm_embedding.weight") or n.endswith("norm_hidden.weight"):
            t = 0.02 * torch.randn(shp, device=device, generator=g)          # (1 + w) form: w near 0
        else:
            t = torch.randn(shp, device=device, generator=g) * (shp[-1] ** -0.5)
        out[n] = t.to(torch.bfloat16)
    return out


def _rms1p(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + w.float())).to(x.dtype)


def _rope_partial(x: torch.Tensor, pos: torch.Tensor, rotary_dim: int, theta: float) -> torch.Tensor:
    """x [T, H, D]: NeoX half-rotate pairing on the first ``rotary_dim`` dims."""
    half = rotary_dim // 2
    inv = theta ** (-torch.arange(half, device=x.device, dtype=torch.float32) * 2.0 / rotary_dim)
    ang = pos.to(torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xf = x.float()
    lo, hi = xf[..., :half], xf[..., half:rotary_dim]
    return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin, xf[..., rotary_dim:]], -1).to(x.dtype)


class MTPDrafter:
    wants_tokens = True            # append_context needs the committed rows' token ids as well as their hidden states

    def __init__(self, target_cfg: Qwen35Config, weights: Dict[str, torch.Tensor], device, dtype=torch.float32,
                 chain: str = "pre"):
        if chain not in ("pre", "post"):
            raise ValueError("chain must be 'pre' or 'post'")
        validate_mtp_geometry(target_cfg, {k: tuple(v.shape) for k, v in weights.items()})
        self.c, self.device, self.dtype, self.chain = target_cfg, torch.device(device), dtype, chain
        self.cfg = SimpleNamespace(target_layer_ids=[target_cfg.num_hidden_layers - 1])
        self.w = {k: v.to(device=self.device, dtype=dtype) for k, v in weights.items() if k.startswith(MP)}
        self.embed = None
        self.lm_head_logits = None
        self.k_cache = self.v_cache = None
        self.reset()

    @staticmethod
    def from_dir(model_dir, target_cfg: Qwen35Config, device, dtype=torch.float32, chain: str = "pre") -> "MTPDrafter":
        """Reads the ``mtp.*`` tensors of a BF16 Hugging Face model directory."""
        from ...io.model_dir import ShardCollection
        col = ShardCollection(model_dir)
        w = {}
        for n in mtp_tensor_shapes(target_cfg):
            if not col.has(n):
                raise ValueError(f"{model_dir} has no MTP head (missing {n})")
            w[n] = col.tensor(n).clone()
        col.close()
        return MTPDrafter(target_cfg, w, device, dtype, chain)

    def bind(self, embed, lm_head_logits) -> None:
        """``embed(ids)`` -> target embedding rows, ``lm_head_logits(h)`` -> fp32 logits of the (tied) target head."""
        self.embed, self.lm_head_logits = embed, lm_head_logits

    def reset(self) -> None:
        self.kv_len = 0                 # committed rows of the head's KV state
        self.h_prev = None              # target hidden of the last committed position (its next token is still unknown)

    # ------------------------------------------------------------------ one forward over n rows at KV rows pos0..
    def _reserve(self, n: int) -> None:
        c = self.c
        cap = 0 if self.k_cache is None else self.k_cache.shape[0]
        if n <= cap:
            return
        new = max(256, cap * 2, n)
        k = torch.zeros(new, c.num_key_value_heads, c.head_dim, device=self.device, dtype=self.dtype)
        v = torch.zeros_like(k)
        if cap:
            k[:cap], v[:cap] = self.k_cache, self.v_cache
        self.k_cache, self.v_cache = k, v

    def forward(self, emb: torch.Tensor, hid: torch.Tensor, pos0: int) -> torch.Tensor:
        """Rows (emb[i], hid[i]) at KV rows pos0 + i; writes their K/V and returns ``hidden_out`` [n, H]."""
        c, w, eps = self.c, self.w, self.c.rms_norm_eps
        n = emb.shape[0]
        Hq, Hkv, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        e = _rms1p(emb.to(self.dtype), w[MP + "pre_fc_norm_embedding.weight"], eps)
        h = _rms1p(hid.to(self.dtype), w[MP + "pre_fc_norm_hidden.weight"], eps)
        x = torch.cat([e, h], -1) @ w[MP + "fc.weight"].T
        a = _rms1p(x, w[LP + "input_layernorm.weight"], eps)
        qg = (a @ w[LP + "self_attn.q_proj.weight"].T).reshape(n, Hq, 2 * D)
        q, gate = qg[..., :D], qg[..., D:]
        k = (a @ w[LP + "self_attn.k_proj.weight"].T).reshape(n, Hkv, D)
        v = (a @ w[LP + "self_attn.v_proj.weight"].T).reshape(n, Hkv, D)
        pos = torch.arange(pos0, pos0 + n, device=self.device)
        q = _rope_partial(_rms1p(q, w[LP + "self_attn.q_norm.weight"], eps), pos, c.rotary_dim, c.rope_theta)
        k = _rope_partial(_rms1p(k, w[LP + "self_attn.k_norm.weight"], eps), pos, c.rotary_dim, c.rope_theta)
        self._reserve(pos0 + n)
        self.k_cache[pos0:pos0 + n], self.v_cache[pos0:pos0 + n] = k, v
        G = Hq // Hkv
        K = self.k_cache[:pos0 + n].repeat_interleave(G, 1).float()
        V = self.v_cache[:pos0 + n].repeat_interleave(G, 1).float()
        s = torch.einsum("thd,shd->hts", q.float(), K) * (D ** -0.5)
        visible = torch.arange(pos0 + n, device=self.device)[None, :] <= pos[:, None]
        s = s.masked_fill(~visible[None], float("-inf"))
        ctx = torch.einsum("hts,shd->thd", torch.softmax(s, -1), V) * torch.sigmoid(gate.float())
        o = ctx.to(self.dtype).reshape(n, Hq * D) @ w[LP + "self_attn.o_proj.weight"].T
        r = o + x
        m = _rms1p(r, w[LP + "post_attention_layernorm.weight"], eps)
        d = (F.silu(m @ w[LP + "mlp.gate_proj.weight"].T) * (m @ w[LP + "mlp.up_proj.weight"].T)) @ w[LP + "mlp.down_proj.weight"].T
        return d + r

    def logits(self, hidden_out: torch.Tensor) -> torch.Tensor:
        return self.lm_head_logits(_rms1p(hidden_out, self.w[MP + "norm.weight"], self.c.rms_norm_eps)).float()

    # ------------------------------------------------------------------ drafter interface
    def append_context(self, taps: Sequence[torch.Tensor], pos_start: int, tokens: Optional[Sequence[int]] = None) -> None:
        """Committed target rows at positions pos_start.. : ``taps[0][i]`` is the hidden state (in front of the final
        norm) of position pos_start + i and ``tokens[i]`` the token fed there.  KV row j pairs hidden j with token
        j + 1, so the last hidden waits for its token until the next call."""
        hid = taps[0]
        n = hid.shape[0]
        if n == 0:
            return
        if tokens is None or len(tokens) != n:
            raise ValueError("the MTP head needs the committed rows' tokens")
        if pos_start != self.kv_len + (0 if self.h_prev is None else 1):
            raise ValueError(f"MTP head: rows arrive at position {pos_start}, KV state holds {self.kv_len} rows")
        hid = hid.to(self.dtype)
        ids = torch.as_tensor(list(tokens), dtype=torch.long, device=self.device)
        if self.h_prev is not None:
            rows_h, rows_t, p0 = torch.cat([self.h_prev[None], hid[:-1]], 0), ids, pos_start - 1
        else:
            rows_h, rows_t, p0 = hid[:-1], ids[1:], pos_start
        if rows_t.numel():
            self.forward(self.embed(rows_t), rows_h, p0)
            self.kv_len = p0 + rows_t.numel()
        self.h_prev = hid[-1].clone()

    def propose(self, anchor: int, k: int, embed=None, lm_head_logits=None, pos_start: int = 0, allowed=None) -> List[int]:
        """k greedy draft tokens after ``anchor`` (the pending token of position ``pos_start``).  Speculative rows
        leave the KV state again: the committed length is unchanged on return."""
        if embed is not None:
            self.bind(embed, lm_head_logits)
        if self.h_prev is None or k <= 0:
            return []
        if pos_start - 1 != self.kv_len:
            raise ValueError(f"MTP head: proposal at position {pos_start}, KV state holds {self.kv_len} rows")
        drafts: List[int] = []
        tok = torch.tensor([anchor], dtype=torch.long, device=self.device)
        hid = self.h_prev[None]
        for i in range(k):
            out = self.forward(self.embed(tok), hid, self.kv_len + i)
            lg = self.logits(out)
            if allowed is not None:
                lg = lg.masked_fill(~allowed[i:i + 1], float("-inf"))
            tok = torch.argmax(lg, -1)                         # first maximal id on ties
            drafts.append(tok)
            hid = out if self.chain == "pre" else _rms1p(out, self.w[MP + "norm.weight"], self.c.rms_norm_eps)
        return torch.cat(drafts).tolist()                      # one host synchronisation per proposal


def mtp_reference_rows(c: Qwen35Config, weights: Dict[str, torch.Tensor], tokens: Sequence[int], hidden: torch.Tensor,
                       lm_head: torch.Tensor, embed_table: torch.Tensor) -> torch.Tensor:
    """fp32 oracle: logits of every head row for one sequence, computed in one full causal pass.  Row j uses
    ``hidden[j]`` and ``tokens[j + 1]`` (so ``len(tokens) == hidden.shape[0] + 1``)."""
    d = MTPDrafter(c, weights, "cpu", torch.float32)
    d.bind(lambda ids: embed_table.float()[ids], lambda h: h.float() @ lm_head.float().T)
    ids = torch.as_tensor(list(tokens[1:]), dtype=torch.long)
    out = d.forward(embed_table.float()[ids], hidden.float(), 0)
    return d.logits(out)
