"""Pure-PyTorch fp32 oracle of the Qwen3.5-style hybrid decoder.

A direct, unoptimised restatement of the network the reference lowers in
src/phaseshift/models/qwen35/model/lower_to_primitives.cpp:522-1015 (numerics from
kernels/correctness/detail/{normalization,gdn,attention}.inc): whole-sequence, no paging, no caches,
no fusion.  Every engine path (CPU reference ops, CUDA kernels, quantised weights, TP) is checked
against this function.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .config import Qwen35Config

P = "model.language_model."


def rms_norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + w)


def rms_norm_direct(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def l2_norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).sum(-1, keepdim=True) + eps)


def rope_neox_partial(x: torch.Tensor, pos: torch.Tensor, rotary_dim: int, theta: float) -> torch.Tensor:
    """x [T, H, D]; rotate the first rotary_dim dims with the half-rotate (NeoX) pairing."""
    half = rotary_dim // 2
    inv_freq = theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / rotary_dim)
    ang = pos.to(torch.float64)[:, None] * inv_freq[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x = x.clone()
    lo, hi = x[..., :half].double(), x[..., half:rotary_dim].double()
    x[..., :half] = (lo * cos - hi * sin).to(x.dtype)
    x[..., half:rotary_dim] = (hi * cos + lo * sin).to(x.dtype)
    return x


def gdn_mixer(cfg: Qwen35Config, w: Dict[str, torch.Tensor], pre: str, n: torch.Tensor) -> torch.Tensor:
    T = n.shape[0]
    Hk, Hv, Dk, Dv = (cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim,
                      cfg.linear_value_head_dim)
    qkv = n @ w[pre + "in_proj_qkv.weight"].T
    z = n @ w[pre + "in_proj_z.weight"].T
    b = n @ w[pre + "in_proj_b.weight"].T
    a = n @ w[pre + "in_proj_a.weight"].T
    cw = w[pre + "conv1d.weight"].reshape(cfg.gdn_conv_dim, 4)          # tap 3 multiplies the current input
    xp = torch.cat([qkv.new_zeros(3, qkv.shape[1]), qkv], 0)
    c = sum(cw[:, j][None, :] * xp[j:j + T] for j in range(4))
    c = torch.nn.functional.silu(c)
    qk = cfg.gdn_qk_dim
    q = l2_norm(c[:, :qk].reshape(T, Hk, Dk)) * (Dk ** -0.5)
    k = l2_norm(c[:, qk:2 * qk].reshape(T, Hk, Dk))
    v = c[:, 2 * qk:].reshape(T, Hv, Dv)
    rep = Hv // Hk
    q = q.repeat_interleave(rep, 1)
    k = k.repeat_interleave(rep, 1)
    beta = torch.sigmoid(b)                                               # [T, Hv]
    g = -torch.exp(w[pre + "A_log"].float()) * torch.nn.functional.softplus(a + w[pre + "dt_bias"].float())
    d = torch.exp(g)
    S = n.new_zeros(Hv, Dk, Dv)
    outs = []
    for t in range(T):
        S = S * d[t][:, None, None]
        kv = torch.einsum("hkv,hk->hv", S, k[t])
        delta = (v[t] - kv) * beta[t][:, None]
        S = S + k[t][:, :, None] * delta[:, None, :]
        outs.append(torch.einsum("hkv,hk->hv", S, q[t]))
    o = torch.stack(outs, 0)                                              # [T, Hv, Dv]
    o = rms_norm_direct(o, w[pre + "norm.weight"], cfg.rms_norm_eps)
    o = o * torch.nn.functional.silu(z.reshape(T, Hv, Dv))
    return o.reshape(T, Hv * Dv) @ w[pre + "out_proj.weight"].T


def attention_mixer(cfg: Qwen35Config, w: Dict[str, torch.Tensor], pre: str, n: torch.Tensor,
                    pos: torch.Tensor) -> torch.Tensor:
    T = n.shape[0]
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    qg = (n @ w[pre + "q_proj.weight"].T).reshape(T, Hq, 2 * D)
    q, gate = qg[..., :D], qg[..., D:]
    k = (n @ w[pre + "k_proj.weight"].T).reshape(T, Hkv, D)
    v = (n @ w[pre + "v_proj.weight"].T).reshape(T, Hkv, D)
    q = rms_norm_one_plus(q, w[pre + "q_norm.weight"], cfg.rms_norm_eps)
    k = rms_norm_one_plus(k, w[pre + "k_norm.weight"], cfg.rms_norm_eps)
    q = rope_neox_partial(q, pos, cfg.rotary_dim, cfg.rope_theta)
    k = rope_neox_partial(k, pos, cfg.rotary_dim, cfg.rope_theta)
    G = Hq // Hkv
    kk = k.repeat_interleave(G, 1)
    vv = v.repeat_interleave(G, 1)
    s = torch.einsum("thd,shd->hts", q, kk) * (D ** -0.5)
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, -1)
    ctx = torch.einsum("hts,shd->thd", p, vv)
    ctx = ctx * torch.sigmoid(gate)
    return ctx.reshape(T, Hq * D) @ w[pre + "o_proj.weight"].T


def reference_forward(cfg: Qwen35Config, weights: Dict[str, torch.Tensor], token_ids,
                      return_hidden_layers: Optional[List[int]] = None):
    """Logits [T, vocab] (fp32) for one sequence starting at position 0.

    With ``return_hidden_layers`` also returns the post-residual hidden state after each listed layer
    (the taps a block drafter is conditioned on).
    """
    w = {k: v.float() for k, v in weights.items()}
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    T = ids.shape[0]
    pos = torch.arange(T)
    x = w[P + "embed_tokens.weight"][ids]
    taps = {}
    for i, lt in enumerate(cfg.layer_types):
        lp = f"{P}layers.{i}."
        n = rms_norm_one_plus(x, w[lp + "input_layernorm.weight"], cfg.rms_norm_eps)
        if lt == 0:
            y = gdn_mixer(cfg, w, lp + "linear_attn.", n)
        else:
            y = attention_mixer(cfg, w, lp + "self_attn.", n, pos)
        r = y + x
        m = rms_norm_one_plus(r, w[lp + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
        mlp = (torch.nn.functional.silu(m @ w[lp + "mlp.gate_proj.weight"].T) * (m @ w[lp + "mlp.up_proj.weight"].T))
        x = mlp @ w[lp + "mlp.down_proj.weight"].T + r
        if return_hidden_layers and i in return_hidden_layers:
            taps[i] = x.clone()
    h = rms_norm_one_plus(x, w[P + "norm.weight"], cfg.rms_norm_eps)
    lm = w.get(P + "lm_head.weight", w.get("lm_head.weight"))
    if lm is None:
        lm = w[P + "embed_tokens.weight"]
    logits = h @ lm.T
    if return_hidden_layers:
        return logits, taps
    return logits


def reference_greedy(cfg: Qwen35Config, weights: Dict[str, torch.Tensor], prompt: List[int], max_new_tokens: int
                     ) -> List[int]:
    """Greedy continuation by full recomputation each step (ties -> lower token id, like the engine)."""
    ids = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        logits = reference_forward(cfg, weights, ids)[-1]
        tok = int(torch.argmax(logits))   # torch.argmax returns the first maximal index
        out.append(tok)
        ids.append(tok)
    return out
