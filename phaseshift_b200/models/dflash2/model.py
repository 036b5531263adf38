"""DFlash2 block drafter: config, weights and forward.

Architecture as documented by the reference (docs/developer/dflash2.md:46-127,221-318,363-416,496-568;
executor: src/phaseshift/models/qwen35/dflash2/executor.hip): a small non-causal transformer that, given
the target's tapped hidden states for the committed context and a block ``[anchor, MASK x K]``, proposes K
draft tokens in ONE forward pass.

* target bridge: ``tf = RMSNorm_direct(fc . concat(taps))`` per committed row; its K (per-head normed, RoPE'd)
  and V per layer are appended to a ring of ``sliding_window`` slots (slot = position % window);
* layer: norm -> grouped dynamic causal conv (prepare) -> q/k/v -> per-head norm on q,k -> RoPE ->
  non-causal attention over [ring context || block rows] with ``|pos_q - pos_k| < window`` -> o -> conv
  (finish) -> residual -> norm -> conv (prepare) -> SwiGLU -> conv (finish) -> residual;
* head: final norm -> ``hidden_projection`` -> logits through the TARGET's lm_head -> exact top-16 ->
  sequential candidate selector (``score_j = logit_j + <pred_cb[prev] * hproj_r, succ_cb[cand_j]>``).

The drafter borrows embedding and lm_head from the target.  This implementation runs on torch tensor ops
on any device (it is a few percent of a round's time; the verify forward of the target dominates); the
INT2 coarse head and the fixed draft-vocabulary profile of the reference are not built.
"""
from __future__ import annotations

import json
import zlib
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F


@dataclass
class DFlash2Config:
    vocab_size: int = 151936
    hidden_size: int = 5120
    intermediate_size: int = 17408
    num_hidden_layers: int = 5
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    sliding_window: int = 2048
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e7
    num_target_layers: int = 64
    block_size: int = 16
    conv_group_size: int = 128
    conv_kernel_size: int = 2
    mask_token_id: int = 0
    selector_rank: int = 64
    selector_top_k: int = 16
    target_layer_ids: List[int] = field(default_factory=lambda: [5, 19, 33, 47, 61])
    is_causal: bool = False
    tie_word_embeddings: bool = False

    def __post_init__(self):
        if self.is_causal:
            raise ValueError("DFlash2 drafter must be non-causal")
        if not (2 <= self.block_size <= 16):
            raise ValueError("block_size must be in [2, 16]")
        if self.conv_kernel_size != 2:
            raise ValueError("conv_kernel_size must be 2")
        t = self.target_layer_ids
        if not (1 <= len(t) <= 8) or any(b <= a for a, b in zip(t, t[1:])):
            raise ValueError("target_layer_ids must be 1..8 strictly increasing layer indices")
        if self.hidden_size % self.conv_group_size:
            raise ValueError("hidden_size must be a multiple of conv_group_size")

    @property
    def groups(self) -> int:
        return self.hidden_size // self.conv_group_size

    def save(self, d) -> None:
        Path(d).mkdir(parents=True, exist_ok=True)
        raw = asdict(self)
        dc = {k: raw.pop(k) for k in ("block_size", "conv_group_size", "conv_kernel_size", "mask_token_id", "selector_rank",
                                      "selector_top_k", "target_layer_ids")}
        raw["dflash_config"] = dc
        raw["architectures"] = ["DFlash2DraftModel"]
        (Path(d) / "config.json").write_text(json.dumps(raw, indent=1))

    @staticmethod
    def from_dir(d) -> "DFlash2Config":
        raw = json.loads((Path(d) / "config.json").read_text())
        if (raw.get("architectures") or [""])[0] != "DFlash2DraftModel":
            raise ValueError("not a DFlash2DraftModel directory")
        kw = {k: v for k, v in raw.items() if k in DFlash2Config.__dataclass_fields__}
        kw.update(raw.get("dflash_config", {}))
        return DFlash2Config(**kw)


def tiny_drafter_config(target_cfg, **over) -> DFlash2Config:
    taps = sorted({min(target_cfg.num_hidden_layers - 1, i) for i in (0, target_cfg.num_hidden_layers // 2,
                                                                     target_cfg.num_hidden_layers - 1)})
    kw = dict(vocab_size=target_cfg.vocab_size, hidden_size=target_cfg.hidden_size, intermediate_size=2 * target_cfg.hidden_size,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64, sliding_window=64,
              num_target_layers=target_cfg.num_hidden_layers, block_size=8, conv_group_size=32, mask_token_id=1,
              selector_rank=16, selector_top_k=8, target_layer_ids=taps)
    kw.update(over)
    return DFlash2Config(**kw)


def drafter_27b_config(**over) -> DFlash2Config:
    return DFlash2Config(**over)


def tensor_shapes(c: DFlash2Config) -> Dict[str, tuple]:
    h, i, D = c.hidden_size, c.intermediate_size, c.head_dim
    q, kv = c.num_attention_heads * D, c.num_key_value_heads * D
    s = {"fc.weight": (h, len(c.target_layer_ids) * h), "fc_norm.weight": (h,), "norm.weight": (h,),
         "selector.hidden_projection.weight": (c.selector_rank, h),
         "selector.pred_codebook": (c.vocab_size, c.selector_rank), "selector.succ_codebook": (c.vocab_size, c.selector_rank)}
    for l in range(c.num_hidden_layers):
        p = f"layers.{l}."
        s.update({p + "input_layernorm.weight": (h,), p + "post_attention_layernorm.weight": (h,),
                  p + "self_attn.q_proj.weight": (q, h), p + "self_attn.k_proj.weight": (kv, h),
                  p + "self_attn.v_proj.weight": (kv, h), p + "self_attn.o_proj.weight": (h, q),
                  p + "self_attn.q_norm.weight": (D,), p + "self_attn.k_norm.weight": (D,),
                  p + "mlp.gate_proj.weight": (i, h), p + "mlp.up_proj.weight": (i, h), p + "mlp.down_proj.weight": (h, i)})
        for cv in ("attn_conv", "mlp_conv"):
            s[p + cv + ".kernel_projection.weight"] = (2 * 2 * c.groups, h)       # [phase, offset, group]
            s[p + cv + ".base_kernel"] = (2, 2, h)                                 # [phase, offset, feature]
    return s


def random_weights(c: DFlash2Config, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
    out = {}
    for n, shp in tensor_shapes(c).items():
        g = torch.Generator(device=device)
        g.manual_seed((seed * 7919 + zlib.crc32(n.encode())) & 0x7FFFFFFF)
        if n.endswith("norm.weight"):
            t = 1.0 + 0.02 * torch.randn(shp, device=device, generator=g)
        elif n.endswith("base_kernel"):
            t = torch.zeros(shp, device=device)
            t[:, 0] = 1.0                                   # identity conv at init: offset 0 passes the row through
        elif "codebook" in n or "kernel_projection" in n:
            t = 0.01 * torch.randn(shp, device=device, generator=g)
        else:
            t = 0.02 * torch.randn(shp, device=device, generator=g)
        out[n] = t.to(torch.bfloat16)
    return out


def _rms(x, w, eps):
    """Direct-weight RMSNorm; the normalised value is rounded to the activation dtype before the weight
    multiply, as the reference documents for the drafter (docs/developer/dflash2.md:303-318)."""
    y = (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
    return y * w.to(x.dtype)


def _rope(x, pos, theta):
    """x [T, H, D], full-dim NeoX rotation; inv_freq in fp32, cos/sin rounded to the activation dtype."""
    D = x.shape[-1]
    inv = theta ** (-torch.arange(0, D, 2, dtype=torch.float32, device=x.device) / D)
    ang = pos.to(torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos().to(x.dtype)[:, None, :], ang.sin().to(x.dtype)[:, None, :]
    lo, hi = x[..., : D // 2], x[..., D // 2:]
    return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], -1)


class DFlash2Drafter:
    def __init__(self, cfg: DFlash2Config, weights: Dict[str, torch.Tensor], device, dtype=torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.w = {k: v.to(device=self.device, dtype=dtype) for k, v in weights.items()}
        c = cfg
        W = c.sliding_window
        kvf = c.num_key_value_heads * c.head_dim
        self.k_ring = torch.zeros(c.num_hidden_layers, W, kvf, device=self.device, dtype=dtype)
        self.v_ring = torch.zeros_like(self.k_ring)
        self.ring_pos = torch.full((W,), -1, dtype=torch.long, device=self.device)   # absolute position held by a slot
        self.context_len = 0
        self.use_graph = True          # CUDA devices: proposals replay a captured graph (see _propose_captured)
        self._graphs: Dict[int, tuple] = {}
        self.graph_error: Optional[str] = None

    @staticmethod
    def from_dir(d, device, dtype=torch.float32) -> "DFlash2Drafter":
        """Loads a BF16 drafter directory, or a bundle written by the offline quantizer's DFlash2 adapter
        (block-quantised backbone projections are expanded once at load: the drafter's products run in
        ``dtype``)."""
        from ...io.model_dir import ShardCollection, is_quantized_dir
        cfg = DFlash2Config.from_dir(d)
        col = ShardCollection(d)
        if not is_quantized_dir(d):
            w = {n: col.tensor(n).clone() for n in tensor_shapes(cfg)}
            return DFlash2Drafter(cfg, w, device, dtype)
        from ...quant import formats
        from ...quant.manifest import Manifest
        entries = Manifest.load(d).by_name()
        w = {}
        for n, shape in tensor_shapes(cfg).items():
            e = entries[n]
            if e.encoding == "bf16":
                w[n] = col.tensor(e.data).clone().reshape(shape)
            else:
                q = formats.QuantizedTensor(e.encoding, tuple(e.logical_shape), e.k_padded, col.tensor(e.codes),
                                            col.tensor(e.metadata1), e.metadata2 if e.metadata2 is not None else 1.0)
                w[n] = formats.dequantize(q).reshape(shape)
        return DFlash2Drafter(cfg, w, device, dtype)

    def save(self, d) -> None:
        from ...io.model_dir import ShardWriter
        self.cfg.save(d)
        wr = ShardWriter(d)
        ws = {k: v.to(torch.bfloat16).cpu() for k, v in self.w.items()}
        for n, t in ws.items():
            wr.add(n, t.dtype, t.shape)
        wr.begin()
        for n, t in ws.items():
            wr.write(n, t)
        wr.finish()

    def reset(self) -> None:
        self.ring_pos.fill_(-1)
        self.context_len = 0

    def snapshot(self):
        """The context ring as of now (clones): what a prefix-cache entry keeps beside the target's state, so that a
        restored prefix can be drafted from at once (reference: docs/developer/prefix_cache.md:27-47)."""
        return (self.k_ring.clone(), self.v_ring.clone(), self.ring_pos.clone(), self.context_len)

    def restore(self, snap) -> None:
        k, v, p, n = snap
        self.k_ring.copy_(k)
        self.v_ring.copy_(v)
        self.ring_pos.copy_(p)
        self.context_len = n

    # ------------------------------------------------------------------ pieces
    def _conv(self, x, prefix: str, phase: int, dyn=None):
        """Grouped dynamic causal conv over the block rows (kernel 2, block-local, zero left padding).
        Returns (out, dyn) where dyn is the per-row dynamic kernel computed at phase 0 and re-used at phase 1."""
        c = self.cfg
        if dyn is None:
            dyn = (x @ self.w[prefix + ".kernel_projection.weight"].T).reshape(x.shape[0], 2, 2, c.groups)
        base = self.w[prefix + ".base_kernel"]                                  # [2, 2, H]
        k = base[phase][None] + dyn[:, phase].repeat_interleave(c.conv_group_size, -1)   # [T, 2(offset), H]
        prev = torch.cat([torch.zeros_like(x[:1]), x[:-1]], 0)
        return k[:, 0] * x + k[:, 1] * prev, dyn

    def target_feature(self, taps: Sequence[torch.Tensor]) -> torch.Tensor:
        cat = torch.cat([t.to(self.dtype) for t in taps], -1)
        return _rms(cat @ self.w["fc.weight"].T, self.w["fc_norm.weight"], self.cfg.rms_norm_eps)

    def append_context(self, taps: Sequence[torch.Tensor], pos_start: int) -> None:
        """Append committed target rows (their tapped hidden states) to every layer's K/V ring."""
        c = self.cfg
        n = taps[0].shape[0]
        if n == 0:
            return
        tf = self.target_feature(taps)
        pos = torch.arange(pos_start, pos_start + n, device=self.device)
        slots = pos % c.sliding_window
        for l in range(c.num_hidden_layers):
            p = f"layers.{l}.self_attn."
            k = (tf @ self.w[p + "k_proj.weight"].T).reshape(n, c.num_key_value_heads, c.head_dim)
            v = tf @ self.w[p + "v_proj.weight"].T
            k = _rope(_rms(k, self.w[p + "k_norm.weight"], c.rms_norm_eps), pos, c.rope_theta)
            self.k_ring[l, slots] = k.reshape(n, -1)
            self.v_ring[l, slots] = v
        self.ring_pos[slots] = pos
        self.context_len = pos_start + n

    def backbone(self, x: torch.Tensor, pos: torch.Tensor, static: bool = False) -> torch.Tensor:
        """``static``: attend over every ring slot and mask the empty ones instead of compacting the live slots, so
        that all shapes are fixed and the call can be captured in a CUDA graph (same mathematics)."""
        c = self.cfg
        T = x.shape[0]
        G = c.num_attention_heads // c.num_key_value_heads
        if static:
            live = None
            ctx_pos = self.ring_pos
        else:
            live = torch.nonzero(self.ring_pos >= 0).squeeze(1)   # one host synchronisation per call, none per layer
            ctx_pos = self.ring_pos.index_select(0, live)
        for l in range(c.num_hidden_layers):
            p = f"layers.{l}."
            n = _rms(x, self.w[p + "input_layernorm.weight"], c.rms_norm_eps)
            a, dyn = self._conv(n, p + "attn_conv", 0)
            q = (a @ self.w[p + "self_attn.q_proj.weight"].T).reshape(T, c.num_attention_heads, c.head_dim)
            kn = (a @ self.w[p + "self_attn.k_proj.weight"].T).reshape(T, c.num_key_value_heads, c.head_dim)
            vn = (a @ self.w[p + "self_attn.v_proj.weight"].T).reshape(T, c.num_key_value_heads, c.head_dim)
            q = _rope(_rms(q, self.w[p + "self_attn.q_norm.weight"], c.rms_norm_eps), pos, c.rope_theta)
            kn = _rope(_rms(kn, self.w[p + "self_attn.k_norm.weight"], c.rms_norm_eps), pos, c.rope_theta)
            kc = (self.k_ring[l] if static else self.k_ring[l].index_select(0, live)).reshape(-1, c.num_key_value_heads, c.head_dim)
            vc = (self.v_ring[l] if static else self.v_ring[l].index_select(0, live)).reshape(-1, c.num_key_value_heads, c.head_dim)
            K = torch.cat([kc, kn], 0).repeat_interleave(G, 1)
            V = torch.cat([vc, vn], 0).repeat_interleave(G, 1)
            kpos = torch.cat([ctx_pos, pos], 0)
            s = torch.einsum("thd,shd->hts", q.float(), K.float()) * (c.head_dim ** -0.5)
            ok = ((pos[:, None] - kpos[None, :]).abs() < c.sliding_window) & (kpos >= 0)[None, :]   # non-causal window
            s = s.masked_fill(~ok[None], float("-inf"))
            att = torch.einsum("hts,shd->thd", torch.softmax(s, -1), V.float()).to(x.dtype)
            o = att.reshape(T, -1) @ self.w[p + "self_attn.o_proj.weight"].T
            o, _ = self._conv(o, p + "attn_conv", 1, dyn)
            x = x + o
            m = _rms(x, self.w[p + "post_attention_layernorm.weight"], c.rms_norm_eps)
            m, dyn2 = self._conv(m, p + "mlp_conv", 0)
            g = F.silu(m @ self.w[p + "mlp.gate_proj.weight"].T).to(x.dtype)
            d = (g * (m @ self.w[p + "mlp.up_proj.weight"].T)) @ self.w[p + "mlp.down_proj.weight"].T
            d, _ = self._conv(d, p + "mlp_conv", 1, dyn2)
            x = x + d
        return _rms(x, self.w["norm.weight"], c.rms_norm_eps)

    # ------------------------------------------------------------------ proposal
    def propose(self, anchor: int, k: int, embed, lm_head_logits, pos_start: int, allowed=None) -> List[int]:
        """``embed(ids)`` -> [n, H] target embeddings, ``lm_head_logits(h)`` -> [n, vocab] fp32 target-head logits."""
        c = self.cfg
        # one graph, for the draft count the decoder normally asks for; the shorter proposals at the end of a request
        # run eagerly (a capture costs more than the handful of calls it would serve)
        if self.device.type == "cuda" and allowed is None and self.use_graph and k >= 1 and (not self._graphs or k in self._graphs):
            try:
                return self._propose_captured(anchor, k, embed, lm_head_logits, pos_start)
            except RuntimeError as e:                  # capture refused (e.g. an op that synchronises): stay eager
                self.use_graph, self.graph_error = False, str(e)
                torch.cuda.synchronize(self.device)
        ids = torch.tensor([anchor] + [c.mask_token_id] * k, device=self.device)
        x = embed(ids).to(self.dtype)
        pos = torch.arange(pos_start, pos_start + k + 1, device=self.device)
        h = self.backbone(x, pos)[1:]                      # draft rows only
        logits = lm_head_logits(h).float()
        if allowed is not None:
            logits = logits.masked_fill(~allowed, float("-inf"))
        return self.select(h, logits, anchor)

    def _propose_captured(self, anchor: int, k: int, embed, lm_head_logits, pos_start: int) -> List[int]:
        """The whole proposal (embedding, backbone over the full ring, target head, top-k, selector chain) as one CUDA
        graph per draft count: a proposal is a few hundred small launches, so eager dispatch costs more than the math.
        Inputs live in fixed tensors (token ids, positions); the K/V ring and its position table are updated in place
        between replays by ``append_context``."""
        st = self._graphs.get(k)
        if st is None:
            c = self.cfg
            ids = torch.full((k + 1,), c.mask_token_id, dtype=torch.long, device=self.device)
            base = torch.arange(k + 1, device=self.device)
            pos = torch.zeros(k + 1, dtype=torch.long, device=self.device)

            def run():
                x = embed(ids).to(self.dtype)
                h = self.backbone(x, pos, static=True)[1:]
                return self.select_device(h, lm_head_logits(h).float(), ids[0])
            ids[0] = anchor
            torch.add(base, pos_start, out=pos)
            cur = torch.cuda.current_stream(self.device)
            side = torch.cuda.Stream(self.device)
            side.wait_stream(cur)
            with torch.cuda.stream(side):                 # warm-up off the capture: workspaces get allocated here
                for _ in range(2):
                    run()
            cur.wait_stream(side)
            from ...utils.graphs import capture as capture_graph
            graph, out = capture_graph(self.device, run)
            st = (graph, ids, base, pos, out)
            self._graphs[k] = st
        graph, ids, base, pos, out = st
        ids[0] = anchor
        torch.add(base, pos_start, out=pos)
        graph.replay()
        return out.tolist()

    def select(self, h: torch.Tensor, logits: torch.Tensor, anchor: int) -> List[int]:
        picks = self.select_device(h, logits, torch.tensor(anchor, device=logits.device))
        return picks.tolist() if picks is not None else []

    def select_device(self, h: torch.Tensor, logits: torch.Tensor, prev: torch.Tensor):
        """Exact top-k (logit desc, id asc) then the sequential candidate selector chain.  The chain runs on the
        device without reading intermediate winners back: one host synchronisation per proposal."""
        c = self.cfg
        kk = min(c.selector_top_k, logits.shape[-1])
        topk = getattr(self, "topk_fn", None)
        if topk is not None and logits.is_cuda and logits.dtype == torch.float32 and kk <= 128:
            order, top_l = topk(logits.contiguous(), kk)          # radix top-k kernel: same tie rule
            order, top_l = order.long(), top_l.clone()
        else:
            # stable tie rule: higher logit first, lower id first among equals
            order = torch.argsort(logits, dim=-1, descending=True, stable=True)[:, :kk]
            top_l = torch.gather(logits, 1, order)
        hproj = (h @ self.w["selector.hidden_projection.weight"].T).float()     # [K, rank]
        pred, succ = self.w["selector.pred_codebook"], self.w["selector.succ_codebook"]
        # Every index below is a one-element tensor used through index_select: indexing with a zero-dimensional
        # tensor would read it back to the host (a synchronisation per step, and illegal during graph capture).
        prev = prev.reshape(1)
        picks = []
        for r in range(h.shape[0]):
            cand = order[r]
            score = top_l[r] + (pred.index_select(0, prev)[0].float() * hproj[r]) @ succ.index_select(0, cand).float().T
            j = torch.argmax(score).reshape(1)             # first maximal index = best-ranked candidate on ties
            prev = cand.index_select(0, j)
            picks.append(prev)
        return torch.cat(picks) if picks else None
