"""DFlash2 drafter on the engine's own CUDA kernels.

Same interface and the same mathematics as ``DFlash2Drafter`` (model.py), built the way the reference builds its
drafter (src/phaseshift/models/qwen35/dflash2/executor.hip: one executor that owns the ring, the workspaces and the
launch order; kernels under src/phaseshift/models/qwen35/kernels/dflash2/):

* every projection runs on the block-scaled tcgen05 kernel through ``CudaOps.linear`` -- backbone projections are
  quantised to NVFP4 at load (the reference's drafter preset), q|k|v and gate|up are fused into one projection each,
  and the per-layer context K/V projections of all layers are ONE projection of the target feature;
* everything else is the block kernels of csrc/kernels/dflash2.cu;
* a proposal makes no host synchronisation: token ids, positions and the anchor live on the device, the launch
  sequence is captured in one CUDA graph per draft count, and the proposed tokens stay on the device for the
  verification step to read (``propose_device``).

Embedding table and lm_head are the target's.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence

import torch

from ...ops import _lib
from ...ops._lib import c_float, c_int, ptr
from ...quant.act_quant import calibrate_act_scale
from ...quant.formats import quantize, to_kernel_format
from ...utils.graphs import capture as capture_graph
from ..qwen35.weights import LinearW
from .model import DFlash2Config, tensor_shapes

MAX_BLOCK_ROWS = 16


class DFlash2NativeDrafter:
    native = True

    def __init__(self, cfg: DFlash2Config, weights: Dict[str, torch.Tensor], engine, fmt: str = "nvfp4"):
        """``weights``: full-precision tensors by the names of ``tensor_shapes``; ``fmt``: storage format of the
        backbone projections (``nvfp4`` | ``mxfp8`` | ``bf16``)."""
        if engine.device.type != "cuda" or not hasattr(engine.ops, "linear_bs"):
            raise ValueError("the native drafter needs an engine on the CUDA op set")
        c = cfg
        if c.head_dim != 128 or MAX_BLOCK_ROWS * (c.num_attention_heads // c.num_key_value_heads) > 64:
            raise ValueError("ring attention kernel: head_dim 128 and at most 4 query heads per KV head")
        self.cfg, self.eng, self.ops, self.device, self.fmt = cfg, engine, engine.ops, engine.device, fmt
        dev = self.device
        bf = lambda n: weights[n].to(device=dev, dtype=torch.bfloat16).contiguous()
        self.H, self.q_dim, self.kv_dim = c.hidden_size, c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim

        def lin(w: torch.Tensor, f: Optional[str] = None) -> LinearW:
            f = f or fmt
            lw = LinearW(to_kernel_format(quantize(w.to(device=dev, dtype=torch.float32), f)))
            if f in ("nvfp4", "mxfp8"):
                lw.make_umma()
            return lw

        def interleave(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
            return torch.stack([a, b], 1).reshape(2 * a.shape[0], a.shape[1])

        self.fc = lin(weights["fc.weight"])
        self.fc_norm, self.final_norm = bf("fc_norm.weight"), bf("norm.weight")
        # tiny projections (dynamic conv taps: 4 * groups outputs; selector projection: rank outputs) stay bf16 and run
        # inside the fused norm kernel (ps_dfl_norm_proj4) when their shape fits it, else as separate projections
        self.fused_small = (c.selector_rank % 4 == 0 and c.hidden_size % (c.selector_rank // 4) == 0
                            and (c.hidden_size // (c.selector_rank // 4)) % 2 == 0 and c.conv_group_size % 2 == 0
                            and c.hidden_size % 8 == 0)
        small = "bf16"
        self.hidden_projection = lin(weights["selector.hidden_projection.weight"], small)
        self.hproj_w = bf("selector.hidden_projection.weight")
        self.pred_cb, self.succ_cb = bf("selector.pred_codebook"), bf("selector.succ_codebook")
        self.layers = []
        kv_ctx, k_norms = [], []
        for l in range(c.num_hidden_layers):
            p = f"layers.{l}."
            a = p + "self_attn."
            L = dict(
                in_norm=bf(p + "input_layernorm.weight"), post_norm=bf(p + "post_attention_layernorm.weight"),
                qkv=lin(torch.cat([weights[a + "q_proj.weight"], weights[a + "k_proj.weight"], weights[a + "v_proj.weight"]], 0)),
                o=lin(weights[a + "o_proj.weight"]), q_norm=bf(a + "q_norm.weight"), k_norm=bf(a + "k_norm.weight"),
                gate_up=lin(interleave(weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"])),
                down=lin(weights[p + "mlp.down_proj.weight"]),
                attn_kproj=lin(weights[p + "attn_conv.kernel_projection.weight"], small),
                mlp_kproj=lin(weights[p + "mlp_conv.kernel_projection.weight"], small),
                attn_kproj_w=bf(p + "attn_conv.kernel_projection.weight"), mlp_kproj_w=bf(p + "mlp_conv.kernel_projection.weight"),
                attn_base=bf(p + "attn_conv.base_kernel"), mlp_base=bf(p + "mlp_conv.base_kernel"))
            self.layers.append(L)
            kv_ctx += [weights[a + "k_proj.weight"], weights[a + "v_proj.weight"]]
            k_norms.append(bf(a + "k_norm.weight"))
        self.kv_ctx = lin(torch.cat(kv_ctx, 0))                     # [layers * 2 * kv_dim, H]: context K | V of every layer
        self.k_norms = torch.stack(k_norms).contiguous()            # [layers, D]
        W = c.sliding_window
        self.k_ring = torch.zeros(c.num_hidden_layers, W, self.kv_dim, device=dev, dtype=torch.bfloat16)
        self.v_ring = torch.zeros_like(self.k_ring)
        self.ring_pos = torch.full((W,), -1, dtype=torch.int32, device=dev)
        self.context_len = 0
        self.ids = torch.zeros(MAX_BLOCK_ROWS, dtype=torch.int32, device=dev)
        self.pos = torch.zeros(MAX_BLOCK_ROWS, dtype=torch.int32, device=dev)
        self.ctl = torch.zeros(2, dtype=torch.int32, device=dev)                 # anchor token, first block position
        self.h_ctl = torch.zeros(2, dtype=torch.int32, pin_memory=True)
        self.tokens = torch.zeros(MAX_BLOCK_ROWS, dtype=torch.int32, device=dev)
        self.use_graph = True
        self.sub_head: Optional[LinearW] = None       # draft-vocabulary head (rows of the target's lm_head) + id map
        self.idmap: Optional[torch.Tensor] = None
        self._graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self._calibrated = {"ctx": fmt != "nvfp4", "blk": fmt != "nvfp4"}
        self._collect: Optional[Dict[int, float]] = None
        self.launches = 0
        self.graph_launches: Dict[int, int] = {}

    # ------------------------------------------------------------------ construction helpers
    @staticmethod
    def from_dir(d, engine, fmt: str = "nvfp4") -> "DFlash2NativeDrafter":
        """Loads a BF16 drafter directory or a quantised bundle (expanded, then stored in ``fmt``)."""
        from .model import DFlash2Drafter
        t = DFlash2Drafter.from_dir(d, "cpu", torch.float32)
        return DFlash2NativeDrafter(t.cfg, t.w, engine, fmt)

    @staticmethod
    def from_torch(drafter, engine, fmt: str = "nvfp4") -> "DFlash2NativeDrafter":
        return DFlash2NativeDrafter(drafter.cfg, drafter.w, engine, fmt)

    def set_draft_vocab(self, ids) -> None:
        """Restrict the drafter's head to the given target token ids (ascending; models/dflash2/draft_vocab.py): the
        head pass streams only those rows of the target's lm_head, top-k runs on local ids and is mapped back to global
        ids before the selector.  ``None`` restores the full vocabulary.  Captured proposals are dropped."""
        self._graphs.clear()
        if ids is None:
            self.sub_head = self.idmap = None
            return
        from ...quant.act_quant import pack_sf_atoms, unpack_sf_atoms
        from ...quant.formats import QuantizedTensor
        head = self.eng.runner.w.lm_head
        idx = torch.as_tensor([int(i) for i in ids], dtype=torch.long, device=self.device)
        if head.fmt == "bf16":
            q = QuantizedTensor("bf16", (idx.numel(), head.K), head.K, head.q.codes.index_select(0, idx).contiguous(), None, 1.0)
            sub = LinearW(q)
        else:
            if head.sf_atoms is None:
                raise ValueError("the draft-vocabulary head needs the target's lm_head in the tensor-core layout")
            blk = 16 if head.fmt == "nvfp4" else 32
            scales = unpack_sf_atoms(head.sf_atoms, head.N, head.k_padded // blk).index_select(0, idx).contiguous()
            q = QuantizedTensor(head.fmt, (idx.numel(), head.K), head.k_padded, head.codes.index_select(0, idx).contiguous(),
                                scales, head.tensor_scale)
            sub = LinearW(q).make_umma(keep_canonical=True)
            sub.act_scale = head.act_scale
        self.sub_head, self.idmap = sub, idx.to(torch.int32).contiguous()

    def weight_bytes(self) -> int:
        n = sum(L[k].nbytes for L in self.layers for k in ("qkv", "o", "gate_up", "down", "attn_kproj", "mlp_kproj"))
        return n + self.fc.nbytes + self.kv_ctx.nbytes + self.hidden_projection.nbytes

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

    # ------------------------------------------------------------------ op wrappers
    def _linear(self, x: torch.Tensor, W: LinearW, name: str, **kw) -> torch.Tensor:
        if self._collect is not None:
            self._collect[id(W)] = max(self._collect.get(id(W), 0.0), float(x.float().abs().max()))
        return self.ops.linear(x, W, name="dfl_" + name, **kw)

    def _finish_calibration(self, which: str) -> None:
        seen = self._collect or {}
        for W in self._all_linears():
            if id(W) in seen and W.fmt == "nvfp4":
                W.act_scale = calibrate_act_scale(seen[id(W)])
        self._collect = None
        self._calibrated[which] = True

    def _all_linears(self):
        yield from (self.fc, self.kv_ctx, self.hidden_projection)
        for L in self.layers:
            yield from (L["qkv"], L["o"], L["gate_up"], L["down"], L["attn_kproj"], L["mlp_kproj"])

    def _rms(self, x: torch.Tensor, w: torch.Tensor, name: str) -> torch.Tensor:
        out = self.ops.buf("dfl_" + name, x.shape[0], x.shape[1])
        _lib.call("ps_dfl_rmsnorm", ptr(x), c_int(x.stride(0)), ptr(w), c_float(self.cfg.rms_norm_eps), c_int(x.shape[0]),
                  c_int(x.shape[1]), ptr(out), c_int(out.stride(0)))
        self.launches += 1
        return out

    def _conv(self, x: torch.Tensor, dyn: torch.Tensor, base: torch.Tensor, phase: int, name: str,
              residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = self.ops.buf("dfl_" + name, x.shape[0], x.shape[1])
        _lib.call("ps_dfl_conv_apply", ptr(x), c_int(x.stride(0)), ptr(dyn), c_int(dyn.stride(0)), ptr(base), c_int(phase),
                  c_int(x.shape[0]), c_int(x.shape[1]), c_int(self.cfg.groups), ptr(residual),
                  c_int(residual.stride(0) if residual is not None else 0), ptr(out), c_int(out.stride(0)))
        self.launches += 1
        return out

    def _norm_proj4(self, x: torch.Tensor, norm_w: torch.Tensor, wp: torch.Tensor, C: int, mode: int, base, name: str):
        """Fused RMSNorm + 4C-output projection + (mode 1) conv prepare / (mode 0) normalised rows.  Returns (y, proj)."""
        T, H = x.shape
        y = self.ops.buf("dfl_" + name, T, H)
        proj = self.ops.buf("dfl_" + name + "_p", T, 4 * C, torch.bfloat16 if mode == 1 else torch.float32)
        _lib.call("ps_dfl_norm_proj4", ptr(x), c_int(x.stride(0)), ptr(norm_w), c_float(self.cfg.rms_norm_eps), ptr(wp), c_int(C), c_int(T),
                  c_int(H), c_int(mode), ptr(base), ptr(proj), c_int(proj.stride(0)), ptr(y), c_int(y.stride(0)))
        self.launches += 1
        return y, proj

    def _attn_workspace(self, T: int) -> torch.Tensor:
        L = _lib.lib()
        L.ps_dfl_ring_attention_workspace_floats.restype = ctypes.c_longlong
        n = int(L.ps_dfl_ring_attention_workspace_floats(c_int(T), c_int(self.cfg.sliding_window), c_int(self.cfg.num_key_value_heads)))
        return self.ops.buf("dfl_attn_part", n // 132, 132, torch.float32)

    # ------------------------------------------------------------------ context
    def target_feature(self, taps: Sequence[torch.Tensor], cat: Optional[torch.Tensor] = None) -> torch.Tensor:
        c = self.cfg
        if cat is None:
            n = taps[0].shape[0]
            cat = self.ops.buf("dfl_cat", n, len(taps) * self.H)
            srcs = (ctypes.c_void_p * len(taps))(*[t.data_ptr() for t in taps])
            lds = (ctypes.c_int * len(taps))(*[t.stride(0) for t in taps])
            _lib.call("ps_dfl_feature_concat", srcs, lds, c_int(len(taps)), c_int(n), c_int(self.H), ptr(cat))
            self.launches += 1
        raw = self._linear(cat, self.fc, "fc")
        return self._rms(raw, self.fc_norm, "tf")

    def append_context(self, taps: Sequence[torch.Tensor], pos_start: int, cat: Optional[torch.Tensor] = None,
                       ctl: Optional[torch.Tensor] = None) -> None:
        """Append committed target rows to every layer's ring.  ``taps``: the tapped hidden states, bf16 [n, H] each
        (``cat``: the same rows already side by side, [n, taps * H], when the target step wrote them that way).
        ``ctl`` (int32[4] on the device: {-, rows to keep, -, first position}): only the first ctl[1] of the given rows
        are appended, starting at position ctl[3]; the launch sequence then depends on nothing the host knows only
        after a read-back, so it can sit in a captured graph (``pos_start`` is ignored; the caller tracks the length)."""
        c = self.cfg
        n = taps[0].shape[0] if cat is None else cat.shape[0]
        if n == 0:
            return
        if n > c.sliding_window:                       # two rows of one call must never share a slot
            cut = n - c.sliding_window
            taps = [t[cut:] for t in taps]
            cat = cat[cut:] if cat is not None else None
            pos_start, n = pos_start + cut, c.sliding_window
        collecting = not self._calibrated["ctx"]
        if collecting:
            self._collect = {}
        taps = [t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16) for t in taps]
        tf = self.target_feature(taps, cat)
        kv = self._linear(tf, self.kv_ctx, "kv_ctx")
        _lib.call("ps_dfl_kv_ring_append", ptr(kv), c_int(kv.stride(0)), c_int(c.num_hidden_layers), c_int(c.num_key_value_heads),
                  c_int(c.head_dim), ptr(self.k_norms), c_float(c.rms_norm_eps), c_int(pos_start), c_int(c.sliding_window),
                  c_float(c.rope_theta), c_int(n), ptr(self.k_ring), ptr(self.v_ring), ptr(self.ring_pos), ptr(ctl))
        self.launches += 1
        if ctl is None:
            self.context_len = pos_start + n
        if collecting:
            self._finish_calibration("ctx")

    # ------------------------------------------------------------------ block forward
    def _block(self, k: int) -> torch.Tensor:
        """The launch sequence of one proposal of k drafts; reads ``ctl``, leaves the tokens in ``self.tokens[:k]``."""
        c, ops, eng = self.cfg, self.ops, self.eng
        T = k + 1
        _lib.call("ps_dfl_noise_ids", ptr(self.ctl), c_int(c.mask_token_id), c_int(k), ptr(self.ids), ptr(self.pos))
        table = eng.runner.w.embed
        x = ops.buf("dfl_x", T, self.H)
        if table.fmt == "bf16":
            _lib.call("ps_embedding", ptr(self.ids), ptr(table.q.codes), c_int(T), c_int(table.N), c_int(self.H), ptr(x),
                      c_int(self.H), ptr(eng.state.status), ptr(None), c_int(0))
        else:
            _lib.call("ps_embedding_mxfp8", ptr(self.ids), ptr(table.q.codes), ptr(table.q.scales), c_int(T), c_int(table.N),
                      c_int(self.H), ptr(x), c_int(self.H), ptr(eng.state.status), ptr(None), c_int(0))
        self.launches += 2
        qd, kvd, D = self.q_dim, self.kv_dim, c.head_dim
        hq, hkv = c.num_attention_heads, c.num_key_value_heads
        for l, L in enumerate(self.layers):
            if self.fused_small:
                a, dyn = self._norm_proj4(x, L["in_norm"], L["attn_kproj_w"], c.groups, 1, L["attn_base"], "a")
            else:
                n = self._rms(x, L["in_norm"], "n")
                dyn = self._linear(n, L["attn_kproj"], "dyn_a")
                a = self._conv(n, dyn, L["attn_base"], 0, "a")
            qkv = self._linear(a, L["qkv"], "qkv")
            # per-head norm + RoPE of the q and k heads in place (v untouched)
            _lib.call("ps_dfl_headnorm_rope", ptr(qkv), c_int(qkv.stride(0)), c_int(hq + hkv), c_int(D), ptr(L["q_norm"]), c_int(hq),
                      ptr(L["k_norm"]), c_float(c.rms_norm_eps), ptr(self.pos), c_float(c.rope_theta), c_int(T), ptr(qkv),
                      c_int(qkv.stride(0)))
            att = ops.buf("dfl_att", T, qd)
            part = self._attn_workspace(T)
            _lib.call("ps_dfl_ring_attention", ptr(qkv), c_int(qkv.stride(0)), ptr(qkv[:, qd:]), ptr(qkv[:, qd + kvd:]),
                      c_int(qkv.stride(0)), ptr(self.k_ring[l]), ptr(self.v_ring[l]), ptr(self.ring_pos), ptr(self.pos), c_int(T),
                      c_int(c.sliding_window), c_int(hq), c_int(hkv), c_int(D), c_float(D ** -0.5), ptr(att), c_int(att.stride(0)),
                      ptr(part))
            self.launches += 3
            o = self._linear(att, L["o"], "o")
            x = self._conv(o, dyn, L["attn_base"], 1, "x", residual=x, out=x)
            if self.fused_small:
                m2, dyn2 = self._norm_proj4(x, L["post_norm"], L["mlp_kproj_w"], c.groups, 1, L["mlp_base"], "m2")
            else:
                m = self._rms(x, L["post_norm"], "m")
                dyn2 = self._linear(m, L["mlp_kproj"], "dyn_m")
                m2 = self._conv(m, dyn2, L["mlp_base"], 0, "m2")
            act = self._linear(m2, L["gate_up"], "act", swiglu=True)
            d = self._linear(act, L["down"], "d")
            x = self._conv(d, dyn2, L["mlp_base"], 1, "x", residual=x, out=x)
        if self.fused_small:
            hn, hp = self._norm_proj4(x, self.final_norm, self.hproj_w, c.selector_rank // 4, 0, None, "h")
            h, hproj = hn[1:T], hp[1:T]                                   # draft rows
        else:
            h = self._rms(x, self.final_norm, "h")[1:T]
            hproj = self._linear(h, self.hidden_projection, "hproj", out_f32=True)
        head = self.sub_head if self.sub_head is not None else eng.runner.w.lm_head
        logits = ops.linear(h, head, name="dfl_logits", out_f32=True)
        kk = min(c.selector_top_k, logits.shape[1])
        top_ids, top_vals = ops.topk(logits, kk)
        if self.idmap is not None:
            _lib.call("ps_dfl_remap_ids", ptr(top_ids), c_int(top_ids.numel()), ptr(self.idmap), c_int(self.idmap.numel()))
            self.launches += 1
        _lib.call("ps_dfl_select", ptr(top_ids), ptr(top_vals), c_int(kk), ptr(hproj), c_int(c.selector_rank), ptr(self.pred_cb),
                  ptr(self.succ_cb), ptr(self.ids), c_int(0), c_int(k), c_int(c.vocab_size), ptr(self.tokens))
        self.launches += 1
        self.last_logits, self.last_hidden = logits, h
        return self.tokens[:k]

    def propose_device(self, anchor: int, k: int, pos_start: int) -> torch.Tensor:
        """k draft tokens as an int32 device tensor; nothing is read back."""
        if not (1 <= k < MAX_BLOCK_ROWS):
            raise ValueError("1 <= k <= 15")
        self.h_ctl[0], self.h_ctl[1] = int(anchor), int(pos_start)
        self.ctl.copy_(self.h_ctl, non_blocking=True)
        if not self._calibrated["blk"]:
            self._collect = {}
            self._block(k)
            self._finish_calibration("blk")
        if not self.use_graph:
            return self._block(k)
        g = self._graphs.get(k)
        if g is None:
            self._block(k)                                # warm-up: workspaces, kernel attributes
            torch.cuda.current_stream().synchronize()
            n0 = self.launches
            g, _ = capture_graph(self.device, lambda: self._block(k))
            self._graphs[k] = g
            self.graph_launches[k] = self.launches - n0   # kernels in one proposal graph
        g.replay()
        return self.tokens[:k]

    def propose(self, anchor: int, k: int, embed=None, lm_head_logits=None, pos_start: int = 0, allowed=None) -> List[int]:
        if allowed is not None:
            raise ValueError("constrained proposals are served by the torch drafter")
        return self.propose_device(anchor, k, pos_start).tolist()
