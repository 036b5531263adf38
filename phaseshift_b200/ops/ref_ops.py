"""Reference op set in plain PyTorch (fp32, any device): the engine's correctness backend.

It implements exactly the same op contract as :class:`CudaOps` (paged KV through block tables, ring
conv history, per-slot recurrent state, batch descriptors) with straightforward tensor code, the role
the reference gives its single correctness mega-kernel
(src/phaseshift/models/qwen35/kernels/correctness/model_dispatch_correctness.hip:59): it is the
bit-reference for end-to-end token exactness on CPU and lets scheduler, batcher, prefix cache,
speculative decoding and tensor-parallel logic be tested without a GPU.
"""
from __future__ import annotations

from typing import Optional

import torch

from .trace import OpTrace
import torch.nn.functional as F

from ..models.qwen35.config import Qwen35Config
from ..models.qwen35.weights import AttnW, GdnW, LinearW
from ..runtime.batch import StepBatch
from ..runtime.state import GdnLayerState, KVLayer, ModelState
from ..utils.sampling import sample_row_host


class RefOps(OpTrace):
    act_dtype = torch.float32
    name = "ref"

    def __init__(self, cfg: Qwen35Config, device, act_quant: bool = False, **_):
        """``act_quant``: quantise the input of every block-quantised projection to the weights' block format
        (quant/act_quant.py), the arithmetic of the CUDA tensor-core layout; off = bf16/fp32 activations, the
        arithmetic of the streaming layout."""
        self.cfg, self.device = cfg, device
        self.act_quant = act_quant
        half = cfg.rotary_dim // 2
        self.inv_freq = cfg.rope_theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / cfg.rotary_dim)
        self.launches = 0
        self.exact_rows = False

    def _dense(self, W: LinearW) -> torch.Tensor:
        return W.dense().to(self.device)

    def embed(self, b: StepBatch, rows: int, table: LinearW, status, ssq_out=None) -> torch.Tensor:
        return self._dense(table)[b.ids[:rows].long()]

    def linear(self, x, W: LinearW, *, name: str, norm_w=None, eps: float = 0.0, residual=None, swiglu=False,
               out_f32=False, out=None, ssq_in=None, ssq_out=None, prefetch=None, **_):
        x = x.float()
        if self.act_quant and W.fmt in ("nvfp4", "mxfp8"):
            # the tensor-core layout's arithmetic: quantise x (1 + w), apply the row factor 1/rms after the product
            from ..quant.act_quant import fake_quant
            inv = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) if norm_w is not None else None
            if norm_w is not None:
                x = x * (1.0 + norm_w.float())
            y = fake_quant(x, W.fmt, W.act_scale) @ self._dense(W).T
            if inv is not None:
                y = y * inv
        else:
            if norm_w is not None:
                x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + norm_w.float())
            y = x @ self._dense(W).T
        if swiglu:
            y = F.silu(y[:, 0::2]) * y[:, 1::2]
        if residual is not None:
            y = y + residual.float()
        if out is not None:
            out.copy_(y)
            return out
        return y

    def attn_prep(self, qkv, aw: AttnW, hq: int, hkv: int, b: StepBatch, kv: KVLayer, st: ModelState):
        cfg = self.cfg
        rows, D = qkv.shape[0], cfg.head_dim
        qg = qkv[:, :2 * hq * D].reshape(rows, hq, 2 * D)
        q = qg[..., :D]
        k = qkv[:, 2 * hq * D: 2 * hq * D + hkv * D].reshape(rows, hkv, D)
        v = qkv[:, 2 * hq * D + hkv * D:].reshape(rows, hkv, D)
        eps = cfg.rms_norm_eps
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + aw.q_norm.float())
        k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + aw.k_norm.float())
        pos = b.row_pos[:rows]
        half = cfg.rotary_dim // 2
        ang = pos.to(torch.float64)[:, None] * self.inv_freq.to(pos.device)[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

        def rope(t):
            t = t.clone()
            lo, hi = t[..., :half].double(), t[..., half:2 * half].double()
            t[..., :half] = (lo * cos - hi * sin).float()
            t[..., half:2 * half] = (hi * cos + lo * sin).float()
            return t
        q, k = rope(q), rope(k)
        pt = st.sc.page_tokens
        for r in range(rows):
            slot, p = int(b.row_slot[r]), int(pos[r])
            if slot < 0:
                continue
            page = int(st.block_table[slot, p // pt])
            if page < 0:
                raise RuntimeError("KV append into an unmapped page")
            kv.k[page, :, p % pt, :] = k[r]
            kv.v[page, :, p % pt, :] = v[r]
        return q.reshape(rows, hq * D)

    def paged_attention(self, q, qkv, hq: int, hkv: int, b: StepBatch, kv: KVLayer, st: ModelState,
                        max_visible: int):
        cfg = self.cfg
        rows, D = q.shape[0], cfg.head_dim
        G = hq // hkv
        pt = st.sc.page_tokens
        out = q.new_zeros(rows, hq, D)
        gate = qkv[:, :2 * hq * D].reshape(rows, hq, 2 * D)[..., D:]
        qh = q.reshape(rows, hq, D)
        for r in range(rows):
            slot, p = int(b.row_slot[r]), int(b.row_pos[r])
            if slot < 0:
                continue
            vis = p + 1
            nblk = -(-vis // pt)
            pages = st.block_table[slot, :nblk].long()
            K = kv.k[pages].permute(1, 0, 2, 3).reshape(hkv, nblk * pt, D)[:, :vis].float()
            V = kv.v[pages].permute(1, 0, 2, 3).reshape(hkv, nblk * pt, D)[:, :vis].float()
            K = K.repeat_interleave(G, 0)
            V = V.repeat_interleave(G, 0)
            s = torch.einsum("hd,htd->ht", qh[r].float(), K) * (D ** -0.5)
            pr = torch.softmax(s, -1)
            out[r] = torch.einsum("ht,htd->hd", pr, V)
        out = out * torch.sigmoid(gate.float())
        return out.reshape(rows, hq * D)

    def gdn(self, proj, gw: GdnW, hk: int, hv: int, b: StepBatch, gs: GdnLayerState, st: ModelState, log=None,
            to_alt: bool = False):
        cfg = self.cfg
        Dk, Dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        rows = proj.shape[0]
        qk = hk * Dk
        ring = st.sc.conv_ring
        rep = hv // hk
        out = proj.new_zeros(rows, hv * Dv)
        cw = gw.conv_w.float()
        A = -torch.exp(gw.A_log.float())
        z_off, b_off = 2 * qk + hv * Dv, 2 * qk + 2 * hv * Dv
        # per-head channel gather (matches the per-value-head private history layout)
        idx = []
        for h in range(hv):
            kh = h // rep
            idx.append(torch.cat([torch.arange(kh * Dk, (kh + 1) * Dk), torch.arange(qk + kh * Dk, qk + (kh + 1) * Dk),
                                  torch.arange(2 * qk + h * Dv, 2 * qk + (h + 1) * Dv)]))
        idx = torch.stack(idx).to(proj.device)          # [hv, 2Dk+Dv]
        for s in range(b.n_seqs):
            row0, n, slot, pos0 = (int(v) for v in b.seq_desc[s])
            if n <= 0:
                continue
            S = gs.rec[slot].clone()
            for i in range(n):
                row, pos = row0 + i, pos0 + i
                x = proj[row, :2 * qk + hv * Dv].float()
                xh = x[idx]                              # [hv, CH]
                wh = cw[idx]                             # [hv, CH, 4]
                y = wh[..., 3] * xh
                for j in (1, 2, 3):
                    if pos - j >= 0:
                        if i - j >= 0:
                            tap = proj[row - j, :2 * qk + hv * Dv].float()[idx]
                        else:
                            tap = gs.conv[slot, :, (pos - j) % ring, :].float()
                        y = y + wh[..., 3 - j] * tap
                gs.conv[slot, :, pos % ring, :] = xh.to(gs.conv.dtype)
                c = F.silu(y)
                q = c[:, :Dk]
                k = c[:, Dk:2 * Dk]
                v = c[:, 2 * Dk:]
                q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * (Dk ** -0.5)
                k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
                beta = torch.sigmoid(proj[row, b_off:b_off + hv].float())
                g = A * F.softplus(proj[row, b_off + hv:b_off + 2 * hv].float() + gw.dt_bias.float())
                d = torch.exp(g)
                S = S * d[:, None, None]
                kvm = torch.einsum("hkv,hk->hv", S, k)
                delta = (v - kvm) * beta[:, None]
                S = S + k[:, :, None] * delta[:, None, :]
                o = torch.einsum("hkv,hk->hv", S, q)
                if log is not None:
                    log[0][row] = k
                    log[1][row] = delta
                    log[2][row] = d
                o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * gw.norm_w.float()
                zz = proj[row, z_off:z_off + hv * Dv].float().reshape(hv, Dv)
                out[row] = (o * F.silu(zz)).reshape(-1)
            (gs.rec_alt if to_alt else gs.rec)[slot] = S
        return out

    def gdn_replay(self, gs: GdnLayerState, hv: int, seq_desc, n_seqs: int, log) -> None:
        for s in range(n_seqs):
            row0, n, slot, _ = (int(v) for v in seq_desc[s])
            S = gs.rec[slot]
            for i in range(n):
                S = S * log[2][row0 + i][:, None, None]
                S = S + log[0][row0 + i][:, :, None] * log[1][row0 + i][:, None, :]
            gs.rec[slot] = S

    def gather_rows(self, x, rows_idx, n: int, name: str, status):
        return x[rows_idx[:n].long()]

    def sample(self, logits, b: StepBatch, n: int, mask=None, mask_active=None, status=None):
        out = torch.empty(n, dtype=torch.int32)
        params = b._np_samp
        lg = logits.detach().float().cpu()
        for r in range(n):
            m = None
            if mask is not None and (mask_active is None or bool(mask_active[r])):
                m = mask[r].cpu()
            out[r] = sample_row_host(lg[r], params[r], m)
        return out.to(logits.device)

    def rmsnorm(self, x, w, eps: float, name: str, one_plus: bool = True, add=None, sum_out=None):
        x = x.float()
        if add is not None:
            x = x + add.float()
            if sum_out is not None:
                sum_out.copy_(x)
        ww = (1.0 + w.float()) if one_plus else w.float()
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * ww
