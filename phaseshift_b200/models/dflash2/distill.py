"""Distil a DFlash2 drafter on samples of its target (for acceptance studies with random-init targets).

The target generates continuations of random prompts; for every position the drafter is trained to predict
the K tokens that follow an anchor from the block ``[anchor, MASK x K]`` and the target's tapped hidden
states of the preceding context (cross-entropy through the target's frozen lm_head, selector codebooks
trained through the same loss).  Plain PyTorch autograd on the torch drafter; not a hot path.
Reference workflow: tools/ HF exporters and docs/rnd/dflash2 notes (the reference ships trained drafters
rather than a trainer).
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch
import torch.nn.functional as F

from ..qwen35.reference import reference_forward
from .model import DFlash2Config, DFlash2Drafter


def target_samples(cfg, hf_weights: Dict[str, torch.Tensor], n_seqs: int, prompt_len: int, gen_len: int, seed: int = 0):
    """Greedy continuations + tapped hidden states from the fp32 oracle (small configs)."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n_seqs):
        ids = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=g).tolist()
        for _ in range(gen_len):
            ids.append(int(torch.argmax(reference_forward(cfg, hf_weights, ids)[-1])))
        out.append(ids)
    return out


def distill(drafter: DFlash2Drafter, cfg, hf_weights, sequences: Sequence[List[int]], k: int, steps: int = 200,
            lr: float = 2e-3, log=None) -> float:
    dcfg: DFlash2Config = drafter.cfg
    params = [p.requires_grad_(True) for p in drafter.w.values()]
    opt = torch.optim.AdamW(params, lr=lr, weight_decay=0.0)
    P = "model.language_model."
    emb = hf_weights[P + "embed_tokens.weight"].float()
    lm = hf_weights.get(P + "lm_head.weight", hf_weights[P + "embed_tokens.weight"]).float()
    taps_all = []
    for ids in sequences:
        _, taps = reference_forward(cfg, hf_weights, ids, return_hidden_layers=dcfg.target_layer_ids)
        taps_all.append([taps[l] for l in dcfg.target_layer_ids])
    g = torch.Generator().manual_seed(1)
    last = 0.0
    for step in range(steps):
        si = int(torch.randint(0, len(sequences), (1,), generator=g))
        ids = sequences[si]
        p = int(torch.randint(4, len(ids) - k - 1, (1,), generator=g))
        drafter.reset()
        with torch.no_grad():
            drafter.append_context([t[:p] for t in taps_all[si]], 0)
        block = torch.tensor([ids[p]] + [dcfg.mask_token_id] * k)
        h = drafter.backbone(emb[block], torch.arange(p, p + k + 1))[1:]
        loss = F.cross_entropy(h @ lm.T, torch.tensor(ids[p + 1:p + 1 + k]))
        opt.zero_grad()
        loss.backward()
        opt.step()
        last = float(loss)
        if log and step % 20 == 0:
            log(f"distill step {step} loss {last:.3f}")
    for p_ in params:
        p_.requires_grad_(False)
    return last


# ---------------------------------------------------------------------------------------------------------------
# Distillation against the serving engine itself (any size, on the GPU): the samples are what the ENGINE decodes
# greedily and the hidden states it taps while doing so -- exactly what the drafter is fed at inference time.

def engine_samples(engine, tap_layers: Sequence[int], n_seqs: int, prompt_len: int, gen_len: int, seed: int = 0,
                   prefill_chunk: int = 2048):
    """[(token ids, [tap tensor [len - 1, H] per tapped layer])]: greedy continuations of random prompts decoded by
    ``engine`` with the tapped hidden states of every position that was fed to it."""
    from ...runtime.batch import SeqRows
    g = torch.Generator().manual_seed(seed)
    out = []
    taps_l = list(tap_layers)
    for _ in range(n_seqs):
        ids = torch.randint(0, engine.cfg.vocab_size, (prompt_len,), generator=g).tolist()
        rows: List[List[torch.Tensor]] = [[] for _ in taps_l]
        s = engine.open_sequence()
        try:
            tok = None
            for c0 in range(0, prompt_len, prefill_chunk):
                chunk = ids[c0:c0 + prefill_chunk]
                last = c0 + prefill_chunk >= prompt_len
                toks, o = engine.step([SeqRows(s.slot, c0, chunk, (len(chunk) - 1,) if last else ())], [s], tap_layers=taps_l)
                for j, l in enumerate(taps_l):
                    rows[j].append(o.taps[l][:len(chunk)].clone())
                if toks:
                    tok = toks[0]
            for _ in range(gen_len):
                ids.append(tok)
                toks, o = engine.step([SeqRows(s.slot, s.position, [tok], (0,))], [s], tap_layers=taps_l)
                for j, l in enumerate(taps_l):
                    rows[j].append(o.taps[l][:1].clone())
                tok = toks[0]
            ids.append(tok)
        finally:
            engine.close_sequence(s)
        out.append((ids, [torch.cat(r, 0) for r in rows]))
    return out


def distill_on_engine(drafter: DFlash2Drafter, engine, samples, k: int, steps: int = 200, lr: float = 1e-3, ctx: int = 256,
                      log=None) -> float:
    """Train the torch drafter (on the engine's device) to predict the K tokens that follow an anchor, from
    ``[anchor, MASK x K]`` and the taps of up to ``ctx`` preceding positions, through the target's frozen embedding
    and lm_head.  Returns the last loss.  The trained weights can then be handed to ``DFlash2NativeDrafter``."""
    from .decoder import embed_rows
    dcfg: DFlash2Config = drafter.cfg
    dev = drafter.device
    W = engine.runner.w
    lm = W.lm_head.dense().to(device=dev, dtype=drafter.dtype)                # frozen target head [vocab, H]
    params = [p.requires_grad_(True) for n, p in drafter.w.items() if "codebook" not in n]
    opt = torch.optim.AdamW(params, lr=lr, weight_decay=0.0)
    g = torch.Generator().manual_seed(1)
    last = 0.0
    for step in range(steps):
        ids, taps = samples[int(torch.randint(0, len(samples), (1,), generator=g))]
        p = int(torch.randint(min(8, len(ids) - k - 2), len(ids) - k - 1, (1,), generator=g))
        c0 = max(0, p - ctx)
        drafter.reset()
        with torch.no_grad():
            drafter.append_context([t[c0:p].to(drafter.dtype) for t in taps], c0)
        block = torch.tensor([ids[p]] + [dcfg.mask_token_id] * k, device=dev)
        x = embed_rows(W.embed, block).to(drafter.dtype)
        h = drafter.backbone(x, torch.arange(p, p + k + 1, device=dev))[1:]
        loss = F.cross_entropy((h @ lm.T).float(), torch.tensor(ids[p + 1:p + 1 + k], device=dev))
        opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(params, 1.0)
        opt.step()
        last = float(loss)
        if log and step % 20 == 0:
            log(f"distill step {step} loss {last:.3f}")
    for p_ in params:
        p_.requires_grad_(False)
    drafter.reset()
    return last
