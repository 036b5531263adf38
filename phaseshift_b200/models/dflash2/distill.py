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
