"""Host implementation of the sampling contract in ``csrc/include/ps_sampling.h``.

Used by the CPU reference op set and by tests that check host == device randomness (the reference's
`test_qwen35_sampling_rng`).  Vectorised with numpy uint64 arithmetic (wrap-around is intended).
"""
from __future__ import annotations

import numpy as np
import torch

MAX_ATTEMPTS = 4096
_M = np.uint64(0xFFFFFFFFFFFFFFFF)


def _mix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = x + np.uint64(0x9E3779B97F4A7C15)
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return x ^ (x >> np.uint64(31))


def sampling_bits(seed: int, sample_index: int, attempt: int, token_ids: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        h = _mix64(np.uint64(seed) ^ np.uint64(0x6A09E667F3BCC908))
        h = _mix64(h + np.uint64(sample_index) * np.uint64(0xD6E8FEB86659FD93))
        h = _mix64(h + np.uint64(attempt) * np.uint64(0xA0761D6478BD642F))
        h = _mix64(h + token_ids.astype(np.uint64) * np.uint64(0xE7037ED1A0B428DB))
    return (h >> np.uint64(32)).astype(np.uint32)


def sampling_uniform(seed: int, sample_index: int, attempt: int, token_ids: np.ndarray) -> np.ndarray:
    bits = sampling_bits(seed, sample_index, attempt, token_ids)
    return ((bits >> np.uint32(9)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 8388608.0)


def _allowed(vocab: int, mask) -> np.ndarray:
    if mask is None:
        return np.ones(vocab, dtype=bool)
    words = np.asarray(mask, dtype=np.uint32)
    ids = np.arange(vocab)
    return ((words[ids >> 5] >> (ids & 31).astype(np.uint32)) & 1).astype(bool)


def sample_row_host(logits: torch.Tensor, p, mask=None) -> int:
    """p: structured row (mode, temperature, top_p, top_k, seed, sample_index).  Returns -1 on failure."""
    lg = logits.numpy().astype(np.float32)
    vocab = lg.shape[0]
    mode = int(p["mode"])
    if mode == 0:
        return -1
    if not np.all(np.isfinite(lg)):
        return -1
    ok = _allowed(vocab, mask)
    if not ok.any():
        return -1
    masked = np.where(ok, lg, -np.inf)
    best = int(np.argmax(masked))            # first maximal index = lower id on ties
    temp = float(p["temperature"])
    if mode == 1 or not temp > 0:
        return best
    mx = lg[best]
    inv_t = np.float32(1.0 / temp)
    top_p, top_k = float(p["top_p"]), int(p["top_k"])
    need_mass = top_p < 1.0
    ids = np.arange(vocab)
    w = np.where(ok, np.exp(((lg - mx) * inv_t).astype(np.float32)).astype(np.float64), 0.0)
    Z = w.sum() if need_mass else 0.0
    for attempt in range(MAX_ATTEMPTS):
        u = sampling_uniform(int(p["seed"]), int(p["sample_index"]), attempt, ids)
        s = (lg - mx) * inv_t - np.log(-np.log(u))
        s = np.where(ok, s, -np.inf)
        c = int(np.argmax(s))
        good = True
        if top_k > 0 or need_mass:
            before = ok & ((lg > lg[c]) | ((lg == lg[c]) & (ids < c)))
            if top_k > 0 and before.sum() >= top_k:
                good = False
            if need_mass and not (w[before].sum() < top_p * Z):
                good = False
        if good:
            return c
    return -1
