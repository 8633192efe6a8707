"""Synthetic token batches (host side).

The reference draws windows of T+1 tokens from a tokenised text corpus
(packages/train/src/data.ts:18-119: inputs = window[:-1], targets = window[1:]); the
benchmark configurations name no corpus, so the windows are filled with seeded random ids
instead: uniform over the vocabulary, or Zipf(s) with p(k) ~ 1/(k+1)^s.
"""
from __future__ import annotations

import numpy as np


def _windows(w: np.ndarray):
    return np.ascontiguousarray(w[:, :-1]), np.ascontiguousarray(w[:, 1:])


def uniform_batches(seed: int, n_steps: int, batch: int, T: int, vocab: int):
    g = np.random.default_rng(seed)
    return [_windows(g.integers(0, vocab, size=(batch, T + 1), dtype=np.int32)) for _ in range(n_steps)]


def zipf_batches(seed: int, n_steps: int, batch: int, T: int, vocab: int, s: float = 1.1):
    g = np.random.default_rng(seed)
    p = 1.0 / np.power(np.arange(1, vocab + 1, dtype=np.float64), s)
    cdf = np.cumsum(p / p.sum())
    out = []
    for _ in range(n_steps):
        u = g.random(size=(batch, T + 1))
        out.append(_windows(np.minimum(np.searchsorted(cdf, u), vocab - 1).astype(np.int32)))
    return out
