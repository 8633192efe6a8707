"""TEST INFRASTRUCTURE — CPU restatement of the reference's batch construction.

Only tests may import this module.  It restates, loop for loop, DataLoader.nextBatchRandom
(packages/train/src/data.ts:91-119) and DataLoader.nextBatchPacked (:130-167) for one
process; the package's loader must equal it for world == 1 and, for world > 1, the union of
the ranks' batches must equal this loader run with batch size B*world.

Parity status: the reference's tests hold no golden batches for this path, and its loader
cannot run here (no JavaScript runtime), so this restatement is unpinned by reference
outputs; the packed-mode wrap-around case is additionally checked against a hand-computed
answer in tests/test_data_eval.py.
"""
from __future__ import annotations

import math

import numpy as np


class OracleLoader:
    def __init__(self, tokens, rng, batchSize, blockSize, packed=False):
        self.tokens = [int(t) for t in tokens]
        self.rng, self.B, self.T, self.packed = rng, batchSize, blockSize, packed
        if packed:                                   # data.ts:37-46
            stride = len(self.tokens) // batchSize
            self.cursors = [b * stride for b in range(batchSize)]

    def nextBatch(self):
        return self._packed() if self.packed else self._random()

    def _random(self):                               # data.ts:91-119
        B, T, tok = self.B, self.T, self.tokens
        if len(tok) <= T:
            raise ValueError("Token count must exceed block size")
        maxStart = len(tok) - T
        inputs = np.zeros((B, T), np.int32)
        targets = np.zeros((B, T), np.int32)
        for b in range(B):
            start = int(math.floor(self.rng.next() * maxStart))
            for i in range(T):
                inputs[b, i] = tok[start + i]
                targets[b, i] = tok[start + 1 + i]
        return inputs, targets

    def _packed(self):                               # data.ts:130-167
        B, T, tok = self.B, self.T, self.tokens
        N = len(tok)
        inputs = np.zeros((B, T), np.int32)
        targets = np.zeros((B, T), np.int32)
        for b in range(B):
            pos, remaining, dst = self.cursors[b], T, 0
            while remaining > 0:
                span = min(remaining, N - pos)
                for i in range(span):
                    inputs[b, dst + i] = tok[pos + i]
                if pos + span < N:
                    for i in range(span):
                        targets[b, dst + i] = tok[pos + 1 + i]
                else:
                    for i in range(span - 1):
                        targets[b, dst + i] = tok[pos + 1 + i]
                    targets[b, dst + span - 1] = tok[0]
                dst += span
                remaining -= span
                pos += span
                if pos == N:
                    pos = 0
            self.cursors[b] = pos
        return inputs, targets
