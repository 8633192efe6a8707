"""Synthetic token batches (host side).

The reference draws windows of T+1 tokens from a tokenised text corpus
(packages/train/src/data.ts:18-119: inputs = window[:-1], targets = window[1:]); the
benchmark configurations name no corpus, so the windows are filled with seeded random ids
instead: uniform over the vocabulary, or Zipf(s) with p(k) ~ 1/(k+1)^s.
"""
from __future__ import annotations

import math

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


class DataLoader:
    """Batches of (inputs, targets) int32 [B, T] windows from a token array — the reference's
    DataLoader (packages/train/src/data.ts:18-177) with per-rank sharding added for data
    parallel runs.

    random mode (data.ts:91-119): every batch item starts at ``floor(rng.next() * (N - T))``;
    one draw per item, in item order.  With ``world > 1`` all ranks consume the same stream
    of draws and rank r keeps items r*B .. r*B+B-1 of every global batch of B*world, so the
    union over ranks equals the single-process loader with batch B*world.
    packed mode (data.ts:130-167): cursors ``b * floor(N / (B*world))`` advance by T per batch
    and wrap at N; the target of the last token of the corpus is token 0.  Rank r owns
    cursors r*B .. r*B+B-1.

    Two reusable host buffers alternate between calls (data.ts:48-58).  ``pin`` puts them in
    page-locked memory: ``nextDeviceBatch`` then only enqueues the copies and returns, and an
    event recorded behind each pair of copies guards the slot — the loader waits on that event
    before it writes the slot again, so a host that runs several micro-steps or whole steps
    ahead of the device can never overwrite tokens whose copy has not run yet.  ``slots``
    (>= 2) is how many batches the host may prepare ahead before that wait can block.
    """

    def __init__(self, tokens, rng, batchSize: int, blockSize: int, packed: bool = False, rank: int = 0,
                 world: int = 1, backend=None, pin: bool = False, slots: int = 2):
        self.tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        self.rng, self.batchSize, self.blockSize, self.packed = rng, int(batchSize), int(blockSize), bool(packed)
        self.rank, self.world = int(rank), int(world)
        self.backend = backend
        n = len(self.tokens)
        if self.packed:
            stride = n // (self.batchSize * self.world)
            self.cursors = [(self.rank * self.batchSize + b) * stride for b in range(self.batchSize)]
        self._ring = []
        self._pinned = []
        elems = self.batchSize * self.blockSize
        self._events = []           # per slot: event recorded behind the last upload from it
        self._in_flight = []        # per slot: True while that event has not been waited on
        for _ in range(max(2, int(slots))):
            if pin and backend is not None:
                a, pa = backend.pinned_array((self.batchSize, self.blockSize), np.int32)
                b, pb = backend.pinned_array((self.batchSize, self.blockSize), np.int32)
                self._pinned += [pa, pb]
            else:
                a = np.zeros((self.batchSize, self.blockSize), np.int32)
                b = np.zeros((self.batchSize, self.blockSize), np.int32)
            assert a.size == elems
            self._ring.append((a, b))
            self._events.append(None)
            self._in_flight.append(False)
        self._idx = 0
        self._last = 0

    @property
    def stepsPerEpoch(self) -> int:
        return len(self.tokens) // (self.batchSize * self.blockSize * self.world)

    def __len__(self) -> int:
        return len(self.tokens)

    def nextBatch(self):
        """(inputs, targets): int32 [B, T] host arrays, valid until the call after next."""
        slot = self._idx
        if self._in_flight[slot]:                       # a queued copy still reads this slot
            self.backend.eventSync(self._events[slot])
            self._in_flight[slot] = False
        inputs, targets = self._ring[slot]
        self._last = slot
        self._idx = (self._idx + 1) % len(self._ring)
        B, T, N, tok = self.batchSize, self.blockSize, len(self.tokens), self.tokens
        if not self.packed:
            if N <= T:
                raise ValueError(f"Token count ({N}) must exceed block size ({T}) — need at least {T + 1} tokens "
                                 "for input+target windows")
            maxStart = N - T
            for g in range(B * self.world):
                start = int(math.floor(self.rng.next() * maxStart))
                b = g - self.rank * B
                if 0 <= b < B:
                    inputs[b] = tok[start:start + T]
                    targets[b] = tok[start + 1:start + T + 1]
            return inputs, targets
        for b in range(B):
            pos, remaining, dst = self.cursors[b], T, 0
            while remaining > 0:
                span = min(remaining, N - pos)
                inputs[b, dst:dst + span] = tok[pos:pos + span]
                if pos + span < N:
                    targets[b, dst:dst + span] = tok[pos + 1:pos + span + 1]
                else:
                    if span > 1:
                        targets[b, dst:dst + span - 1] = tok[pos + 1:N]
                    targets[b, dst + span - 1] = tok[0]
                dst += span
                remaining -= span
                pos += span
                if pos == N:
                    pos = 0
            self.cursors[b] = pos
        return inputs, targets

    def nextDeviceBatch(self):
        """The next batch as device tensors, copied on the backend's stream.  The tensors own
        their device storage and keep no reference to the loader's host buffers (``.data``
        reads the device copy back).  Pageable buffers are staged by the driver before the
        copy call returns; pinned ones are guarded by the slot's event (see the class text)."""
        inputs, targets = self.nextBatch()
        B = self.backend
        if not self._pinned:
            return B.upload(inputs.copy(), "i32"), B.upload(targets.copy(), "i32")
        slot = self._last
        out = (B.uploadAsync(inputs, "i32"), B.uploadAsync(targets, "i32"))
        if self._events[slot] is None:
            self._events[slot] = B.eventCreate()
        B.eventRecord(self._events[slot])
        self._in_flight[slot] = True
        return out

    def close(self) -> None:
        """Wait for queued copies and give the pinned buffers and events back."""
        if self.backend is None:
            return
        for i, ev in enumerate(self._events):
            if ev is not None:
                if self._in_flight[i]:
                    self.backend.eventSync(ev)
                self.backend.eventDestroy(ev)
        for p in self._pinned:
            self.backend.free_pinned(p)
        self._events, self._pinned, self._in_flight = [None] * len(self._ring), [], [False] * len(self._ring)
