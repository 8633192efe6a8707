"""Train step of the reference, restated.  TEST INFRASTRUCTURE ONLY.

Follows ``packages/train/src/trainer.ts`` — LR schedule (:1088-1096, :1150-1158), the
micro-step loop (:1188-1273), gradient norm on the path a backend without
``sumOfSquares`` takes (:1352-1375: ``mul(g,g)`` then ``sum`` per tensor, f64 total),
clip folding into ``effectiveGradScale`` (:1297, :1650-1656), optimizer call and zero-grad
(:1750-1780) — and ``packages/train/src/optimizers.ts`` (AdamW :21-115).  The no-decay
name set is the CLI's (``apps/cli/src/commands/train.ts:320-331``): wte, wpe, lnF.*, every
layer's ln1.*/ln2.*; ``lmHead`` is decayed because the set holds the non-existent name
``lmHead.weight``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

from . import lib
from .autograd import Tape
from .cpu_ref import CpuRef, SeededRng, f32, f64
from .gpt import ModelConfig, gpt_forward, init_gpt


@dataclass
class TrainConfig:
    """packages/core/src/types.ts:66-142 (the fields the step uses) with its defaults."""
    iters: int = 1000
    batchSize: int = 64
    lr: float = 3e-4
    lrMin: float = 0.0
    warmupIters: int = 0
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weightDecay: float = 0.1
    gradClip: float = 1.0
    seed: int = 42
    gradAccumSteps: int = 1


def no_decay_names(cfg: ModelConfig) -> set:
    """apps/cli/src/commands/train.ts:320-331."""
    s = {"wte", "wpe", "lnF.weight", "lnF.bias", "lmHead.weight"}
    for i in range(cfg.nLayer):
        for ln in ("ln1", "ln2"):
            s.add(f"layer.{i}.{ln}.weight")
            s.add(f"layer.{i}.{ln}.bias")
    return s


def lr_at(tc: TrainConfig, step: int) -> float:
    """trainer.ts:1088-1096 and :1150-1158 (step is 0-based)."""
    total = tc.iters
    warmup = tc.warmupIters if tc.warmupIters > 0 else (0 if tc.warmupIters < 0 else min(2000, total // 5))
    lr_min = tc.lr / 10 if (tc.lrMin or 0) == 0 else tc.lrMin
    decay_denom = max(1, total - warmup)
    if step < warmup:
        base = lr_min + (tc.lr - lr_min) * (step + 1) / warmup
    else:
        decay = (step - warmup) / decay_denom
        base = lr_min + (tc.lr - lr_min) * 0.5 * (1 + math.cos(math.pi * decay))
    return max(lr_min * 0.1, base * 1.0)


class AdamW:
    """optimizers.ts:21-115."""

    def __init__(self, lr=3e-4, beta1=0.9, beta2=0.999, eps=1e-8, weightDecay=0.01, noDecayNames=None):
        self.lr, self.beta1, self.beta2, self.eps, self.wd = lr, beta1, beta2, eps, weightDecay
        self.no_decay = noDecayNames or set()
        self.step_count = 0
        self.b1pow = 1.0
        self.b2pow = 1.0
        self.m: dict[str, np.ndarray] = {}
        self.v: dict[str, np.ndarray] = {}

    def set_lr(self, lr):
        self.lr = lr

    def step(self, params: dict, grads: dict, grad_scale: float = 1.0):
        """params/grads: name -> float32 array (updated in place)."""
        self.step_count += 1
        self.b1pow *= self.beta1
        self.b2pow *= self.beta2
        bc1, bc2 = 1 - self.b1pow, 1 - self.b2pow
        for name, p in params.items():
            g = grads.get(name)
            if g is None:
                continue
            if name not in self.m:
                self.m[name] = np.zeros(p.size, f32)
                self.v[name] = np.zeros(p.size, f32)
            wd = 0.0 if name in self.no_decay else self.wd
            assert p.flags.c_contiguous and p.dtype == f32
            gc = np.ascontiguousarray(g, dtype=f32)
            lib().alpha_oracle_adamw_f32(p.ctypes.data, gc.ctypes.data, self.m[name].ctypes.data,
                                         self.v[name].ctypes.data, p.size, self.lr, self.beta1,
                                         self.beta2, self.eps, wd, bc1, bc2, float(grad_scale))


def adamw_reference_loop(p, g, m, v, lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale):
    """Pure-Python twin of optimizers.ts:84-92 for cross-checking the C loop (small inputs)."""
    for j in range(p.size):
        gj = float(g[j]) * grad_scale
        if wd > 0:
            p[j] = f32(float(p[j]) - lr * wd * float(p[j]))
        m[j] = f32(beta1 * float(m[j]) + (1 - beta1) * gj)
        v[j] = f32(beta2 * float(v[j]) + (1 - beta2) * gj * gj)
        mhat = float(m[j]) / bc1
        vhat = float(v[j]) / bc2
        p[j] = f32(float(p[j]) - lr * mhat / (math.sqrt(vhat) + eps))


def grad_norm(B: CpuRef, grads: list, grad_scale_abs: float) -> float:
    """trainer.ts:1352-1375 on a backend with neither sumOfSquares nor totalSumOfSquares."""
    total = 0.0
    for g in grads:
        total += float(B.sum(B.mul(g, g)))
    return math.sqrt(total) * grad_scale_abs


class Trainer:
    """One object = one training run of trainer.ts:563 restricted to the step math."""

    def __init__(self, mc: ModelConfig, tc: TrainConfig, params: dict | None = None):
        self.mc, self.tc = mc, tc
        self.B = CpuRef()
        self.P = params if params is not None else init_gpt(mc, SeededRng(tc.seed))
        self.opt = AdamW(lr=tc.lr, beta1=tc.beta1, beta2=tc.beta2, eps=tc.eps,
                         weightDecay=tc.weightDecay, noDecayNames=no_decay_names(mc))
        self.tape = Tape()
        self.step_index = 0

    def train_step(self, batches):
        """batches: list (one per micro-step) of (tokens [B,T] int32, targets [B,T] int32).
        Returns dict(loss, gradNorm, lr, clipCoef)."""
        tc = self.tc
        accum = len(batches)
        lr = lr_at(tc, self.step_index)
        self.opt.set_lr(lr)
        loss_val = 0.0
        loss_acc = None
        for tokens, targets in batches:
            _, loss = gpt_forward(self.mc, self.P, self.B, self.tape, tokens, targets)
            if accum > 1:   # trainer.ts:1210-1226: accumulate scale(loss, 1/accum) in f32
                sl = self.B.scale(loss.data, 1 / accum)
                loss_acc = sl if loss_acc is None else self.B.add(loss_acc, sl)
            else:
                loss_val = float(loss.data)
            self.tape.backward(loss, self.B)
            self.tape.clear()
        if accum > 1:
            loss_val = float(loss_acc)
        grad_scale = 1.0 / accum
        grads = {n: v.grad for n, v in self.P.items() if v.grad is not None}
        gnorm = grad_norm(self.B, list(grads.values()), abs(grad_scale))
        clip = 1.0
        eff = grad_scale
        if tc.gradClip > 0 and gnorm > tc.gradClip:      # trainer.ts:1650-1656
            clip = tc.gradClip / gnorm
            eff *= clip
        self.opt.step({n: v.data for n, v in self.P.items()}, grads, eff)
        for v in self.P.values():
            v.grad = None
        self.step_index += 1
        return {"loss": loss_val, "gradNorm": gnorm, "lr": lr, "clipCoef": clip}


def uniform_batches(seed: int, n_steps: int, batch: int, T: int, vocab: int):
    """Synthetic data of the tiny byte-level GPT: each row is a window of T+1 tokens drawn uniform
    in [0, vocab); inputs are w[:-1], targets w[1:].  (The reference draws windows from a
    tokenised text file, packages/train/src/data.ts:18-119; no text corpus is used here.)"""
    g = np.random.default_rng(seed)
    out = []
    for _ in range(n_steps):
        w = g.integers(0, vocab, size=(batch, T + 1), dtype=np.int32)
        out.append((np.ascontiguousarray(w[:, :-1]), np.ascontiguousarray(w[:, 1:])))
    return out


def zipf_batches(seed: int, n_steps: int, batch: int, T: int, vocab: int, s: float = 1.1):
    """Synthetic data of the larger model shapes: token ids Zipf(s) over the vocabulary
    (p(k) ~ 1/(k+1)^s), same windowing as uniform_batches."""
    g = np.random.default_rng(seed)
    p = 1.0 / np.power(np.arange(1, vocab + 1, dtype=f64), s)
    cdf = np.cumsum(p / p.sum())
    out = []
    for _ in range(n_steps):
        u = g.random(size=(batch, T + 1))
        w = np.minimum(np.searchsorted(cdf, u), vocab - 1).astype(np.int32)
        out.append((np.ascontiguousarray(w[:, :-1]), np.ascontiguousarray(w[:, 1:])))
    return out
