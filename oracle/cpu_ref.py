"""numpy restatement of the reference's CPU tensor backend.  TEST INFRASTRUCTURE ONLY.

Every function follows one method of ``CpuRefBackend`` in
``packages/tensor/src/cpu_ref.ts`` (line ranges in each docstring).  The reference
computes in JavaScript doubles and stores each op's output into a ``Float32Array``; the
restatement therefore promotes to float64, evaluates the same expression in the same
association order, and rounds to float32 exactly where the reference stores.

Tensors are plain C-contiguous numpy arrays (float32 or int32).
"""
from __future__ import annotations

import ctypes
import math

import numpy as np

from . import _Rng, lib

f32 = np.float32
f64 = np.float64


def _a(x):
    return np.ascontiguousarray(x)


class SeededRng:
    """packages/core/src/rng.ts:6-68 (through the C restatement in oracle/rng.c)."""

    def __init__(self, seed: int = 42):
        self._st = _Rng()
        self._seed = seed
        self.seed(seed)

    def seed(self, s: int) -> None:
        self._seed = s
        lib().alpha_rng_seed(ctypes.byref(self._st), ctypes.c_uint32(s & 0xFFFFFFFF))

    def state(self) -> int:
        return self._seed

    def next(self) -> float:
        return lib().alpha_rng_next(ctypes.byref(self._st))

    def next_gauss(self) -> float:
        return lib().alpha_rng_gauss(ctypes.byref(self._st))

    def fill_gauss(self, shape, std: float) -> np.ndarray:
        out = np.empty(shape, dtype=f32)
        lib().alpha_rng_fill_gauss_f32(ctypes.byref(self._st), out.ctypes.data, out.size, float(std))
        return out

    def fill_uniform_int(self, shape, hi: int) -> np.ndarray:
        out = np.empty(shape, dtype=np.int32)
        lib().alpha_rng_fill_uniform_i32(ctypes.byref(self._st), out.ctypes.data, out.size, int(hi))
        return out


class PySeededRng:
    """Pure-Python twin of SeededRng (rng.ts:6-68) used to cross-check the C code."""

    def __init__(self, seed: int = 42):
        self.seed(seed)

    def seed(self, s: int) -> None:
        self.s0 = s & 0xFFFFFFFF
        self.s1 = (s ^ 0xDEADBEEF) & 0xFFFFFFFF
        self.has_spare = False
        self.spare = 0.0
        for _ in range(20):
            self.next()

    def next(self) -> float:
        M = 0xFFFFFFFF
        s1 = self.s0
        s0 = self.s1
        self.s0 = s0
        s1 ^= (s1 << 23) & M
        s1 ^= s1 >> 17
        s1 ^= s0
        s1 ^= s0 >> 26
        self.s1 = s1
        return ((self.s0 + self.s1) & M) / 4294967296.0

    def next_gauss(self) -> float:
        if self.has_spare:
            self.has_spare = False
            return self.spare
        while True:
            u = self.next() * 2 - 1
            v = self.next() * 2 - 1
            s = u * u + v * v
            if not (s >= 1 or s == 0):
                break
        mul = math.sqrt(-2.0 * math.log(s) / s)
        self.spare = v * mul
        self.has_spare = True
        return u * mul


class CpuRef:
    """The reference CPU backend, method for method (cpu_ref.ts:109-933)."""

    name = "cpu_ref_oracle"

    # ── creation (cpu_ref.ts:115-147) ─────────────────────────────────────
    def zeros(self, shape, dtype=f32):
        return np.zeros(shape, dtype=dtype)

    def ones(self, shape, dtype=f32):
        return np.ones(shape, dtype=dtype)

    def full(self, shape, value, dtype=f32):
        return np.full(shape, value, dtype=dtype)

    def fromArray(self, data, shape, dtype=f32):
        arr = np.asarray(data, dtype=dtype)
        if arr.size != int(np.prod(shape, dtype=np.int64)):
            raise ValueError(f"Data length {arr.size} does not match shape size")
        return arr.reshape(shape).copy()

    # ── binary / unary (cpu_ref.ts:55-84, 151-165, 337-362) ───────────────
    def add(self, a, b):
        return (a.astype(f64) + b.astype(f64)).astype(f32)

    def sub(self, a, b):
        return (a.astype(f64) - b.astype(f64)).astype(f32)

    def mul(self, a, b):
        return (a.astype(f64) * b.astype(f64)).astype(f32)

    def div(self, a, b):
        with np.errstate(divide="ignore", invalid="ignore"):
            return (a.astype(f64) / b.astype(f64)).astype(f32)

    def neg(self, a):
        return (-a).astype(f32)

    def exp(self, a):
        with np.errstate(over="ignore"):
            return np.exp(a.astype(f64)).astype(f32)

    def log(self, a):
        with np.errstate(divide="ignore", invalid="ignore"):
            return np.log(a.astype(f64)).astype(f32)

    def sqrt(self, a):
        with np.errstate(invalid="ignore"):
            return np.sqrt(a.astype(f64)).astype(f32)

    def pow(self, a, e):
        return np.power(a.astype(f64), e).astype(f32)

    def scale(self, a, s):
        return (a.astype(f64) * float(s)).astype(f32)

    def clamp(self, a, lo, hi):
        return np.maximum(lo, np.minimum(hi, a.astype(f64))).astype(f32)

    # ── matmul (cpu_ref.ts:166-258): f64 dot, one f32 rounding per output ──
    def matmul(self, a, b):
        if a.ndim < 2 or b.ndim < 2:
            raise ValueError("matmul requires at least 2D tensors")
        if a.shape[-1] != b.shape[-2]:
            raise ValueError(f"matmul shape mismatch: {a.shape} x {b.shape}")
        return np.matmul(a.astype(f64), b.astype(f64)).astype(f32)

    def matmul_sequential(self, a, b):
        """The literal triple loop of cpu_ref.ts:246-254 (2-D only), in C."""
        a = _a(a.astype(f32))
        b = _a(b.astype(f32))
        M, K = a.shape
        N = b.shape[1]
        c = np.empty((M, N), dtype=f32)
        lib().alpha_oracle_matmul_f32(a.ctypes.data, b.ctypes.data, c.ctypes.data, M, K, N)
        return c

    # ── reductions (cpu_ref.ts:260-333) ───────────────────────────────────
    def sum(self, a, axis=None, keepdims=False):
        if axis is None:
            s = np.sum(a.astype(f64))
            shape = tuple(1 for _ in a.shape) if keepdims else ()
            return np.full(shape, s, dtype=f32)
        return np.sum(a.astype(f64), axis=axis, keepdims=keepdims).astype(f32)

    def mean(self, a, axis=None, keepdims=False):
        if axis is None:
            s = np.sum(a.astype(f64)) / a.size
            shape = tuple(1 for _ in a.shape) if keepdims else ()
            return np.full(shape, s, dtype=f32)
        st = self.sum(a, axis, keepdims)            # rounds the sum to f32 first (:326-332)
        return (st.astype(f64) / a.shape[axis]).astype(f32)

    # ── nn (cpu_ref.ts:364-563) ───────────────────────────────────────────
    def embedding(self, weight, indices):
        return weight[indices.reshape(-1)].reshape(tuple(indices.shape) + (weight.shape[1],)).copy()

    def layerNorm(self, x, weight, bias, eps):
        """cpu_ref.ts:387-420: biased variance, f64 statistics."""
        xd = x.astype(f64)
        dim = x.shape[-1]
        mean = xd.sum(axis=-1, keepdims=True) / dim
        d = xd - mean
        var = (d * d).sum(axis=-1, keepdims=True) / dim
        inv = 1.0 / np.sqrt(var + eps)
        return ((xd - mean) * inv * weight.astype(f64) + bias.astype(f64)).astype(f32)

    def gelu(self, a):
        """cpu_ref.ts:422-427 (tanh approximation)."""
        x = a.astype(f64)
        c = math.sqrt(2 / math.pi)
        return (0.5 * x * (1 + np.tanh(c * (x + 0.044715 * x * x * x)))).astype(f32)

    def relu(self, a):
        return np.where(a > 0, a, 0).astype(f32)

    def silu(self, a):
        x = a.astype(f64)
        with np.errstate(over="ignore"):
            return (x / (1 + np.exp(-x))).astype(f32)

    def softmax(self, a, axis=-1):
        """cpu_ref.ts:439-493.  exp values are stored to f32 before the divide while the
        running sum keeps the unrounded doubles (:476-486)."""
        x = a.astype(f64)
        mx = x.max(axis=axis, keepdims=True)
        with np.errstate(invalid="ignore"):
            e = np.exp(x - mx)
        s = e.sum(axis=axis, keepdims=True)
        return (e.astype(f32).astype(f64) / s).astype(f32)

    def logSoftmax(self, a, axis=-1):
        """cpu_ref.ts:495-541."""
        x = a.astype(f64)
        mx = x.max(axis=axis, keepdims=True)
        s = np.exp(x - mx).sum(axis=axis, keepdims=True)
        lse = mx + np.log(s)
        return (x - lse).astype(f32)

    def crossEntropy(self, logits, targets):
        """cpu_ref.ts:543-563: mean over rows of -logSoftmax[target], f64 running sum."""
        n = logits.shape[0]
        lp = self.logSoftmax(logits, 1)
        picked = lp[np.arange(n), targets.reshape(-1)].astype(f64)
        # sequential f64 subtraction as in the reference; pairwise numpy sum for very long
        # inputs (the two differ only below f32 resolution)
        loss = _seq_neg_sum(picked) if n <= (1 << 16) else -float(np.sum(picked))
        return np.full((), loss / n, dtype=f32)

    # ── reshape / slice (cpu_ref.ts:567-692) ──────────────────────────────
    def reshape(self, a, shape):
        if int(np.prod(shape, dtype=np.int64)) != a.size:
            raise ValueError(f"Cannot reshape {a.shape} to {shape}: size mismatch")
        return a.reshape(shape).copy()

    def transpose(self, a, d0, d1):
        return _a(np.swapaxes(a, d0, d1)).copy()

    def slice(self, a, starts, ends):
        idx = tuple(slice(s, e) for s, e in zip(starts, ends))
        return _a(a[idx]).copy()

    def scatterSlice(self, grad, orig_shape, starts, ends):
        out = np.zeros(orig_shape, dtype=grad.dtype)
        idx = tuple(slice(s, s + n) for s, n in zip(starts, grad.shape))
        out[idx] = grad
        return out

    def cat(self, tensors, axis):
        if not tensors:
            raise ValueError("cat: empty tensor list")
        return np.concatenate(tensors, axis=axis)

    # ── utility (cpu_ref.ts:696-880) ──────────────────────────────────────
    def argmax(self, a, axis=None):
        return np.asarray(np.argmax(a, axis=axis), dtype=np.int32)

    def gather(self, a, axis, indices):
        return np.take_along_axis(a, indices.astype(np.int64), axis=axis).copy()

    def clone(self, a):
        return a.copy()

    def equal(self, a, b):
        return a.shape == b.shape and a.dtype == b.dtype and bool(np.all(a == b))

    def allClose(self, a, b, atol=1e-5, rtol=1e-8):
        if a.shape != b.shape:
            return False
        return bool(np.all(np.abs(a.astype(f64) - b.astype(f64)) <= atol + rtol * np.abs(b.astype(f64))))

    # ── mask (cpu_ref.ts:884-915) ─────────────────────────────────────────
    def causalMask(self, size):
        m = np.zeros((size, size), dtype=f32)
        m[np.triu_indices(size, 1)] = -np.inf
        return m

    def maskedFill(self, a, mask, value):
        out = a.copy()
        if mask.size == a.size:
            out[mask.reshape(a.shape) != 0] = value
        else:
            flat = out.reshape(-1, mask.size)
            flat[:, mask.reshape(-1) != 0] = value
        return out


def _seq_neg_sum(picked: np.ndarray) -> float:
    loss = 0.0
    for v in picked.tolist():
        loss -= v
    return loss
