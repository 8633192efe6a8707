"""Tape autograd of the reference, restated for the CPU path.  TEST INFRASTRUCTURE ONLY.

Follows ``packages/autograd/src/tape.ts:29-157`` (Variable, Tape.backward: reverse walk,
``clone`` for the first gradient reaching a variable and ``add`` for every later one) and
the op wrappers of ``packages/autograd/src/ops.ts``.  Only the branches that the
reference takes when its backend is ``cpu_ref`` are restated, i.e. the JavaScript
fallbacks (cpu_ref implements none of the optional fused hooks except ``scatterSlice``):
transpose+matmul for ``matmulTransposed`` (ops.ts:200-234), the composed ``softCap``
(:329-340), host-loop GELU backward (:404-418, :451-466), layerNorm backward (:523-569),
embedding scatter-add (:495-505) and cross-entropy backward (:713-727).

Extensions that the benchmarked model shapes need but the reference lacks (RMSNorm, RoPE,
tied head) are written in the same discipline (f64 arithmetic, f32 stores per op) and
marked EXTENSION.
"""
from __future__ import annotations

import math

import numpy as np

from . import lib
from .cpu_ref import CpuRef, f32, f64


class Variable:
    __slots__ = ("data", "grad", "requires_grad")

    def __init__(self, data, requires_grad=False):
        self.data = data
        self.grad = None
        self.requires_grad = requires_grad


class Tape:
    """tape.ts:43-157."""

    def __init__(self):
        self.entries = []

    def record(self, output, inputs, backward):
        self.entries.append((output, inputs, backward))

    def backward(self, loss: Variable, B: CpuRef, initial_grad=None):
        loss.grad = initial_grad if initial_grad is not None else B.ones(loss.data.shape)
        for output, inputs, backward in reversed(self.entries):
            g_out = output.grad
            if g_out is None:
                continue
            needs = [v.requires_grad for v in inputs]
            grads = backward(g_out, B, needs)
            for inp, g in zip(inputs, grads):
                if g is None or not inp.requires_grad:
                    continue
                if inp.grad is not None:
                    inp.grad = B.add(inp.grad, g)      # cpu_ref has no addInplace (:121-123)
                else:
                    inp.grad = B.clone(g)              # :126
            output.grad = None

    def clear(self):
        for output, _, _ in self.entries:
            output.grad = None
        self.entries = []


class Ctx:
    def __init__(self, tape: Tape, backend: CpuRef):
        self.tape = tape
        self.backend = backend


def _record(ctx, data, inputs, backward):
    out = Variable(data, True)
    ctx.tape.record(out, inputs, backward)
    return out


def _reduce_broadcast(B, g, shape):
    """ops.ts:888-911."""
    shape = tuple(shape)
    if g.shape == shape:
        return g
    if len(shape) == 0 or (len(shape) == 1 and shape[0] == 1 and g.ndim > 1):
        return B.sum(g)
    r = g
    while r.ndim > len(shape):
        r = B.sum(r, 0)
    for i, d in enumerate(shape):
        if d == 1 and r.shape[i] != 1:
            r = B.sum(r, i, True)
    return r


# ── arithmetic (ops.ts:100-163) ─────────────────────────────────────────────
def add(ctx, a, b):
    sa, sb = a.data.shape, b.data.shape
    return _record(ctx, ctx.backend.add(a.data, b.data), [a, b],
                   lambda g, B, n: [_reduce_broadcast(B, g, sa), _reduce_broadcast(B, g, sb)])


def sub(ctx, a, b):
    sa, sb = a.data.shape, b.data.shape

    def bw(g, B, n):
        return [_reduce_broadcast(B, g, sa), _reduce_broadcast(B, B.neg(g), sb)]
    return _record(ctx, ctx.backend.sub(a.data, b.data), [a, b], bw)


def mul(ctx, a, b):
    ad, bd = a.data, b.data

    def bw(g, B, n):
        return [_reduce_broadcast(B, B.mul(g, bd), ad.shape), _reduce_broadcast(B, B.mul(g, ad), bd.shape)]
    return _record(ctx, ctx.backend.mul(ad, bd), [a, b], bw)


def div(ctx, a, b):
    ad, bd = a.data, b.data

    def bw(g, B, n):
        ga = B.div(g, bd)
        gb = B.neg(B.div(B.mul(g, ad), B.mul(bd, bd)))
        return [_reduce_broadcast(B, ga, ad.shape), _reduce_broadcast(B, gb, bd.shape)]
    return _record(ctx, ctx.backend.div(ad, bd), [a, b], bw)


def scale(ctx, a, s):
    return _record(ctx, ctx.backend.scale(a.data, s), [a], lambda g, B, n: [B.scale(g, s)])


def exp(ctx, a):
    out = ctx.backend.exp(a.data)
    return _record(ctx, out, [a], lambda g, B, n: [B.mul(g, out)])


def clamp(ctx, a, lo, hi):
    ad = a.data

    def bw(g, B, n):  # ops.ts:317-321
        return [np.where((ad > lo) & (ad < hi), g, f32(0)).astype(f32)]
    return _record(ctx, ctx.backend.clamp(ad, lo, hi), [a], bw)


def relu(ctx, a):
    ad = a.data
    return _record(ctx, ctx.backend.relu(ad), [a],
                   lambda g, B, n: [B.mul(g, (ad > 0).astype(f32))])


def sum_(ctx, a, axis=None, keepdims=False):
    sa = a.data.shape
    return _record(ctx, ctx.backend.sum(a.data, axis, keepdims), [a],
                   lambda g, B, n: [np.broadcast_to(g, sa).astype(f32).copy()])


def mean(ctx, a, axis=None, keepdims=False):
    sa = a.data.shape
    cnt = sa[axis] if axis is not None else a.data.size

    def bw(g, B, n):
        return [B.scale(np.broadcast_to(g, sa).astype(f32), 1 / cnt)]
    return _record(ctx, ctx.backend.mean(a.data, axis, keepdims), [a], bw)


# ── matmul family ───────────────────────────────────────────────────────────
def matmul(ctx, a, b):
    """ops.ts:165-189."""
    ad, bd = a.data, b.data

    def bw(g, B, needs):
        ga = B.matmul(g, B.transpose(bd, -2, -1)) if needs[0] else None
        gb = B.matmul(B.transpose(ad, -2, -1), g) if needs[1] else None
        return [ga, gb]
    return _record(ctx, ctx.backend.matmul(ad, bd), [a, b], bw)


def matmulTransposed(ctx, a, b):
    """ops.ts:197-234, fallback branch: C = A @ transpose(B)."""
    B0 = ctx.backend
    ad, bd = a.data, b.data
    out = B0.matmul(ad, B0.transpose(bd, -2, -1))

    def bw(g, B, needs):
        ga = B.matmul(g, bd) if needs[0] else None
        gb = B.matmul(B.transpose(g, -2, -1), ad) if needs[1] else None
        return [ga, gb]
    return _record(ctx, out, [a, b], bw)


_S2PI = math.sqrt(2 / math.pi)


def _gelu_grad(x32):
    x = x32.astype(f64)
    inner = _S2PI * (x + 0.044715 * x * x * x)
    t = np.tanh(inner)
    sech2 = 1 - t * t
    d_inner = _S2PI * (1 + 3 * 0.044715 * x * x)
    return 0.5 * (1 + t) + 0.5 * x * sech2 * d_inner


def gelu(ctx, a):
    """ops.ts:401-419: the derivative is stored to f32, then multiplied (two roundings)."""
    ad = a.data
    return _record(ctx, ctx.backend.gelu(ad), [a],
                   lambda g, B, n: [B.mul(g, _gelu_grad(ad).astype(f32))])


def matmulTransposedGelu(ctx, a, b):
    """ops.ts:426-487: gelu(A @ B^T) as one tape entry; grad*gelu' rounded once (:451-466)."""
    B0 = ctx.backend
    ad, bd = a.data, b.data
    mm = B0.matmul(ad, B0.transpose(bd, -2, -1))
    out = B0.gelu(mm)

    def bw(g, B, needs):
        dmm = (g.astype(f64) * _gelu_grad(mm)).astype(f32)
        ga = B.matmul(dmm, bd) if needs[0] else None
        gb = B.matmul(B.transpose(dmm, -2, -1), ad) if needs[1] else None
        return [ga, gb]
    return _record(ctx, out, [a, b], bw)


def silu(ctx, a):
    ad = a.data

    def bw(g, B, n):  # ops.ts:347-356
        x = ad.astype(f64)
        sig = 1 / (1 + np.exp(-x))
        return [(g.astype(f64) * (sig * (1 + x * (1 - sig)))).astype(f32)]
    return _record(ctx, ctx.backend.silu(ad), [a], bw)


def siluMul(ctx, a, b):
    """ops.ts:364-399, fallback branch: silu(a) stored, then multiplied by b."""
    B0 = ctx.backend
    ad, bd = a.data, b.data
    silu_a = B0.silu(ad)
    out = B0.mul(silu_a, bd)

    def bw(g, B, n):
        ga = B.mul(g, bd)
        x = ad.astype(f64)
        sig = 1 / (1 + np.exp(-x))
        da = (ga.astype(f64) * (sig * (1 + x * (1 - sig)))).astype(f32)
        db = B.mul(g, silu_a)
        return [da, db]
    return _record(ctx, out, [a, b], bw)


def softCap(ctx, a, cap):
    """ops.ts:329-340: tanh(x/cap)*cap composed from scale/clamp/exp/sub/add/div/scale."""
    x_scaled = scale(ctx, a, 2 / cap)
    x_safe = clamp(ctx, x_scaled, -80, 80)
    e2x = exp(ctx, x_safe)
    ones = Variable(ctx.backend.ones(e2x.data.shape), False)
    numer = sub(ctx, e2x, ones)
    denom = add(ctx, e2x, ones)
    return scale(ctx, div(ctx, numer, denom), cap)


# ── nn ──────────────────────────────────────────────────────────────────────
def embedding(ctx, weight, indices):
    """ops.ts:491-507."""
    wshape = weight.data.shape

    def bw(g, B, n):
        dw = np.zeros(wshape, dtype=f32)
        idx = np.ascontiguousarray(indices.reshape(-1).astype(np.int32))
        g2 = np.ascontiguousarray(g.reshape(-1, wshape[1]))
        lib().alpha_oracle_embedding_bwd_f32(dw.ctypes.data, idx.ctypes.data, g2.ctypes.data,
                                             idx.size, wshape[1])
        return [dw]
    return _record(ctx, ctx.backend.embedding(weight.data, indices), [weight], bw)


def layerNorm(ctx, x, weight, bias, eps):
    """ops.ts:509-571."""
    xd, wd = x.data, weight.data

    def bw(g, B, n):
        dim = xd.shape[-1]
        rows = xd.size // dim
        xc = np.ascontiguousarray(xd)
        gc = np.ascontiguousarray(g)
        dx = np.empty_like(xc)
        dw = np.empty(dim, dtype=f32)
        db = np.empty(dim, dtype=f32)
        lib().alpha_oracle_layernorm_bwd_f32(xc.ctypes.data, wd.ctypes.data, gc.ctypes.data,
                                             dx.ctypes.data, dw.ctypes.data, db.ctypes.data,
                                             rows, dim, float(eps))
        return [dx, dw.reshape(wd.shape), db.reshape(wd.shape)]
    return _record(ctx, ctx.backend.layerNorm(xd, wd, bias.data, eps), [x, weight, bias], bw)


def rmsNorm(ctx, x, weight, eps):
    """EXTENSION (no reference counterpart): y = x * rsqrt(mean(x^2)+eps) * w."""
    xd, wd = x.data, weight.data
    x64 = xd.astype(f64)
    dim = xd.shape[-1]
    inv = 1.0 / np.sqrt((x64 * x64).sum(-1, keepdims=True) / dim + eps)
    out = (x64 * inv * wd.astype(f64)).astype(f32)

    def bw(g, B, n):
        g64 = g.astype(f64)
        xhat = x64 * inv
        dw = (g64 * xhat).reshape(-1, dim).sum(0).astype(f32).reshape(wd.shape)
        dy = g64 * wd.astype(f64)
        s2 = (dy * xhat).sum(-1, keepdims=True)
        dx = (inv * (dy - xhat * s2 / dim)).astype(f32)
        return [dx, dw]
    return _record(ctx, out, [x, weight], bw)


def rope(ctx, x, n_head, theta=10000.0):
    """EXTENSION: rotary embedding on x [B,T,E] per head, pairing (d, d+D/2) — the
    "rotate-half" convention; angle(t, i) = t * theta^(-2i/D)."""
    xd = x.data
    Bn, T, E = xd.shape
    D = E // n_head
    half = D // 2
    inv_freq = theta ** (-np.arange(half, dtype=f64) * 2.0 / D)
    ang = np.arange(T, dtype=f64)[:, None] * inv_freq[None, :]
    cos, sin = np.cos(ang)[None, :, None, :], np.sin(ang)[None, :, None, :]

    def rot(v, sgn):
        v4 = v.astype(f64).reshape(Bn, T, n_head, D)
        a, b = v4[..., :half], v4[..., half:]
        o = np.concatenate([a * cos - sgn * b * sin, b * cos + sgn * a * sin], axis=-1)
        return o.reshape(Bn, T, E).astype(f32)
    return _record(ctx, rot(xd, 1.0), [x], lambda g, B, n: [rot(g, -1.0)])


def softmax(ctx, a, axis=-1):
    """ops.ts:687-700."""
    out = ctx.backend.softmax(a.data, axis)

    def bw(g, B, n):
        sg = B.mul(out, g)
        s = B.sum(sg, axis, True)
        diff = B.sub(g, np.broadcast_to(s, out.shape))
        return [B.mul(out, diff)]
    return _record(ctx, out, [a], bw)


def crossEntropy(ctx, logits, targets):
    """ops.ts:702-729."""
    ld = logits.data

    def bw(g, B, n):
        probs = B.softmax(ld, -1)
        N, C = ld.shape
        one_hot = np.zeros((N, C), dtype=f32)
        one_hot[np.arange(N), targets.reshape(-1)] = 1.0
        diff = B.sub(probs, one_hot)
        return [B.scale(diff, float(g.reshape(-1)[0]) / N)]
    return _record(ctx, ctx.backend.crossEntropy(ld, targets), [logits], bw)


def maskedFillEntry(ctx, scores, mask, value):
    """packages/model/src/gpt.ts:266-274 (a hand-recorded tape entry)."""
    out = Variable(ctx.backend.maskedFill(scores.data, mask, value), True)
    ctx.tape.record(out, [scores], lambda g, B, n: [B.maskedFill(g, mask, 0)])
    return out


# ── views ───────────────────────────────────────────────────────────────────
def slice_(ctx, a, starts, ends):
    """ops.ts:775-811 with cpu_ref's scatterSlice (cpu_ref.ts:640-656)."""
    orig = a.data.shape
    return _record(ctx, ctx.backend.slice(a.data, starts, ends), [a],
                   lambda g, B, n: [B.scatterSlice(g, orig, starts, ends)])


def sliceQkv(ctx, a):
    """ops.ts:818-858, fallback branch: three slices."""
    rows, c3 = a.data.shape
    D = c3 // 3
    return (slice_(ctx, a, [0, 0], [rows, D]), slice_(ctx, a, [0, D], [rows, 2 * D]),
            slice_(ctx, a, [0, 2 * D], [rows, 3 * D]))


def reshape(ctx, a, shape):
    orig = a.data.shape
    return _record(ctx, ctx.backend.reshape(a.data, shape), [a], lambda g, B, n: [B.reshape(g, orig)])


def transpose(ctx, a, d0, d1):
    return _record(ctx, ctx.backend.transpose(a.data, d0, d1), [a],
                   lambda g, B, n: [B.transpose(g, d0, d1)])
