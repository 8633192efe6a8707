"""A numpy stand-in for CudaBackend, for CPU tests of the host layer only.

The reference tests its GPU lifetime logic without a GPU by running the tape on
CpuRefBackend with a release spy (packages/tests/src/memory-leak.test.ts:20-25).  This is
the same idea: every method the host layer (autograd / gpt / trainer / optimizers) calls
on the backend exists here with float64 numpy math, so the tape, the fused-op backward
closures, the schedule and the optimizer wiring can be checked against the oracle on CPU.
It is test infrastructure: nothing in the package imports it and it never runs on a GPU.
"""
from __future__ import annotations

import math

import numpy as np

from alpha2_b200.backend import TensorData
from oracle.gpt import flash_attention_dense, flash_attention_dense_backward

f32, f64 = np.float32, np.float64


def T(arr, dtype="f32"):
    if dtype == "i32":
        arr = np.ascontiguousarray(arr, dtype=np.int32)
    else:
        arr = np.ascontiguousarray(arr, dtype=f32)
    return TensorData(arr.shape, dtype, None, arr)


def _gelu(x):
    c = math.sqrt(2 / math.pi)
    return 0.5 * x * (1 + np.tanh(c * (x + 0.044715 * x ** 3)))


def _gelu_grad(x):
    c = math.sqrt(2 / math.pi)
    t = np.tanh(c * (x + 0.044715 * x ** 3))
    return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * c * (1 + 3 * 0.044715 * x * x)


class NumpyBackend:
    name = "numpy_fake"
    device = 0
    param_grads_f32 = True

    def __init__(self):
        self.released = 0
        self.ops = 0
        self.lib = None

    def _o(self, arr, dtype="f32"):
        self.ops += 1
        return T(arr, dtype)

    # lifetime
    def releaseGpuTensor(self, td):
        self.released += 1
        td._host = None

    def resetStepOps(self): self._mark = self.ops
    @property
    def gpuOpsThisStep(self): return self.ops - getattr(self, "_mark", 0)
    def syncGpu(self): pass
    def flush(self): pass

    # creation
    def zeros(self, shape, dtype="f32"): return self._o(np.zeros(shape), dtype)
    def ones(self, shape, dtype="f32"): return self._o(np.ones(shape), dtype)
    def full(self, shape, v, dtype="f32"): return self._o(np.full(shape, v), dtype)
    def upload(self, arr, dtype=None): return T(arr, dtype or ("i32" if np.issubdtype(arr.dtype, np.integer) else "f32"))
    def fromArray(self, data, shape, dtype="f32"): return T(np.asarray(data).reshape(shape), dtype)
    def clone(self, a): return self._o(a.data.copy(), a.dtype)
    def castDtype(self, a, dtype): return self._o(a.data.copy(), "f32")

    def castInto(self, src, dst):
        self.ops += 1
        dst._host = np.asarray(src.data, dtype=f32).reshape(dst.shape).copy()

    # elementwise
    def add(self, a, b): return self._o(a.data.astype(f64) + b.data)
    def sub(self, a, b): return self._o(a.data.astype(f64) - b.data)
    def mul(self, a, b): return self._o(a.data.astype(f64) * b.data)
    def div(self, a, b): return self._o(a.data.astype(f64) / b.data)
    def neg(self, a): return self._o(-a.data)
    def exp(self, a): return self._o(np.exp(a.data.astype(f64)))
    def scale(self, a, s): return self._o(a.data.astype(f64) * s)
    def gelu(self, a): return self._o(_gelu(a.data.astype(f64)))
    def geluBackward(self, x, g): return self._o(g.data.astype(f64) * _gelu_grad(x.data.astype(f64)))
    def relu(self, a): return self._o(np.maximum(a.data, 0))
    def reluBackward(self, x, g): return self._o(np.where(x.data > 0, g.data, 0))
    def softCap(self, a, cap): return self._o(np.tanh(a.data.astype(f64) / cap) * cap)
    def softCapBackward(self, g, x, cap): return self._o(g.data * (1 - np.tanh(x.data.astype(f64) / cap) ** 2))

    def siluMul(self, a, b):
        x = a.data.astype(f64)
        return self._o(x / (1 + np.exp(-x)) * b.data)

    def siluMulBackward(self, a, b, g):
        x, y, gg = a.data.astype(f64), b.data.astype(f64), g.data.astype(f64)
        s = 1 / (1 + np.exp(-x))
        return [self._o(gg * y * (s * (1 + x * (1 - s)))), self._o(gg * x * s)]

    def addInplace(self, a, b):
        self.ops += 1
        a._host = (a.data.astype(f64) + b.data.reshape(a.shape)).astype(f32)

    def broadcast(self, a, shape): return self._o(np.broadcast_to(a.data, shape))

    # matmul
    def matmul(self, a, b): return self._o(a.data.astype(f64) @ b.data.astype(f64))
    def matmulTransposed(self, a, b): return self._o(a.data.astype(f64) @ b.data.astype(f64).T)

    def matmulTransposedA(self, a, b, into=None):
        A = a.data.astype(f64).reshape(-1, a.shape[-1])
        Bm = b.data.astype(f64).reshape(-1, b.shape[-1])
        if into is not None:
            self.ops += 1
            into._host = (into.data.astype(f64) + A.T @ Bm).astype(f32)
            return into
        return self._o(A.T @ Bm)

    def pairSupported(self, first, second):
        return True

    def matmulTransposedAPair(self, first, second):
        """Both weight gradients "in one launch": the host logic around it (ACCUMULATED, hand-off)
        is what the CPU tests exercise."""
        self.pair_calls = getattr(self, "pair_calls", 0) + 1
        return [self.matmulTransposedA(a, b, into) for a, b, into in (first, second)]

    def matmulInto(self, a, b, into):
        self.ops += 1
        into._host = (into.data.astype(f64) + (a.data.astype(f64) @ b.data.astype(f64)).reshape(into.shape)).astype(f32)
        return into

    def matmulTransposedGelu(self, a, b):
        pre = a.data.astype(f64) @ b.data.astype(f64).T
        return self._o(pre), self._o(_gelu(pre))

    def matmulTransposedAdd(self, a, b, r):
        return self._o(r.data + a.data.astype(f64) @ b.data.astype(f64).T)

    def matmulGeluBackward(self, g, w, pre):
        return self._o((g.data.astype(f64) @ w.data.astype(f64)) * _gelu_grad(pre.data.astype(f64)))

    # reductions
    def sum(self, a, axis=None, keepdims=False):
        return self._o(np.sum(a.data.astype(f64), axis=axis, keepdims=keepdims))

    def softmax(self, a, axis=None):
        x = a.data.astype(f64)
        e = np.exp(x - x.max(-1, keepdims=True))
        return self._o(e / e.sum(-1, keepdims=True))

    def totalSumOfSquares(self, ts):
        return self._o(np.array(sum(float(np.sum(t.data.astype(f64) ** 2)) for t in ts)))

    # nn
    def embedding(self, w, idx): return self._o(w.data[idx.data.reshape(-1)].reshape(idx.shape + (w.shape[1],)))

    def embeddingPos(self, wte, wpe, tok):
        Bn, Tn = tok.shape
        return self._o(wte.data[tok.data] + wpe.data[np.arange(Tn)][None])

    def embeddingBackward(self, idx, g, vocab, out=None):
        dw = np.zeros((vocab, g.shape[-1]), f64)
        np.add.at(dw, idx.data.reshape(-1), g.data.reshape(-1, g.shape[-1]).astype(f64))
        if out is not None:
            self.ops += 1
            out._host = (out.data.astype(f64) + dw).astype(f32)
            return out
        return self._o(dw)

    def _ln_stats(self, x, eps, rms):
        mean = 0.0 if rms else x.mean(-1, keepdims=True)
        var = ((x - mean) ** 2).mean(-1, keepdims=True)
        return mean, 1 / np.sqrt(var + eps)

    def layerNorm(self, x, w, b, eps):
        X = x.data.astype(f64)
        m, r = self._ln_stats(X, eps, False)
        return self._o((X - m) * r * w.data + b.data)

    def layerNormBackward(self, x, w, g, eps, dxInto=None, rms=False):
        X, G = x.data.astype(f64), g.data.astype(f64)
        dim = X.shape[-1]
        m, r = self._ln_stats(X, eps, rms)
        xhat = (X - m) * r
        dy = G * w.data
        s1 = 0.0 if rms else dy.sum(-1, keepdims=True)
        s2 = (dy * xhat).sum(-1, keepdims=True)
        dx = r * (dy - (s1 + xhat * s2) / dim)
        if dxInto is not None:
            self.ops += 1
            dxInto._host = (dxInto.data.astype(f64) + dx).astype(f32)
            return {"dx": dxInto, "dw": self._o((G * xhat).reshape(-1, dim).sum(0)),
                    "db": self._o(G.reshape(-1, dim).sum(0))}
        return {"dx": self._o(dx), "dw": self._o((G * xhat).reshape(-1, dim).sum(0)),
                "db": self._o(G.reshape(-1, dim).sum(0))}

    def rmsNorm(self, x, w, eps):
        X = x.data.astype(f64)
        _, r = self._ln_stats(X, eps, True)
        return self._o(X * r * w.data)

    def rmsNormBackward(self, x, w, g, eps, dxInto=None):
        r = self.layerNormBackward(x, w, g, eps, dxInto, rms=True)
        return {"dx": r["dx"], "dw": r["dw"]}

    def rope(self, x, batch, Tn, heads, D, ld, col_offset=0, theta=10000.0, inverse=False):
        self.ops += 1
        a = x.data.astype(f64).copy().reshape(batch, Tn, ld)
        half = D // 2
        inv = theta ** (-np.arange(half) * 2.0 / D)
        ang = np.arange(Tn)[:, None] * inv[None]
        c, s = np.cos(ang)[None, :, None], np.sin(ang)[None, :, None] * (-1 if inverse else 1)
        blk = a[:, :, col_offset:col_offset + heads * D].reshape(batch, Tn, heads, D)
        p, q = blk[..., :half].copy(), blk[..., half:].copy()
        blk[..., :half], blk[..., half:] = p * c - q * s, q * c + p * s
        a[:, :, col_offset:col_offset + heads * D] = blk.reshape(batch, Tn, heads * D)
        x._host = a.reshape(x.shape).astype(f32)

    def ropeQkv(self, qkv, batch, Tn, heads, theta=10000.0, inverse=False):
        E3 = qkv.shape[-1]
        E = E3 // 3
        out = self.clone(qkv)
        self.rope(out, batch, Tn, heads, E // heads, E3, 0, theta, inverse)
        self.rope(out, batch, Tn, heads, E // heads, E3, E, theta, inverse)
        return out

    def crossEntropy(self, logits, targets):
        x = logits.data.astype(f64)
        lse = np.log(np.exp(x - x.max(-1, keepdims=True)).sum(-1)) + x.max(-1)
        return self._o(np.array((lse - x[np.arange(x.shape[0]), targets.data]).mean()))

    def crossEntropyBackward(self, logits, targets, g):
        p = self.softmax(logits).data.astype(f64)
        p[np.arange(p.shape[0]), targets.data] -= 1
        return self._o(p * float(g.data.reshape(-1)[0]) / p.shape[0])

    def lmHeadLoss(self, x, w, targets, gradScale=1.0):
        logits = T(x.data.astype(f64) @ w.data.astype(f64).T)
        loss = self.crossEntropy(logits, targets)
        dl = self.crossEntropyBackward(logits, targets, T(np.array([gradScale])))
        return loss, dl, w.shape[0]

    def lmHeadBackward(self, dl, ld, x, w, dw_out):
        return self._o(dl.data.astype(f64) @ w.data), self._o(dl.data.astype(f64).T @ x.data)

    # layout
    def reshape(self, a, shape): return T(a.data.reshape(shape), a.dtype)
    def transpose(self, a, d0, d1): return self._o(np.swapaxes(a.data, d0, d1))
    def slice(self, a, s, e): return self._o(a.data[:, s[1]:e[1]])

    def scatterSlice(self, g, shape, s, e):
        out = np.zeros(shape, f32)
        out[:, s[1]:e[1]] = g.data
        return self._o(out)

    def sliceQkv(self, a):
        d = a.shape[1] // 3
        return tuple(self._o(a.data[:, i * d:(i + 1) * d]) for i in range(3))

    def causalMask(self, n):
        m = np.zeros((n, n), f32)
        m[np.triu_indices(n, 1)] = -np.inf
        return self._o(m)

    def maskedFill(self, a, mask, v):
        out = a.data.copy().reshape(-1, mask.size)
        out[:, mask.data.reshape(-1) != 0] = v
        return self._o(out.reshape(a.shape))

    # attention
    def flashAttention(self, Q, K, V, Tn, scale, cap):
        o, lse = flash_attention_dense(Q.data, K.data, V.data, Tn, scale, cap)
        return {"output": self._o(o), "lse": self._o(lse)}

    def flashAttentionBackward(self, Q, K, V, O, dO, lse, Tn, scale, cap):
        dq, dk, dv = flash_attention_dense_backward(Q.data, K.data, V.data, O.data, dO.data, lse.data, Tn, scale, cap)
        return {"dQ": self._o(dq), "dK": self._o(dk), "dV": self._o(dv)}

    def _split(self, qkv, Bn, Tn, H):
        E = qkv.shape[-1] // 3
        D = E // H
        parts = [qkv.data[:, i * E:(i + 1) * E].reshape(Bn, Tn, H, D).transpose(0, 2, 1, 3).reshape(Bn * H, Tn, D)
                 for i in range(3)]
        return parts, E, D

    def attentionQkv(self, qkv, Bn, Tn, H, scale, cap):
        (q, k, v), E, D = self._split(qkv, Bn, Tn, H)
        o, lse = flash_attention_dense(q, k, v, Tn, scale, cap)
        out = o.reshape(Bn, H, Tn, D).transpose(0, 2, 1, 3).reshape(Bn * Tn, E)
        return self._o(out), self._o(lse)

    def attentionQkvBackward(self, qkv, out, dout, lse, Bn, Tn, H, scale, cap):
        (q, k, v), E, D = self._split(qkv, Bn, Tn, H)
        hs = lambda t: t.data.reshape(Bn, Tn, H, D).transpose(0, 2, 1, 3).reshape(Bn * H, Tn, D)
        dq, dk, dv = flash_attention_dense_backward(q, k, v, hs(out), hs(dout), lse.data, Tn, scale, cap)
        merge = lambda t: t.reshape(Bn, H, Tn, D).transpose(0, 2, 1, 3).reshape(Bn * Tn, E)
        return self._o(np.concatenate([merge(dq), merge(dk), merge(dv)], axis=1))

    # optimizer
    def _adam(self, p, g, m, v, lr, b1, b2, eps, wd, bc1, bc2, gs):
        P, G, M, V = (t.data.astype(f64) for t in (p, g, m, v))
        G = G.reshape(P.shape) * gs
        if wd > 0:
            P = P - lr * wd * P
        M = b1 * M + (1 - b1) * G
        V = b2 * V + (1 - b2) * G * G
        P = P - lr * (M / bc1) / (np.sqrt(V / bc2) + eps)
        p._host, m._host, v._host = P.astype(f32), M.astype(f32), V.astype(f32)

    def adamwStep(self, p, g, m, v, lr, b1, b2, eps, wd, bc1, bc2, gradScale=1.0, shadow=None):
        self.ops += 1
        self._adam(p, g, m, v, lr, b1, b2, eps, wd, bc1, bc2, gradScale)

    def adamwStepMulti(self, entries, lr, b1, b2, eps, bc1, bc2, gradScale=1.0, clipSumSq=None, maxNorm=0.0):
        self.ops += 1
        gs = gradScale
        if clipSumSq is not None:
            gn = math.sqrt(float(clipSumSq.data.reshape(-1)[0])) * abs(gradScale)
            if not math.isfinite(gn):
                return                          # the step is skipped: p, m, v stay as they are
            if maxNorm > 0 and gn > maxNorm:
                gs *= maxNorm / gn
        for (p, g, m, v, wd, sh) in entries:
            self._adam(p, g, m, v, lr, b1, b2, eps, wd, bc1, bc2, gs)
