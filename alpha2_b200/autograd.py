"""Tape autograd over a ``Backend`` — host-side mirror of ``packages/autograd/src``.

``Variable`` / ``Tape`` follow tape.ts:29-196: ops record a backward closure; ``backward``
walks the tape in reverse, accumulates gradients (first arrival is kept, later ones are
added in place) and releases consumed gradients and activations eagerly.  The op wrappers
follow ops.ts and take the backend's fused hooks exactly where the reference probes for
them (``matmulTransposed``, ``matmulTransposedA``, ``geluBackward``, ``layerNormBackward``,
``crossEntropyBackward``, ``embeddingBackward``, ``scatterSlice``, ``flashAttention`` ...).
Unlike the reference there is no JavaScript fallback arithmetic: a backend without a hook
raises, because this host layer exists to drive the CUDA library.

The second half of the file holds the fused ops that only this backend offers
(``linear``, ``linearGelu``, ``linearAdd``, ``attentionQkv``, ``lmHeadLoss``, ``rmsNorm``):
same math, fewer launches and no head-split / head-merge / slice copies.
"""
from __future__ import annotations

import sys
from typing import Callable, Sequence

from .backend import TensorData

_next_id = 0


class Variable:
    """tape.ts:29-41."""
    __slots__ = ("id", "data", "grad", "requiresGrad")

    def __init__(self, data: TensorData, requiresGrad: bool = False):
        global _next_id
        self.id = _next_id
        _next_id += 1
        self.data = data
        self.grad: TensorData | None = None
        self.requiresGrad = requiresGrad


class _Entry:
    __slots__ = ("output", "inputs", "backward", "cleanup", "in_place")

    def __init__(self, output, inputs, backward, cleanup=None, in_place=False):
        self.output, self.inputs, self.backward, self.cleanup = output, inputs, backward, cleanup
        self.in_place = in_place


class _Accumulated:
    """Returned by a backward closure in place of a gradient that it has already added into
    the input's existing ``grad`` (fused accumulation); the tape then has nothing to add."""
    __slots__ = ()


ACCUMULATED = _Accumulated()


def _exclusive(td: TensorData) -> bool:
    """True when no other TensorData shares td's device buffer."""
    return td._buf is not None and sys.getrefcount(td._buf) <= 2


class Tape:
    """tape.ts:43-200."""

    def __init__(self):
        self.entries: list[_Entry] = []

    def record(self, output: Variable, inputs: Sequence[Variable], backward: Callable, cleanup: Callable | None = None,
               in_place: bool = False):
        """``in_place``: the closure takes a fifth argument, the inputs' current gradients, and
        may add into them itself, returning ACCUMULATED for those inputs."""
        self.entries.append(_Entry(output, list(inputs), backward, cleanup, in_place))

    @property
    def size(self) -> int:
        return len(self.entries)

    def backward(self, loss: Variable, backend, releaseTensor: Callable | None = None,
                 initialGrad: TensorData | None = None, onEntryDone: Callable | None = None) -> None:
        loss.grad = initialGrad if initialGrad is not None else backend.ones(loss.data.shape, loss.data.dtype)

        def release_once(td: TensorData | None):
            # guards against double release when a closure aliases one gradient across
            # several inputs (tape.ts:66-73)
            if releaseTensor is None or td is None or td._released:
                return
            td._released = True
            releaseTensor(td)

        for entry in reversed(self.entries):
            out_grad = entry.output.grad
            if out_grad is None:
                if entry.cleanup:
                    entry.cleanup(releaseTensor)
                if onEntryDone is not None:
                    onEntryDone(entry)
                continue
            needs = [v.requiresGrad for v in entry.inputs]
            if entry.in_place:
                grads = entry.backward(out_grad, backend, releaseTensor, needs,
                                       [v.grad if v.requiresGrad else None for v in entry.inputs])
            else:
                grads = entry.backward(out_grad, backend, releaseTensor, needs)
            uses: dict[int, int] = {}
            for v, g in zip(entry.inputs, grads):
                if g is not None and g is not ACCUMULATED and v.requiresGrad:
                    uses[id(g)] = uses.get(id(g), 0) + 1
            for v, g in zip(entry.inputs, grads):
                if g is None or g is ACCUMULATED:
                    continue
                if not v.requiresGrad:
                    if id(g) not in uses:
                        release_once(g)
                    continue
                remaining = uses[id(g)] - 1
                uses[id(g)] = remaining
                if v.grad is not None:
                    backend.addInplace(v.grad, g)                     # tape.ts:118-120
                elif remaining == 0 and _exclusive(g):
                    # The reference clones here (tape.ts:126).  When nobody else can see the
                    # buffer the clone is a pure copy, so the buffer is adopted instead.
                    v.grad = TensorData(g.shape, g.dtype, g._buf, None)
                else:
                    v.grad = backend.clone(g)
                if remaining == 0:
                    release_once(g)
            release_once(out_grad)
            entry.output.grad = None
            if releaseTensor is not None:                             # tape.ts:146-150
                release_once(entry.output.data)
                entry.output.data = None
            if entry.cleanup:
                entry.cleanup(releaseTensor)
            if onEntryDone is not None:
                onEntryDone(entry)

    def clear(self, releaseTensor: Callable | None = None, keepOutput: Variable | None = None) -> None:
        for entry in self.entries:
            if releaseTensor is not None:
                keep = keepOutput is not None and entry.output.id == keepOutput.id
                if not keep and entry.output.data is not None:
                    releaseTensor(entry.output.data)
                if entry.output.grad is not None:
                    releaseTensor(entry.output.grad)
            if entry.cleanup:
                entry.cleanup(releaseTensor)
            entry.output.grad = None
        self.entries = []


class Ctx:
    __slots__ = ("tape", "backend", "dropoutRng", "release")

    def __init__(self, tape: Tape, backend, dropoutRng=None, release=None):
        self.tape, self.backend, self.dropoutRng, self.release = tape, backend, dropoutRng, release


def _record(ctx, data, inputs, backward, cleanup=None, in_place=False) -> Variable:
    out = Variable(data, True)
    ctx.tape.record(out, inputs, backward, cleanup, in_place)
    return out


class DropoutRng:
    """ops.ts:25-83: counter-based mask parameters (the mask itself is made on the device)."""

    def __init__(self, seed: int):
        self.seed = _i32(seed)
        self.counter = 0

    def reset(self, seed: int, counter: int = 0):
        self.seed, self.counter = _i32(seed), _i32(counter)

    def nextMaskParams(self):
        r = {"seed": self.seed, "counter": self.counter}
        self.counter += 1
        return r

    def saveCounter(self):
        return self.counter

    def restoreCounter(self, n):
        self.counter = n


def _i32(x: int) -> int:
    x &= 0xFFFFFFFF
    return x - (1 << 32) if x & 0x80000000 else x


# ── broadcasting helpers (ops.ts:888-944) ─────────────────────────────────────
def _reduce_broadcast(B, g: TensorData, shape) -> TensorData:
    shape = tuple(shape)
    if g.shape == shape:
        return g
    if len(shape) == 0 or (len(shape) == 1 and shape[0] == 1 and len(g.shape) > 1):
        return B.sum(g)
    r = g
    while len(r.shape) > len(shape):
        r = B.sum(r, 0)
    for i, d in enumerate(shape):
        if d == 1 and r.shape[i] != 1:
            r = B.sum(r, i, True)
    return r


def _broadcast_to(B, t: TensorData, shape) -> TensorData:
    shape = tuple(shape)
    return t if t.shape == shape else B.broadcast(t, shape)


# ── arithmetic (ops.ts:100-163) ───────────────────────────────────────────────
def add(ctx, a: Variable, b: Variable) -> Variable:
    sa, sb = a.data.shape, b.data.shape
    return _record(ctx, ctx.backend.add(a.data, b.data), [a, b],
                   lambda g, B, rel, n: [_reduce_broadcast(B, g, sa), _reduce_broadcast(B, g, sb)])


def sub(ctx, a, b):
    sa, sb = a.data.shape, b.data.shape
    return _record(ctx, ctx.backend.sub(a.data, b.data), [a, b],
                   lambda g, B, rel, n: [_reduce_broadcast(B, g, sa), _reduce_broadcast(B, B.neg(g), sb)])


def mul(ctx, a, b):
    ad, bd = a.data, b.data
    return _record(ctx, ctx.backend.mul(ad, bd), [a, b],
                   lambda g, B, rel, n: [_reduce_broadcast(B, B.mul(g, bd), ad.shape),
                                         _reduce_broadcast(B, B.mul(g, ad), bd.shape)])


def div(ctx, a, b):
    ad, bd = a.data, b.data

    def bw(g, B, rel, n):
        ga = B.div(g, bd)
        gb = B.neg(B.div(B.mul(g, ad), B.mul(bd, bd)))
        return [_reduce_broadcast(B, ga, ad.shape), _reduce_broadcast(B, gb, bd.shape)]
    return _record(ctx, ctx.backend.div(ad, bd), [a, b], bw)


def scale(ctx, a, s):
    return _record(ctx, ctx.backend.scale(a.data, s), [a], lambda g, B, rel, n: [B.scale(g, s)])


def neg(ctx, a):
    return _record(ctx, ctx.backend.neg(a.data), [a], lambda g, B, rel, n: [B.neg(g)])


def exp(ctx, a):
    out = ctx.backend.exp(a.data)
    return _record(ctx, out, [a], lambda g, B, rel, n: [B.mul(g, out)])


def log(ctx, a):
    ad = a.data
    return _record(ctx, ctx.backend.log(ad), [a], lambda g, B, rel, n: [B.div(g, ad)])


def sqrt(ctx, a):
    out = ctx.backend.sqrt(a.data)
    return _record(ctx, out, [a], lambda g, B, rel, n: [B.div(g, B.scale(out, 2))])


def relu(ctx, a):
    ad = a.data
    return _record(ctx, ctx.backend.relu(ad), [a], lambda g, B, rel, n: [B.reluBackward(ad, g)])


def clamp(ctx, a, lo, hi):
    ad = a.data
    return _record(ctx, ctx.backend.clamp(ad, lo, hi), [a], lambda g, B, rel, n: [B.clampBackward(ad, g, lo, hi)])


def softCap(ctx, a, cap):
    """ops.ts:287-327, native-kernel branch."""
    ad = a.data
    return _record(ctx, ctx.backend.softCap(ad, cap), [a], lambda g, B, rel, n: [B.softCapBackward(g, ad, cap)])


def silu(ctx, a):
    ad = a.data
    return _record(ctx, ctx.backend.silu(ad), [a], lambda g, B, rel, n: [B.siluBackward(ad, g)])


def siluMul(ctx, a, b):
    """ops.ts:364-399."""
    ad, bd = a.data, b.data
    return _record(ctx, ctx.backend.siluMul(ad, bd), [a, b], lambda g, B, rel, n: B.siluMulBackward(ad, bd, g))


def gelu(ctx, a):
    ad = a.data
    return _record(ctx, ctx.backend.gelu(ad), [a], lambda g, B, rel, n: [B.geluBackward(ad, g)])


def sum_(ctx, a, axis=None, keepdims=False):
    sa = a.data.shape

    def bw(g, B, rel, n):
        if axis is not None and not keepdims:      # re-insert the reduced axis before expanding
            ax = axis + len(sa) if axis < 0 else axis
            g = B.reshape(g, sa[:ax] + (1,) + sa[ax + 1:])
        return [_broadcast_to(B, g, sa)]
    return _record(ctx, ctx.backend.sum(a.data, axis, keepdims), [a], bw)


def mean(ctx, a, axis=None, keepdims=False):
    sa = a.data.shape
    cnt = a.data.size if axis is None else sa[axis]

    def bw(g, B, rel, n):
        if axis is not None and not keepdims:
            ax = axis + len(sa) if axis < 0 else axis
            g = B.reshape(g, sa[:ax] + (1,) + sa[ax + 1:])
        return [B.scale(_broadcast_to(B, g, sa), 1 / cnt)]
    return _record(ctx, ctx.backend.mean(a.data, axis, keepdims), [a], bw)


# ── matmul family (ops.ts:165-234, 426-487) ───────────────────────────────────
def matmul(ctx, a, b):
    ad, bd = a.data, b.data

    def bw(g, B, rel, needs):
        ga = gb = None
        if needs[0]:
            tb = B.transpose(bd, -2, -1)
            ga = B.matmul(g, tb)
        if needs[1]:
            if len(ad.shape) == 2:
                gb = B.matmulTransposedA(ad, g)
            else:
                gb = B.matmul(B.transpose(ad, -2, -1), g)
        return [ga, gb]
    return _record(ctx, ctx.backend.matmul(ad, bd), [a, b], bw)


def matmulTransposed(ctx, a, b):
    ad, bd = a.data, b.data

    def bw(g, B, rel, needs):
        ga = B.matmul(g, bd) if needs[0] else None
        gb = B.matmulTransposedA(g, ad) if needs[1] else None
        return [ga, gb]
    return _record(ctx, ctx.backend.matmulTransposed(ad, bd), [a, b], bw)


def matmulTransposedGelu(ctx, a, b):
    """ops.ts:426-487: one tape entry for gelu(A @ B^T); here also one launch."""
    ad, bd = a.data, b.data
    pre, act = ctx.backend.matmulTransposedGelu(ad, bd)
    state = {"pre": pre}

    def cleanup(release=None):
        if state["pre"] is not None and release:
            release(state["pre"])
        state["pre"] = None

    def bw(g, B, rel, needs):
        dmm = B.geluBackward(state["pre"], g)
        ga = B.matmul(dmm, bd) if needs[0] else None
        gb = B.matmulTransposedA(dmm, ad) if needs[1] else None
        return [ga, gb]
    return _record(ctx, act, [a, b], bw, cleanup)


# ── nn ops (ops.ts:491-729) ───────────────────────────────────────────────────
def embedding(ctx, weight: Variable, indices: TensorData) -> Variable:
    vocab = weight.data.shape[0]
    return _record(ctx, ctx.backend.embedding(weight.data, indices), [weight],
                   lambda g, B, rel, n: [B.embeddingBackward(indices, g, vocab)])


def layerNorm(ctx, x, weight, bias, eps):
    xd, wd = x.data, weight.data

    def bw(g, B, rel, n, acc):
        into = acc[0] if acc[0] is not None and acc[0].dtype == xd.dtype else None
        r = B.layerNormBackward(xd, wd, g, eps, into) if into is not None else B.layerNormBackward(xd, wd, g, eps)
        return [ACCUMULATED if into is not None else r["dx"], r["dw"], r["db"]]
    return _record(ctx, ctx.backend.layerNorm(xd, wd, bias.data, eps), [x, weight, bias], bw, in_place=True)


def dropout(ctx, a, p, training):
    if not training or p == 0:
        return a
    params = ctx.dropoutRng.nextMaskParams()
    mask = ctx.backend.dropoutMask(a.data.shape, params["seed"], params["counter"], p, a.data.dtype)
    return _record(ctx, ctx.backend.mul(a.data, mask), [a], lambda g, B, rel, n: [B.mul(g, mask)])


def residualDropoutAdd(ctx, residual, projected, p, training):
    """ops.ts:612-685."""
    if not training or p == 0:
        return add(ctx, residual, projected)
    params = ctx.dropoutRng.nextMaskParams()
    mask = ctx.backend.dropoutMask(projected.data.shape, params["seed"], params["counter"], p, projected.data.dtype)
    out = ctx.backend.residualDropoutAdd(residual.data, projected.data, mask)
    return _record(ctx, out, [residual, projected], lambda g, B, rel, n: [g, B.mul(g, mask)])


def softmax(ctx, a, axis=None):
    out = ctx.backend.softmax(a.data, axis)

    def bw(g, B, rel, n):
        sg = B.mul(out, g)
        s = B.sum(sg, -1 if axis is None else axis, True)
        diff = B.sub(g, _broadcast_to(B, s, out.shape))
        return [B.mul(out, diff)]
    return _record(ctx, out, [a], bw)


def crossEntropy(ctx, logits: Variable, targets: TensorData) -> Variable:
    ld = logits.data
    return _record(ctx, ctx.backend.crossEntropy(ld, targets), [logits],
                   lambda g, B, rel, n: [B.crossEntropyBackward(ld, targets, g)])


def flashAttention(ctx, q, k, v, T, scale_, softCap_):
    """ops.ts:741-770: Q, K, V [B*H, T, D]."""
    B0 = ctx.backend
    r = B0.flashAttention(q.data, k.data, v.data, T, scale_, softCap_)
    out, state = r["output"], {"lse": r["lse"]}
    qd, kd, vd = q.data, k.data, v.data

    def cleanup(release=None):
        if state["lse"] is not None and release:
            release(state["lse"])
        state["lse"] = None

    def bw(g, B, rel, needs):
        if state["lse"] is None:
            raise RuntimeError("flashAttention backward missing LSE buffer")
        d = B.flashAttentionBackward(qd, kd, vd, out, g, state["lse"], T, scale_, softCap_)
        return [d["dQ"] if needs[0] else None, d["dK"] if needs[1] else None, d["dV"] if needs[2] else None]
    return _record(ctx, out, [q, k, v], bw, cleanup)


# ── views (ops.ts:775-886) ────────────────────────────────────────────────────
def slice_(ctx, a, starts, ends):
    orig = a.data.shape
    return _record(ctx, ctx.backend.slice(a.data, starts, ends), [a],
                   lambda g, B, rel, n: [B.scatterSlice(g, orig, starts, ends)])


def sliceQkv(ctx, a):
    """ops.ts:818-858: one fused split forward, three scatterSlice backward."""
    rows, c3 = a.data.shape
    D = c3 // 3
    orig = a.data.shape
    qd, kd, vd = ctx.backend.sliceQkv(a.data)
    mk = lambda data, lo: _record(ctx, data, [a],
                                  lambda g, B, rel, n: [B.scatterSlice(g, orig, [0, lo], [rows, lo + D])])
    return mk(qd, 0), mk(kd, D), mk(vd, 2 * D)


def reshape(ctx, a, shape):
    orig = a.data.shape
    return _record(ctx, ctx.backend.reshape(a.data, shape), [a], lambda g, B, rel, n: [B.reshape(g, orig)])


def transpose(ctx, a, d0, d1):
    return _record(ctx, ctx.backend.transpose(a.data, d0, d1), [a], lambda g, B, rel, n: [B.transpose(g, d0, d1)])


# ══ fused ops of this backend (no tape-level counterpart in the reference) ═════════════
def linear(ctx, x: Variable, w: Variable) -> Variable:
    """x [..., K] @ w[N, K]^T.  With bf16 activations `w` carries a bf16 shadow
    (``w.data.shadow``); its gradient is produced in f32 for the f32 AdamW state."""
    xd = x.data
    wd = _compute_weight(w)

    def bw(g, B, rel, needs, acc):
        ga = _dx_gemm(B, g, wd, acc[0]) if needs[0] else None
        gb = _dw_gemm(B, g, xd, acc[1]) if needs[1] else None
        return [ga, gb]
    return _record(ctx, ctx.backend.matmulTransposed(xd, wd), [x, w], bw, in_place=True)


def _dw_gemm(B, g: TensorData, xd: TensorData, acc: TensorData | None):
    """g^T @ x; added inside the GEMM to a weight gradient that already exists (accumulated
    micro-steps, shared weights) when the backend can."""
    if acc is not None and hasattr(B, "matmulInto") and acc.dtype == ("f32" if g.dtype == "bf16" else g.dtype):
        B.matmulTransposedA(g, xd, into=acc)
        return ACCUMULATED
    return B.matmulTransposedA(g, xd)


def _dx_gemm(B, g: TensorData, wd: TensorData, acc: TensorData | None):
    """g @ w; added in the GEMM epilogue to an input gradient that another consumer already left."""
    if acc is not None and hasattr(B, "matmulInto") and acc.dtype == g.dtype and len(wd.shape) == 2:
        B.matmulInto(g, wd, acc)
        return ACCUMULATED
    return B.matmul(g, wd)


def linearGelu(ctx, x: Variable, w: Variable) -> Variable:
    """gelu(x @ w^T) from one GEMM launch (pre-activation kept for backward); backward fuses
    gelu' into the following dX GEMM is left to linearAdd's consumer: here dPre = g*gelu'(pre)."""
    xd = x.data
    wd = _compute_weight(w)
    pre, act = ctx.backend.matmulTransposedGelu(xd, wd)

    def bw(g, B, rel, needs):
        dpre = B.geluBackward(pre, g)
        ga = B.matmul(dpre, wd) if needs[0] else None
        gb = B.matmulTransposedA(dpre, xd) if needs[1] else None
        return [ga, gb]
    return _record(ctx, act, [x, w], bw)


def linearAdd(ctx, x: Variable, w: Variable, residual: Variable) -> Variable:
    """residual + x @ w^T with the add in the GEMM epilogue."""
    xd = x.data
    wd = _compute_weight(w)

    def bw(g, B, rel, needs, acc):
        ga = B.matmul(g, wd) if needs[0] else None
        gb = _dw_gemm(B, g, xd, acc[1]) if needs[1] else None
        return [ga, gb, g]
    return _record(ctx, ctx.backend.matmulTransposedAdd(xd, wd, residual.data), [x, w, residual], bw, in_place=True)


def mlpGelu(ctx, x: Variable, w1: Variable, w2: Variable, residual: Variable) -> Variable:
    """residual + gelu(x @ w1^T) @ w2^T as one tape entry and two launches forward
    (GELU and the residual add live in the GEMM epilogues).  Backward is five GEMMs and no
    elementwise pass: d_pre = (g @ w2) * gelu'(pre) comes out of one GEMM epilogue."""
    xd = x.data
    w1d, w2d = _compute_weight(w1), _compute_weight(w2)
    B0 = ctx.backend
    pre, act = B0.matmulTransposedGelu(xd, w1d)
    out = B0.matmulTransposedAdd(act, w2d, residual.data)

    def bw(g, B, rel, needs, acc):
        dpre = B.matmulGeluBackward(g, w2d, pre)
        dx = B.matmul(dpre, w1d) if needs[0] else None
        if needs[1] and needs[2]:
            # both weight gradients in one launch (each alone would have to split its K)
            dw2, dw1 = _pair_dw(B, (g, act, acc[2]), (dpre, xd, acc[1]))
        else:
            dw2 = _dw_gemm(B, g, act, acc[2]) if needs[2] else None
            dw1 = _dw_gemm(B, dpre, xd, acc[1]) if needs[1] else None
        return [dx, dw1, dw2, g]
    return _record(ctx, out, [x, w1, w2, residual], bw, in_place=True)


def _compute_weight(w: Variable) -> TensorData:
    sh = getattr(w, "shadow", None)
    return sh if sh is not None else w.data


class Param(Variable):
    """A trainable Variable that may carry a bf16 shadow of its f32 master copy."""
    __slots__ = ("shadow", "name")

    def __init__(self, data: TensorData, name: str = "", shadow: TensorData | None = None):
        super().__init__(data, True)
        self.shadow = shadow
        self.name = name


def attentionQkv(ctx, qkv: Variable, Bn: int, T: int, H: int, scale_: float, softCap_: float) -> Variable:
    """Causal MHA on the fused projection [B*T, 3E] -> [B*T, E] (see CudaBackend.attentionQkv)."""
    qd = qkv.data
    out, lse = ctx.backend.attentionQkv(qd, Bn, T, H, scale_, softCap_)
    return _record(ctx, out, [qkv],
                   lambda g, B, rel, n: [B.attentionQkvBackward(qd, out, g, lse, Bn, T, H, scale_, softCap_)])


def _pair_dw(B, first, second):
    """Two weight gradients (g, x, acc) -> g^T @ x, in one launch where the backend offers it
    for these operands (``pairSupported``); otherwise one GEMM each."""
    (g0, x0, a0), (g1, x1, a1) = first, second
    if hasattr(B, "matmulTransposedAPair") and B.pairSupported(first, second):
        r0, r1 = B.matmulTransposedAPair((g0, x0, a0), (g1, x1, a1))
        return (ACCUMULATED if a0 is not None else r0), (ACCUMULATED if a1 is not None else r1)
    return _dw_gemm(B, g0, x0, a0), _dw_gemm(B, g1, x1, a1)


def attentionBlock(ctx, x: Variable, wqkv: Variable, wo: Variable, residual: Variable, Bn: int, T: int, H: int,
                   scale_: float, softCap_: float, ropeTheta: float | None = None) -> Variable:
    """residual + attention(x @ wqkv^T) @ wo^T as one tape entry: the fused projection (with
    q and k rotated in place when ``ropeTheta`` is given), causal attention read in place from
    it, the output projection and the residual add in its GEMM's epilogue.  Backward: dO = g @ wo
    with the row-dots dO.att from that GEMM's epilogue where the backend can, the attention
    backward, the transposed rotation in place, then both weight gradients — g^T att and
    dqkv^T x — in one launch (9 + 27 tiles that alone would each leave most of the device idle),
    and dx = dqkv @ wqkv."""
    B0 = ctx.backend
    xd = x.data
    wqd, wod = _compute_weight(wqkv), _compute_weight(wo)
    qd = B0.matmulTransposed(xd, wqd)
    E3 = qd.shape[-1]
    D = E3 // 3 // H
    if ropeTheta is not None:
        B0.rope(qd, Bn, T, 2 * H, D, E3, 0, ropeTheta)            # q and k: 2H heads side by side
    att, lse = B0.attentionQkv(qd, Bn, T, H, scale_, softCap_)
    out = B0.matmulTransposedAdd(att, wod, residual.data)
    state = {"att": att, "lse": lse, "qkv": qd}

    def cleanup(release=None):      # projection, attention output and row statistics live inside this entry
        for k in ("att", "lse", "qkv"):
            if state[k] is not None and release:
                release(state[k])
            state[k] = None

    def bw(g, B, rel, needs, acc):
        att, lse, qd = state["att"], state["lse"], state["qkv"]
        if hasattr(B, "matmulRowdot") and B.rowdotSupported(g, att, H):
            dO, delta = B.matmulRowdot(g, wod, att, T, H)
            dqkv = B.attentionQkvBackward(qd, att, dO, lse, Bn, T, H, scale_, softCap_, delta=delta)
            if rel:
                rel(delta)
        else:
            dO = B.matmul(g, wod)
            dqkv = B.attentionQkvBackward(qd, att, dO, lse, Bn, T, H, scale_, softCap_)
        if rel:
            rel(dO)
        if ropeTheta is not None:
            B.rope(dqkv, Bn, T, 2 * H, D, E3, 0, ropeTheta, inverse=True)
        if needs[1] and needs[2]:
            dwo, dwq = _pair_dw(B, (g, att, acc[2]), (dqkv, xd, acc[1]))
        else:
            dwo = _dw_gemm(B, g, att, acc[2]) if needs[2] else None
            dwq = _dw_gemm(B, dqkv, xd, acc[1]) if needs[1] else None
        dx = _dx_gemm(B, dqkv, wqd, acc[0]) if needs[0] else None
        if rel:
            rel(dqkv)
        return [dx, dwq, dwo, g]
    return _record(ctx, out, [x, wqkv, wo, residual], bw, cleanup, in_place=True)


def ropeQk(ctx, qkv: Variable, Bn: int, T: int, H: int, theta: float = 10000.0) -> Variable:
    """Rotary embedding of the q and k column blocks of [B*T, 3E], in place (v is not touched);
    the backward is the transposed rotation of the gradient, in place as well.  The projection
    that produced ``qkv`` needs its input and weight for its own backward, not its output, and
    the gradient that arrives here belongs to this entry alone, so neither pass needs a copy:
    4E instead of 6E elements of traffic per token and no allocation.  One launch each way."""
    E3 = qkv.data.shape[-1]
    D = E3 // 3 // H
    ctx.backend.rope(qkv.data, Bn, T, 2 * H, D, E3, 0, theta)      # q and k: 2H heads side by side

    def bw(g, B, rel, n):
        B.rope(g, Bn, T, 2 * H, D, E3, 0, theta, inverse=True)
        return [g]
    return _record(ctx, qkv.data, [qkv], bw)


def rmsNorm(ctx, x, weight, eps):
    xd, wd = x.data, weight.data

    def bw(g, B, rel, n, acc):
        into = acc[0] if acc[0] is not None and acc[0].dtype == xd.dtype else None
        r = B.rmsNormBackward(xd, wd, g, eps, into) if into is not None else B.rmsNormBackward(xd, wd, g, eps)
        return [ACCUMULATED if into is not None else r["dx"], r["dw"]]
    return _record(ctx, ctx.backend.rmsNorm(xd, wd, eps), [x, weight], bw, in_place=True)


def embeddingPos(ctx, wte: Variable, wpe: Variable, tokens: TensorData) -> Variable:
    """wte[tokens] + wpe[arange(T)] as one kernel; backward: scatter-add into wte, and the
    batch-sum of the gradient into wpe (every position index occurs once per batch row)."""
    B0 = ctx.backend
    Bn, T = tokens.shape
    vocab, dim = wte.data.shape
    out = B0.reshape(B0.embeddingPos(_compute_weight(wte), _compute_weight(wpe), tokens), (Bn * T, dim))

    def bw(g, B, rel, needs, acc):
        if acc[0] is not None and acc[0].dtype == "f32":     # tied head: add into the head's dW
            B.embeddingBackward(tokens, g, vocab, out=acc[0])
            dwte = ACCUMULATED
        else:
            dwte = B.embeddingBackward(tokens, g, vocab)
        gp = B.sum(B.reshape(g, (Bn, T * dim)), 0)          # [T*dim], storage dtype
        dwpe = B.reshape(gp, (T, dim))
        if dwpe.dtype != "f32":
            dwpe = B.castDtype(dwpe, "f32")
        if wpe.data.shape[0] != T:                          # blockSize > T: pad rows with zeros
            full = B.zeros(wpe.data.shape, "f32")
            B.lib.alpha_d2d(full.ptr, dwpe.ptr, dwpe.nbytes)
            dwpe = full
        return [dwte, dwpe]
    return _record(ctx, out, [wte, wpe], bw, in_place=True)


def lmHeadLoss(ctx, x: Variable, w: Variable, targets: TensorData, gradScale: float = 1.0) -> Variable:
    """mean cross-entropy of (x @ w^T) against targets: head GEMM + fused softmax-CE
    forward/backward in one pass over a row-padded logits buffer; the logits gradient is
    ready when forward returns and is consumed by the two backward GEMMs."""
    xd = x.data
    wd = _compute_weight(w)
    loss, dlogits, ld = ctx.backend.lmHeadLoss(xd, wd, targets, gradScale)
    state = {"dl": dlogits}

    def cleanup(release=None):
        state["dl"] = None

    def bw(g, B, rel, needs):
        # g is the upstream scalar (ones unless loss scaling is in use; it is folded into
        # gradScale by the caller, as trainer.ts:1297 folds scaling into the optimizer)
        dx, dw = B.lmHeadBackward(state["dl"], ld, xd, wd, None)
        state["dl"] = None
        return [dx, dw]
    return _record(ctx, loss, [x, w], bw, cleanup)


def checkpoint(ctx, fn, input: Variable) -> Variable:
    """Activation checkpointing (packages/autograd/src/checkpoint.ts:36-87): run ``fn(innerCtx,
    input)`` on a throw-away tape, keep only its output, and record ONE entry on the outer tape
    whose backward re-runs ``fn`` on a fresh tape, backpropagates through it (parameter
    gradients accumulate directly on the captured parameters) and returns the input gradient.
    Memory per segment drops from all its intermediates to its input; compute grows by one
    forward of the segment.  Only for deterministic segments (dropout 0)."""
    B = ctx.backend
    tmp = Ctx(Tape(), B, ctx.dropoutRng, None)
    tmp_out = fn(tmp, input)
    out_data = tmp_out.data
    # The trainable parameters the segment reads.  They are listed after the real input on
    # the outer entry so that whoever watches the tape (the data-parallel hand-off counts the
    # entries that feed each parameter) sees that this entry's backward finalises them; the
    # closure returns one gradient only, so the tape itself never touches the extra inputs.
    captured: list = []
    seen = set()
    for e in tmp.tape.entries:
        for v in e.inputs:
            if isinstance(v, Param) and v.id not in seen:
                seen.add(v.id)
                captured.append(v)
    tmp.tape.clear(ctx.release, tmp_out)                      # intermediates go, the output stays

    def bw(g, backend, release, needs):
        re_input = Variable(input.data, True)
        re = Ctx(Tape(), backend, ctx.dropoutRng, None)
        re_out = fn(re, re_input)
        re.tape.backward(re_out, backend, release, backend.clone(g))
        grad = re_input.grad
        re_input.grad = None
        re.tape.clear(release)
        return [grad if grad is not None else backend.zeros(input.data.shape, input.data.dtype)]
    return _record(ctx, out_data, [input] + captured, bw)
