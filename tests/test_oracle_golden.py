"""The oracle against every known-answer test the reference holds for the train-step path.

Each test names the reference test it repeats (packages/tests/src/*.test.ts).
"""
import math

import numpy as np
import pytest

from oracle import autograd as ag
from oracle.autograd import Ctx, Tape, Variable
from oracle.cpu_ref import CpuRef, PySeededRng, SeededRng
from oracle.train import AdamW, adamw_reference_loop

B = CpuRef()
f32 = np.float32


# ── packages/tests/src/tensor.test.ts ───────────────────────────────────────
def test_zeros_ones_fromarray():                      # tensor.test.ts:7-25
    t = B.zeros([2, 3])
    assert t.shape == (2, 3) and t.size == 6 and t.tolist() == [[0, 0, 0], [0, 0, 0]]
    assert B.ones([3]).tolist() == [1, 1, 1]
    t = B.fromArray([1, 2, 3, 4], [2, 2])
    assert t.shape == (2, 2) and t.reshape(-1).tolist() == [1, 2, 3, 4]
    with pytest.raises(ValueError):
        B.fromArray([1, 2, 3], [2, 2])


def test_add():                                       # tensor.test.ts:27-32
    assert B.add(B.fromArray([1, 2, 3], [3]), B.fromArray([4, 5, 6], [3])).tolist() == [5, 7, 9]


def test_matmul_2x2():                                # tensor.test.ts:34-42
    a = B.fromArray([1, 2, 3, 4], [2, 2])
    b = B.fromArray([5, 6, 7, 8], [2, 2])
    for c in (B.matmul(a, b), B.matmul_sequential(a, b)):
        assert c.shape == (2, 2)
        assert [round(float(v)) for v in c.reshape(-1)] == [19, 22, 43, 50]


def test_softmax_sums_to_one():                       # tensor.test.ts:44-49
    s = B.softmax(B.fromArray([1, 2, 3], [1, 3]), -1)
    assert abs(float(s.sum()) - 1.0) < 5e-6


def test_gelu():                                      # tensor.test.ts:51-56
    g = B.gelu(B.fromArray([0, 1, -1], [3]))
    assert abs(g[0]) < 5e-4
    assert abs(g[1] - 0.8413) < 5e-3


def test_embedding():                                 # tensor.test.ts:58-67
    w = B.fromArray([0.1, 0.2, 0.3, 0.4, 0.5, 0.6], [3, 2])
    out = B.embedding(w, B.fromArray([0, 2], [2], np.int32))
    assert out.shape == (2, 2)
    np.testing.assert_allclose(out.reshape(-1), [0.1, 0.2, 0.5, 0.6], atol=5e-3)
    assert np.array_equal(out, w[[0, 2]])            # a gather is an exact copy


def test_layernorm():                                 # tensor.test.ts:69-79
    out = B.layerNorm(B.fromArray([1, 2, 3, 4], [2, 2]), B.ones([2]), B.zeros([2]), 1e-5)
    assert out.shape == (2, 2)
    assert abs(out[0, 0] + out[0, 1]) < 5e-4 and abs(out[1, 0] + out[1, 1]) < 5e-4


def test_cross_entropy():                             # tensor.test.ts:81-89
    loss = B.crossEntropy(B.fromArray([10, 0, 0, 0, 10, 0], [2, 3]), B.fromArray([0, 1], [2], np.int32))
    assert loss.size == 1 and float(loss) < 0.1
    assert abs(float(loss) - math.log(1 + 2 * math.exp(-10))) < 1e-7


def test_causal_mask():                               # tensor.test.ts:91-102
    d = B.causalMask(3)
    assert d.shape == (3, 3)
    assert d[0, 0] == 0 and d[1, 0] == 0 and d[1, 1] == 0
    assert d[0, 1] == -np.inf and d[0, 2] == -np.inf


def test_transpose_reshape():                         # tensor.test.ts:104-116
    a = B.fromArray([1, 2, 3, 4, 5, 6], [2, 3])
    t = B.transpose(a, 0, 1)
    assert t.shape == (3, 2) and t.reshape(-1).tolist() == [1, 4, 2, 5, 3, 6]
    r = B.reshape(a, [3, 2])
    assert r.shape == (3, 2) and r.reshape(-1).tolist() == [1, 2, 3, 4, 5, 6]


def test_sum():                                       # tensor.test.ts:118-129
    assert float(B.sum(B.fromArray([1, 2, 3], [3]))) == 6
    s = B.sum(B.fromArray([1, 2, 3, 4], [2, 2]), 0)
    assert s.shape == (2,) and s.tolist() == [4, 6]


# ── packages/tests/src/autograd.test.ts ─────────────────────────────────────
def _var(data, shape):
    return Variable(B.fromArray(data, shape), True)


def test_add_mul_backward():                          # autograd.test.ts:12-43
    tape = Tape(); ctx = Ctx(tape, B)
    a, b = _var([1, 2, 3], [3]), _var([4, 5, 6], [3])
    tape.backward(ag.sum_(ctx, ag.add(ctx, a, b)), B)
    assert a.grad.tolist() == [1, 1, 1]
    tape = Tape(); ctx = Ctx(tape, B)
    a, b = _var([2, 3], [2]), _var([4, 5], [2])
    tape.backward(ag.sum_(ctx, ag.mul(ctx, a, b)), B)
    assert a.grad.tolist() == [4, 5] and b.grad.tolist() == [2, 3]


def test_matmul_backward():                           # autograd.test.ts:45-58
    tape = Tape(); ctx = Ctx(tape, B)
    a, b = _var([1, 2, 3, 4], [2, 2]), _var([5, 6, 7, 8], [2, 2])
    tape.backward(ag.sum_(ctx, ag.matmul(ctx, a, b)), B)
    assert a.grad.tolist() == [[11, 15], [11, 15]]    # ones @ B^T
    assert b.grad.tolist() == [[4, 4], [6, 6]]        # A^T @ ones


def test_numeric_gradient_add_mul():                  # autograd.test.ts:60-102
    def fn(op, x, y):
        ctx = Ctx(Tape(), B)
        return float(ag.sum_(ctx, op(ctx, _var([x], [1]), _var([y], [1]))).data)
    eps = 1e-4
    assert abs((fn(ag.add, 3 + eps, 4) - fn(ag.add, 3 - eps, 4)) / (2 * eps) - 1.0) < 5e-3 + 2.5e-3
    assert abs((fn(ag.mul, 3 + eps, 4) - fn(ag.mul, 3 - eps, 4)) / (2 * eps) - 4.0) < 1e-2
    assert abs((fn(ag.mul, 3, 4 + eps) - fn(ag.mul, 3, 4 - eps)) / (2 * eps) - 3.0) < 1e-2


def test_broadcast_add_gradients():                   # autograd.test.ts:104-124
    tape = Tape(); ctx = Ctx(tape, B)
    a, b = _var([1, 2, 3], [3, 1]), _var([10, 20, 30, 40], [1, 4])
    loss = ag.sum_(ctx, ag.add(ctx, a, b))
    tape.backward(loss, B)
    assert abs(float(loss.data) - 324) < 5e-3
    assert a.grad.reshape(-1).tolist() == [4, 4, 4]
    assert b.grad.reshape(-1).tolist() == [3, 3, 3, 3]


def test_mean_backward():                             # autograd.test.ts:126-140
    tape = Tape(); ctx = Ctx(tape, B)
    a = _var(list(range(1, 13)), [3, 4])
    tape.backward(ag.sum_(ctx, ag.mean(ctx, a, 1, True)), B)
    np.testing.assert_allclose(a.grad, 0.25, atol=5e-6)


def test_cross_entropy_backward_shape():              # autograd.test.ts:142-155
    tape = Tape(); ctx = Ctx(tape, B)
    logits = _var([2, 1, 0.1, 0.1, 2, 0.1], [2, 3])
    tape.backward(ag.crossEntropy(ctx, logits, B.fromArray([0, 1], [2], np.int32)), B)
    assert logits.grad.shape == (2, 3)
    np.testing.assert_allclose(logits.grad.sum(-1), 0, atol=1e-7)


def test_mul_relu_add_graph():                        # autograd.test.ts:157-189 (non-checkpoint arm)
    tape = Tape(); ctx = Ctx(tape, B)
    x, w = _var([1, -2, 3, 0.5], [2, 2]), _var([0.5, -1.5, 2, 1], [2, 2])
    out = ag.add(ctx, ag.relu(ctx, ag.mul(ctx, x, w)), w)
    loss = ag.sum_(ctx, out)
    tape.backward(loss, B)
    assert abs(float(loss.data) - (0.5 + 3 + 6 + 0.5 + 2.0)) < 1e-6
    np.testing.assert_allclose(x.grad.reshape(-1), [0.5, -1.5, 2, 1], atol=1e-6)
    np.testing.assert_allclose(w.grad.reshape(-1), [2, -1, 4, 1.5], atol=1e-6)


# ── packages/tests/src/optimizer.test.ts ────────────────────────────────────
def test_adamw_gradscale_matches_prescaled():         # optimizer.test.ts:23-45
    p0 = B.fromArray([1.0, -2.0, 0.5, 3.0], [4])
    g0 = B.fromArray([0.4, -0.2, 0.8, -0.5], [4])
    pa, pb = p0.copy(), p0.copy()
    AdamW(lr=3e-4, weightDecay=0.01).step({"w": pa}, {"w": g0.copy()}, 0.125)
    AdamW(lr=3e-4, weightDecay=0.01).step({"w": pb}, {"w": B.scale(g0, 0.125)})
    assert np.max(np.abs(pa - pb)) < 1e-8


def test_adamw_c_loop_matches_python_loop():          # optimizers.ts:84-92, both restatements
    rng = np.random.default_rng(0)
    p = rng.standard_normal(64).astype(f32); g = rng.standard_normal(64).astype(f32)
    p2, m2, v2 = p.copy(), np.zeros(64, f32), np.zeros(64, f32)
    opt = AdamW(lr=1e-3, beta1=0.9, beta2=0.95, weightDecay=0.1)
    b1p = b2p = 1.0
    for _ in range(3):
        opt.step({"w": p}, {"w": g}, 0.5)
        b1p *= 0.9; b2p *= 0.95
        adamw_reference_loop(p2, g, m2, v2, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1 - b1p, 1 - b2p, 0.5)
    assert np.array_equal(p, p2) and np.array_equal(opt.m["w"], m2) and np.array_equal(opt.v["w"], v2)


# ── packages/tests/src/rng.test.ts (no literal goldens there) ───────────────
def test_rng_properties_and_c_equals_python():
    a, b = SeededRng(42), SeededRng(42)
    xs = [a.next() for _ in range(100)]
    assert xs == [b.next() for _ in range(100)]                     # determinism
    assert all(0 <= x < 1 for x in xs)                              # range
    assert xs[:5] != [SeededRng(43).next() for _ in range(5)]        # seed separation
    g = SeededRng(7)
    gs = [g.next_gauss() for _ in range(20000)]
    assert abs(sum(gs) / len(gs)) < 0.05                            # Gaussian mean
    assert abs(np.std(gs) - 1) < 0.05
    py, c = PySeededRng(1234), SeededRng(1234)
    assert [py.next() for _ in range(50)] == [c.next() for _ in range(50)]
    assert [py.next_gauss() for _ in range(51)] == [c.next_gauss() for _ in range(51)]
    a = SeededRng(5); a.next_gauss(); a.seed(5)                      # seed() drops the cached spare
    assert a.next_gauss() == SeededRng(5).next_gauss()


def test_fill_matches_scalar_draws():
    r1, r2 = SeededRng(9), SeededRng(9)
    w = r1.fill_gauss((3, 5), 0.02)
    ref = np.array([f32(r2.next_gauss() * 0.02) for _ in range(15)], dtype=f32).reshape(3, 5)
    assert np.array_equal(w, ref)


# ── blas-backed matmul against the reference's literal loop order ───────────
def test_matmul_blas_vs_sequential():
    # The LCG of apps/cli/src/commands/bench.ts:402-410 (x = x*1664525 + 1013904223,
    # value x/2^32*2-1, seeds 0x1234abcd / 0x5678ef90) supplies the inputs.
    def lcg(seed, n):
        out = np.empty(n, dtype=f32); x = seed
        for i in range(n):
            x = (x * 1664525 + 1013904223) & 0xFFFFFFFF
            out[i] = x / 4294967296 * 2 - 1
        return out
    a = lcg(0x1234ABCD, 48 * 80).reshape(48, 80)
    b = lcg(0x5678EF90, 80 * 40).reshape(80, 40)
    c1, c2 = B.matmul(a, b), B.matmul_sequential(a, b)
    assert np.max(np.abs(c1 - c2)) <= 2 ** -22       # at most a last-bit flip after f32 rounding
    assert np.mean(c1 == c2) > 0.99
