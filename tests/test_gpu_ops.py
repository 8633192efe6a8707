"""Op-level parity of the CUDA library (through the C ABI) against the oracle.

Tolerances: f32 storage -> 1e-5 relative to the tensor's scale unless stated (the oracle
accumulates in f64 and rounds once; the kernels accumulate in f32); bf16 storage -> inputs
are rounded to bf16 first, the oracle runs on those rounded values, and the result must
agree to bf16 resolution (2^-8 relative) plus fp32 accumulation noise.  Index gathers are
bit-exact.
"""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from oracle.cpu_ref import CpuRef
from oracle.gpt import flash_attention_dense, flash_attention_dense_backward

O = CpuRef()
f32 = np.float32


@pytest.fixture(scope="module")
def B():
    from alpha2_b200.backend import CudaBackend
    b = CudaBackend(0)
    yield b
    b.checkAsyncError()


def rel_err(got, ref):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return float(np.max(np.abs(got - ref)) / max(np.max(np.abs(ref)), 1e-30))


def bf16_round(x):
    from alpha2_b200.backend import bf16_to_f32, f32_to_bf16_bits
    return bf16_to_f32(f32_to_bf16_bits(np.asarray(x, f32))).reshape(np.shape(x))


def rng(seed=0):
    return np.random.default_rng(seed)


# ── known answers of packages/tests/src/tensor.test.ts, now on the GPU ─────────
def test_known_answers(B):
    assert B.smokeTest()                                                       # :34-42
    assert B.zeros([2, 3]).data.tolist() == [[0, 0, 0], [0, 0, 0]]             # :7-12
    assert B.ones([3]).data.tolist() == [1, 1, 1]
    assert B.add(B.fromArray([1, 2, 3], [3]), B.fromArray([4, 5, 6], [3])).data.tolist() == [5, 7, 9]
    g = B.gelu(B.fromArray([0, 1, -1], [3])).data                              # :51-56
    assert abs(g[0]) < 5e-4 and abs(g[1] - 0.8413) < 5e-3
    w = B.fromArray([0.1, 0.2, 0.3, 0.4, 0.5, 0.6], [3, 2])                   # :58-67
    out = B.embedding(w, B.fromArray([0, 2], [2], "i32"))
    assert out.shape == (2, 2) and np.array_equal(out.data, w.data[[0, 2]])
    ln = B.layerNorm(B.fromArray([1, 2, 3, 4], [2, 2]), B.ones([2]), B.zeros([2]), 1e-5).data   # :69-79
    assert abs(ln[0, 0] + ln[0, 1]) < 5e-4 and abs(ln[1, 0] + ln[1, 1]) < 5e-4
    loss = B.crossEntropy(B.fromArray([10, 0, 0, 0, 10, 0], [2, 3]), B.fromArray([0, 1], [2], "i32"))   # :81-89
    assert loss.data.size == 1 and loss.item() < 0.1
    m = B.causalMask(3).data                                                   # :91-102
    assert m[0, 0] == 0 and m[1, 0] == 0 and m[1, 1] == 0 and m[0, 1] == -np.inf and m[0, 2] == -np.inf
    a = B.fromArray([1, 2, 3, 4, 5, 6], [2, 3])                                # :104-116
    assert B.transpose(a, 0, 1).data.reshape(-1).tolist() == [1, 4, 2, 5, 3, 6]
    assert B.reshape(a, [3, 2]).data.reshape(-1).tolist() == [1, 2, 3, 4, 5, 6]
    assert B.sum(B.fromArray([1, 2, 3], [3])).item() == 6                      # :118-129
    assert B.sum(B.fromArray([1, 2, 3, 4], [2, 2]), 0).data.tolist() == [4, 6]
    s = B.softmax(B.fromArray([1, 2, 3], [1, 3]), -1).data                     # :44-49
    assert abs(float(s.sum()) - 1) < 5e-6


def test_device_info_and_errors(B):
    from alpha2_b200._lib import AlphaCudaError
    info = B.getDeviceInfo()
    assert info["vendorId"] == 0x10DE and info["computeCapability"][0] == 10 and info["smCount"] > 100
    with pytest.raises(AlphaCudaError, match="shape mismatch"):
        B.matmul(B.zeros([2, 3]), B.zeros([4, 5]))
    with pytest.raises(AlphaCudaError, match="does not match shape"):
        B.fromArray([1, 2, 3], [2, 2])
    with pytest.raises(AlphaCudaError, match="size mismatch"):
        B.reshape(B.zeros([2, 3]), [4, 2])


def test_elementwise_f32(B):
    r = rng(1)
    x = r.standard_normal((37, 53)).astype(f32)
    y = (np.abs(r.standard_normal((37, 53))) + 0.5).astype(f32)
    X, Y = B.upload(x), B.upload(y)
    for name in ("add", "sub", "mul", "div"):
        assert rel_err(getattr(B, name)(X, Y).data, getattr(O, name)(x, y)) < 1e-6, name
    for name in ("neg", "exp", "gelu", "relu", "silu"):
        assert rel_err(getattr(B, name)(X).data, getattr(O, name)(x)) < 2e-6, name
    assert rel_err(B.log(Y).data, O.log(y)) < 2e-6 and rel_err(B.sqrt(Y).data, O.sqrt(y)) < 1e-6
    assert rel_err(B.scale(X, 0.37).data, O.scale(x, 0.37)) < 1e-6
    assert rel_err(B.clamp(X, -0.5, 0.25).data, O.clamp(x, -0.5, 0.25)) == 0
    assert rel_err(B.softCap(X, 0.7).data, np.tanh(x.astype(np.float64) / 0.7) * 0.7) < 2e-6
    # broadcasting add [3,1] + [1,4] (packages/tests/src/autograd.test.ts:104-124)
    a, b = B.fromArray([1, 2, 3], [3, 1]), B.fromArray([10, 20, 30, 40], [1, 4])
    assert B.add(a, b).data.tolist() == [[11, 21, 31, 41], [12, 22, 32, 42], [13, 23, 33, 43]]
    assert B.broadcast(a, (3, 4)).data.tolist() == [[1] * 4, [2] * 4, [3] * 4]
    # empty tensor
    assert B.add(B.zeros([0, 4]), B.zeros([0, 4])).data.shape == (0, 4)


def test_backward_hooks_f32(B):
    r = rng(2)
    x = (r.standard_normal(1001) * 2).astype(f32)
    g = r.standard_normal(1001).astype(f32)
    X, G = B.upload(x), B.upload(g)
    x64, g64 = x.astype(np.float64), g.astype(np.float64)
    c = math.sqrt(2 / math.pi)
    t = np.tanh(c * (x64 + 0.044715 * x64 ** 3))
    gelu_grad = 0.5 * (1 + t) + 0.5 * x64 * (1 - t * t) * c * (1 + 3 * 0.044715 * x64 ** 2)
    assert rel_err(B.geluBackward(X, G).data, g64 * gelu_grad) < 3e-6
    assert rel_err(B.reluBackward(X, G).data, np.where(x > 0, g, 0)) == 0
    s = 1 / (1 + np.exp(-x64))
    assert rel_err(B.siluBackward(X, G).data, g64 * s * (1 + x64 * (1 - s))) < 3e-6
    assert rel_err(B.clampBackward(X, G, -1, 1).data, np.where((x > -1) & (x < 1), g, 0)) == 0
    assert rel_err(B.softCapBackward(G, X, 1.5).data, g64 * (1 - np.tanh(x64 / 1.5) ** 2)) < 3e-6
    y = r.standard_normal(1001).astype(f32)
    Y = B.upload(y)
    assert rel_err(B.siluMul(X, Y).data, x64 * s * y) < 3e-6
    da, db = B.siluMulBackward(X, Y, G)
    assert rel_err(da.data, g64 * y * s * (1 + x64 * (1 - s))) < 3e-6 and rel_err(db.data, g64 * x64 * s) < 3e-6
    A = B.upload(x)
    B.addInplace(A, G)
    assert rel_err(A.data, x + g) < 1e-7
    B.scaleInplace(A, 0.5)
    assert rel_err(A.data, (x + g) * f32(0.5)) < 1e-7


def test_layout_ops(B):
    r = rng(3)
    x = r.standard_normal((2, 3, 5, 4)).astype(f32)
    X = B.upload(x)
    for d0, d1 in ((1, 2), (2, 3), (0, 3), (-1, -2)):
        assert np.array_equal(B.transpose(X, d0, d1).data, np.swapaxes(x, d0, d1))
    big = r.standard_normal((3, 70, 45)).astype(f32)
    assert np.array_equal(B.transpose(B.upload(big), 1, 2).data, np.swapaxes(big, 1, 2))
    m = r.standard_normal((7, 12)).astype(f32)
    M = B.upload(m)
    q, k, v = B.sliceQkv(M)
    assert np.array_equal(q.data, m[:, :4]) and np.array_equal(k.data, m[:, 4:8]) and np.array_equal(v.data, m[:, 8:])
    assert np.array_equal(B.slice(M, [0, 4], [7, 8]).data, m[:, 4:8])
    sc = B.scatterSlice(k, [7, 12], [0, 4], [7, 8]).data
    ref = np.zeros((7, 12), f32); ref[:, 4:8] = m[:, 4:8]
    assert np.array_equal(sc, ref)
    scores = r.standard_normal((2, 2, 5, 5)).astype(f32)
    mask = B.causalMask(5)
    assert np.array_equal(B.maskedFill(B.upload(scores), mask, -1e9).data, O.maskedFill(scores, O.causalMask(5), -1e9))


def test_reductions(B):
    r = rng(4)
    x = r.standard_normal((6, 50, 7)).astype(f32)
    X = B.upload(x)
    for ax in (0, 1, 2, -1):
        assert rel_err(B.sum(X, ax).data, O.sum(x, ax)) < 2e-6
        assert rel_err(B.mean(X, ax, True).data, O.mean(x, ax, True)) < 2e-6
    assert rel_err(B.sum(X).data, O.sum(x)) < 1e-5
    rows = r.standard_normal((33, 1000)).astype(f32) * 3
    assert rel_err(B.softmax(B.upload(rows)).data, O.softmax(rows)) < 2e-6
    assert rel_err(B.logSoftmax(B.upload(rows)).data, O.logSoftmax(rows)) < 2e-6
    ts = [r.standard_normal(n).astype(f32) for n in (5, 70000, 131072, 3)]
    tot = B.totalSumOfSquares([B.upload(t) for t in ts]).item()
    assert abs(tot - sum(float(np.sum(t.astype(np.float64) ** 2)) for t in ts)) < 1e-5 * tot
    bad = ts[1].copy(); bad[17] = np.inf; bad[40000] = np.nan
    assert B.checkFinite(B.upload(bad)).item() == 2 and B.checkFinite(B.upload(ts[1])).item() == 0


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_embedding_gather_is_bit_exact_and_scatter_is_ordered(B, dtype):
    r = rng(5)
    V, E, N = 300, 96, 1000
    w = r.standard_normal((V, E)).astype(f32)
    if dtype == "bf16":
        w = bf16_round(w)
    idx = np.minimum(r.zipf(1.3, size=(4, N // 4)) - 1, V - 1).astype(np.int32)     # many repeats
    W, I = B.upload(w, dtype), B.upload(idx, "i32")
    out = B.embedding(W, I)
    assert out.shape == (4, N // 4, E) and np.array_equal(out.data, w[idx])        # bit-exact gather
    g = r.standard_normal((4, N // 4, E)).astype(f32)
    if dtype == "bf16":
        g = bf16_round(g)
    dw = B.embeddingBackward(I, B.upload(g, dtype), V).data
    # the oracle's sequential f32 scatter-add (packages/autograd/src/ops.ts:495-505)
    ref = np.zeros((V, E), f32)
    flat_idx, flat_g = idx.reshape(-1), g.reshape(-1, E)
    for i, v in enumerate(flat_idx):
        ref[v] = ref[v] + flat_g[i]
    if dtype == "bf16":
        # bf16 gradients: a row named more than 64 times is summed as a fixed tree — ten
        # contiguous segments of its occurrence list, each summed in order, added in order
        counts = np.bincount(flat_idx, minlength=V)
        assert counts.max() > 64                                                     # the case is exercised
        for v in np.nonzero(counts > 64)[0]:
            occ = np.nonzero(flat_idx == v)[0]
            seg = -(-len(occ) // 10)
            tot = np.zeros(E, f32)
            for q in range(10):
                part = np.zeros(E, f32)
                for i in occ[q * seg:(q + 1) * seg]:
                    part = part + flat_g[i]
                tot = tot + part
            ref[v] = tot
    assert np.array_equal(dw, ref)                                                   # same order => same bits
    # tok + pos in one kernel
    wpe = r.standard_normal((N // 4, E)).astype(f32)
    if dtype == "bf16":
        wpe = bf16_round(wpe)
    ep = B.embeddingPos(W, B.upload(wpe, dtype), I).data
    ref_ep = w[idx] + wpe[None]
    assert rel_err(ep, bf16_round(ref_ep) if dtype == "bf16" else ref_ep) < (1e-2 if dtype == "bf16" else 1e-7)
    # empty index list
    assert B.embeddingBackward(B.upload(np.zeros((0,), np.int32), "i32"), B.zeros([0, E], dtype), V).data.sum() == 0


@pytest.mark.parametrize("dim", [64, 384, 768, 1024, 100])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_layernorm_and_rmsnorm(B, dim, dtype):
    from oracle import autograd as oag
    from oracle.autograd import Ctx, Tape, Variable
    r = rng(dim)
    rows = 257
    x = (r.standard_normal((rows, dim)) * 2 + 0.5).astype(f32)
    g = r.standard_normal((rows, dim)).astype(f32)
    w = (1 + 0.1 * r.standard_normal(dim)).astype(f32)
    b = (0.1 * r.standard_normal(dim)).astype(f32)
    tol = 3e-6
    if dtype == "bf16":
        x, g = bf16_round(x), bf16_round(g)
        tol = 1.2e-2
    X, G, W, Bi = B.upload(x, dtype), B.upload(g, dtype), B.upload(w), B.upload(b)
    tape = Tape(); ctx = Ctx(tape, O)
    xv, wv, bv = Variable(x, True), Variable(w, True), Variable(b, True)
    y = oag.layerNorm(ctx, xv, wv, bv, 1e-5)
    y.grad = g
    tape.backward(y, O, initial_grad=g)
    assert rel_err(B.layerNorm(X, W, Bi, 1e-5).data, y.data) < tol
    res = B.layerNormBackward(X, W, G, 1e-5)
    assert rel_err(res["dx"].data, xv.grad) < tol
    assert rel_err(res["dw"].data, wv.grad) < max(tol, 2e-5) and rel_err(res["db"].data, bv.grad) < max(tol, 2e-5)
    tape = Tape(); ctx = Ctx(tape, O)
    xv, wv = Variable(x, True), Variable(w, True)
    y = oag.rmsNorm(ctx, xv, wv, 1e-5)
    tape.backward(y, O, initial_grad=g)
    assert rel_err(B.rmsNorm(X, W, 1e-5).data, y.data) < tol
    res = B.rmsNormBackward(X, W, G, 1e-5)
    assert rel_err(res["dx"].data, xv.grad) < tol and rel_err(res["dw"].data, wv.grad) < max(tol, 2e-5)


@pytest.mark.parametrize("V", [256, 4096, 50257])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_cross_entropy(B, V, dtype):
    r = rng(V)
    N = 96
    logits = (r.standard_normal((N, V)) * 2).astype(f32)
    if dtype == "bf16":
        logits = bf16_round(logits)
    tg = r.integers(0, V, N).astype(np.int32)
    Lg, Tg = B.upload(logits, dtype), B.upload(tg, "i32")
    ref_loss = float(O.crossEntropy(logits, tg))
    # the loss is an fp32 sum over logits that are exact in either storage type (the bf16 case
    # feeds the oracle the rounded logits), so one bound serves both: 2e-6 relative
    assert abs(B.crossEntropy(Lg, Tg).item() - ref_loss) < 2e-6 * ref_loss
    probs = O.softmax(logits).astype(np.float64)
    probs[np.arange(N), tg] -= 1
    ref_grad = probs * 0.5 / N
    got = B.crossEntropyBackward(Lg, Tg, B.full((), 0.5)).data
    assert rel_err(got, ref_grad) < (1e-2 if dtype == "bf16" else 3e-6)
    # fused head: GEMM + CE fwd/bwd on a padded buffer, against the unfused chain
    E = 64
    x = (r.standard_normal((N, E)) * 0.5).astype(f32)
    w = (r.standard_normal((V, E)) * 0.5).astype(f32)
    if dtype == "bf16":
        x, w = bf16_round(x), bf16_round(w)
    Xd, Wd = B.upload(x, dtype), B.upload(w, dtype)
    loss, dl, ld = B.lmHeadLoss(Xd, Wd, Tg, 1.0)
    lg = O.matmul(x, w.T.copy())
    lg_used = bf16_round(lg) if dtype == "bf16" else lg
    assert abs(loss.item() - float(O.crossEntropy(lg_used, tg))) < (3e-2 if dtype == "bf16" else 1e-5)
    assert ld % 64 == 0 and dl.shape == (N, ld)
    p = O.softmax(lg_used).astype(np.float64)
    p[np.arange(N), tg] -= 1
    assert rel_err(dl.data[:, :V], p / N) < (2e-2 if dtype == "bf16" else 1e-5)
    dx, dw = B.lmHeadBackward(dl, ld, Xd, Wd, None)
    dl_used = dl.data[:, :V].astype(np.float64)
    assert rel_err(dx.data, dl_used @ w) < (1e-2 if dtype == "bf16" else 5e-5)
    assert dw.dtype == "f32" and rel_err(dw.data, dl_used.T @ x) < (1e-2 if dtype == "bf16" else 5e-5)


def test_adamw_matches_reference_loop(B):
    """optimizers.ts:84-92 and packages/tests/src/optimizer.test.ts:23-45 (gradScale equals
    pre-scaled gradients)."""
    from oracle.train import AdamW as OAdam
    r = rng(7)
    n = 70001
    p0 = r.standard_normal(n).astype(f32); g = r.standard_normal(n).astype(f32)
    ref_p = p0.copy()
    oa = OAdam(lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weightDecay=0.1)
    from alpha2_b200.optimizers import AdamW
    P, G = B.upload(p0), B.upload(g)
    opt = AdamW(B, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weightDecay=0.1)
    for _ in range(3):
        oa.step({"w": ref_p}, {"w": g}, 0.25)
        opt.step({"w": P}, {"w": G}, 0.25)
    assert rel_err(P.data, ref_p) < 2e-6
    assert rel_err(opt._m["w"].data, oa.m["w"]) < 2e-6 and rel_err(opt._v["w"].data, oa.v["w"]) < 2e-6
    # gradScale == pre-scaled gradients
    Pa, Pb = B.upload(p0), B.upload(p0)
    AdamW(B, lr=3e-4, weightDecay=0.01).step({"w": Pa}, {"w": G}, 0.125)
    AdamW(B, lr=3e-4, weightDecay=0.01).step({"w": Pb}, {"w": B.scale(G, 0.125)})
    assert np.max(np.abs(Pa.data - Pb.data)) < 1e-7
    # multi-tensor launch with device-side clipping == host-side clipping; bf16 shadow follows
    class V:  # minimal Variable-like
        def __init__(s, d, g): s.data, s.grad, s.shadow = d, g, None
    va, vb = V(B.upload(p0), B.upload(g)), V(B.upload(p0), B.upload(g))
    va.shadow = B.zeros((n,), "bf16")
    sumsq = B.totalSumOfSquares([va.grad])
    gn = math.sqrt(sumsq.item()) * 0.5
    AdamW(B, lr=1e-3).stepParamEntries([("w", va)], 0.5, fused=True, clipSumSq=sumsq, maxNorm=1.0)
    AdamW(B, lr=1e-3).stepParamEntries([("w", vb)], 0.5 * (1.0 / gn))
    assert rel_err(va.data.data, vb.data.data) < 1e-6
    assert np.array_equal(va.shadow.data, bf16_round(va.data.data))


@pytest.mark.parametrize("bad", [np.inf, np.nan])
def test_fused_adamw_skips_a_step_with_non_finite_gradients(B, bad):
    """trainer.ts:1495-1527,1750: a step whose gradient norm is not finite does not call the
    optimizer.  The fused update learns the norm on the device, so the kernel itself must leave
    p, m, v and the bf16 shadow bit for bit as they were — for every element, not only those
    whose own gradient is finite — and the host's step count must be taken back."""
    from alpha2_b200.optimizers import AdamW
    r = rng(11)
    n = 200003
    p0, g0 = r.standard_normal(n).astype(f32), r.standard_normal(n).astype(f32)

    class V:
        def __init__(s, d, g, sh): s.data, s.grad, s.shadow = d, g, sh
    va = V(B.upload(p0), B.upload(g0), B.castDtype(B.upload(p0), "bf16"))
    opt = AdamW(B, lr=1e-3, weightDecay=0.1)
    sumsq = B.totalSumOfSquares([va.grad])
    opt.stepParamEntries([("w", va)], 0.5, fused=True, clipSumSq=sumsq, maxNorm=1.0)      # a normal step first
    before = [np.array(t.data).copy() for t in (va.data, opt._m["w"], opt._v["w"], va.shadow)]
    assert not np.array_equal(before[0], p0)
    g1 = g0.copy(); g1[12345] = bad
    va.grad = B.upload(g1)
    sumsq = B.totalSumOfSquares([va.grad])
    assert not math.isfinite(sumsq.item())
    state = (opt._step, opt._beta1Pow, opt._beta2Pow)
    opt.stepParamEntries([("w", va)], 0.5, fused=True, clipSumSq=sumsq, maxNorm=1.0)
    for t, old in zip((va.data, opt._m["w"], opt._v["w"], va.shadow), before):
        t.invalidate_host()
        assert np.array_equal(np.array(t.data), old)
    opt.undoStep()
    assert (opt._step, opt._beta1Pow, opt._beta2Pow) == state


# ── GEMM ────────────────────────────────────────────────────────────────────
def lcg(seed, n):
    """Inputs of the reference's own GEMM check (apps/cli/src/commands/bench.ts:402-410)."""
    out = np.empty(n, dtype=np.float64)
    x = seed
    for i in range(n):
        x = (x * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = x / 4294967296 * 2 - 1
    return out.astype(f32)


def gemm_ref(layout, a, b):
    A, Bm = a.astype(np.float64), b.astype(np.float64)
    if layout == "nt":
        return A @ Bm.T
    return A @ Bm if layout == "nn" else A.T @ Bm


def run_gemm(B, layout, A, Bm):
    return {"nt": B.matmulTransposed, "nn": B.matmul, "tn": B.matmulTransposedA}[layout](A, Bm)


def shapes_for(layout, M, N, K):
    return {"nt": ((M, K), (N, K)), "nn": ((M, K), (K, N)), "tn": ((K, M), (K, N))}[layout]


@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
def test_gemm_f32_reference_fixture(B, layout):
    """The reference's LCG-seeded check, atol 2e-2 + rtol 1e-2 (bench.ts:412-519,669-670),
    and the tighter fp32 bound this kernel is built for."""
    M, N, K = 97, 75, 130
    sa, sb = shapes_for(layout, M, N, K)
    a = lcg(0x1234ABCD, sa[0] * sa[1]).reshape(sa)
    b = lcg(0x5678EF90, sb[0] * sb[1]).reshape(sb)
    got = run_gemm(B, layout, B.upload(a), B.upload(b)).data
    ref = gemm_ref(layout, a, b)
    assert np.all(np.abs(got - ref) <= 2e-2 + 1e-2 * np.abs(ref))
    assert rel_err(got, ref) < 2e-6


def test_gemm_f32_batched_and_epilogues(B):
    r = rng(8)
    q = r.standard_normal((2, 3, 17, 8)).astype(f32)
    k = r.standard_normal((2, 3, 8, 17)).astype(f32)
    assert rel_err(B.matmul(B.upload(q), B.upload(k)).data, q.astype(np.float64) @ k) < 2e-6
    x = r.standard_normal((2, 9, 24)).astype(f32)
    w = r.standard_normal((40, 24)).astype(f32)
    assert rel_err(B.matmulTransposed(B.upload(x), B.upload(w)).data, x.astype(np.float64) @ w.T) < 2e-6
    pre, act = B.matmulTransposedGelu(B.upload(x), B.upload(w))
    assert rel_err(pre.data, x.astype(np.float64) @ w.T) < 2e-6 and rel_err(act.data, O.gelu(pre.data)) < 2e-6
    res = r.standard_normal((2, 9, 40)).astype(f32)
    assert rel_err(B.matmulTransposedAdd(B.upload(x), B.upload(w), B.upload(res)).data,
                   res + x.astype(np.float64) @ w.T) < 2e-6


TC_SHAPES = [
    (128, 256, 64), (128, 128, 128), (256, 512, 256),       # exact tiles
    (200, 300, 72), (1, 8, 8), (130, 264, 200),             # ragged M / N / K
    (384, 2304, 768), (512, 768, 3072),                     # train-step K sizes
    (768, 768, 4096), (96, 3072, 2048),                     # few tiles, long K: split-K
    (4096, 2304, 192), (4104, 1032, 136),                   # more tiles than tile walkers (both accumulators cycle)
]


@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
@pytest.mark.parametrize("shape", TC_SHAPES)
def test_gemm_bf16_tensor_core(B, layout, shape):
    """bf16 operands, fp32 accumulate in tensor memory.  Inputs ~ N(0, 0.02) like the
    train-step GEMMs; the result must match the f64 product of the *rounded* inputs to
    accumulation noise, far inside the reference's own GEMM tolerance
    (packages/tests/src/gpu-perf.test.ts:169: max diff < 0.5 on its f16 path)."""
    M, N, K = shape
    if layout == "tn" and (M % 8 or N % 8):
        pytest.skip("TN reads A as [K, M]: M and N must keep rows 16-byte aligned")
    if layout == "nn" and N % 8:
        pytest.skip("NN reads B as [K, N]: N must keep rows 16-byte aligned")
    r = rng(M * 7 + N * 3 + K)
    sa, sb = shapes_for(layout, M, N, K)
    a = bf16_round(r.standard_normal(sa) * 0.02)
    b = bf16_round(r.standard_normal(sb) * 0.02)
    out = run_gemm(B, layout, B.upload(a, "bf16"), B.upload(b, "bf16"))
    ref = gemm_ref(layout, a, b)
    got = out.data
    assert got.shape == ref.shape
    scale = float(np.sqrt(K)) * 0.02 * 0.02
    tol = scale * (2 ** -7 if out.dtype == "bf16" else 1e-5) * 4 + 1e-12
    err = np.abs(got - ref)
    assert float(err.max()) < tol * 4, (float(err.max()), tol, np.unravel_index(err.argmax(), err.shape))
    B.checkAsyncError()


def test_gemm_bf16_epilogues_and_accumulate(B):
    r = rng(11)
    M, N, K = 300, 520, 192
    x = bf16_round(r.standard_normal((M, K)) * 0.5)
    w = bf16_round(r.standard_normal((N, K)) * 0.1)
    res = bf16_round(r.standard_normal((M, N)))
    X, W, R = B.upload(x, "bf16"), B.upload(w, "bf16"), B.upload(res, "bf16")
    ref = x.astype(np.float64) @ w.T.astype(np.float64)
    pre, act = B.matmulTransposedGelu(X, W)
    assert rel_err(pre.data, ref) < 1e-2
    assert rel_err(act.data, O.gelu(ref.astype(f32))) < 1e-2
    assert rel_err(B.matmulTransposedAdd(X, W, R).data, res + ref) < 1e-2
    g = bf16_round(r.standard_normal((M, N)) * 0.1)
    prek = bf16_round(r.standard_normal((M, K)))
    got = B.matmulGeluBackward(B.upload(g, "bf16"), W, B.upload(prek, "bf16")).data
    c = math.sqrt(2 / math.pi)
    p64 = prek.astype(np.float64)
    t = np.tanh(c * (p64 + 0.044715 * p64 ** 3))
    gg = 0.5 * (1 + t) + 0.5 * p64 * (1 - t * t) * c * (1 + 3 * 0.044715 * p64 ** 2)
    assert rel_err(got, (g.astype(np.float64) @ w) * gg) < 1.5e-2
    # dW in f32, accumulated over two calls (gradient accumulation)
    from alpha2_b200 import _lib as L
    from alpha2_b200._lib import check
    dw = B.zeros((N, K), "f32")
    G = B.upload(g, "bf16")
    for _ in range(2):
        check(B.lib.alpha_gemm(L.GEMM_TN, G.ptr, X.ptr, dw.ptr, N, K, M, N, K, K, L.BF16, L.F32, L.EPI_NONE, 0, 0, 1))
    dw.invalidate_host()
    assert rel_err(dw.data, 2 * (g.astype(np.float64).T @ x)) < 1e-5
    B.checkAsyncError()


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("shape", [(300, 520, 192), (2048, 512, 768)])
def test_gradients_added_inside_the_gemm(B, dtype, shape):
    """matmulInto (into += G @ W, output aliasing the addend) and matmulTransposedA(into=)."""
    M, N, K = shape
    r = rng(12)
    g, w, x, acc = (r.standard_normal(s).astype(f32) * c for s, c in
                    (((M, N), 0.1), ((N, K), 0.1), ((M, K), 0.5), ((M, K), 1.0)))
    if dtype == "bf16":
        g, w, x, acc = (bf16_round(t) for t in (g, w, x, acc))
    G, W, X, ACC = (B.upload(t, dtype) for t in (g, w, x, acc))
    out = B.matmulInto(G, W, ACC)
    assert out is ACC
    assert rel_err(ACC.data, acc + g.astype(np.float64) @ w) < (1e-5 if dtype == "f32" else 1e-2)
    dw0 = r.standard_normal((N, K)).astype(f32)
    DW = B.upload(dw0, "f32")
    assert B.matmulTransposedA(G, X, into=DW) is DW
    assert rel_err(DW.data, dw0 + g.astype(np.float64).T @ x) < 1e-5
    B.checkAsyncError()


PAIRS = [
    # ((M0, N0), (M1, N1), K): the train step's MLP weight gradients (36 + 36 tiles share the device, unsplit)
    ((3072, 768), (768, 3072), 16384),
    ((2304, 768), (768, 768), 8192),          # 27 + 9 tiles
    ((1000, 520), (312, 264), 4100),          # ragged M, N and K in both (rows stay 16-byte multiples, as TMA needs)
    ((128, 768), (768, 768), 8192),           # M <= 128 in one of them: runs as two GEMMs inside the library
    ((4096, 4096), (768, 768), 2048),         # too many tiles to share one wave: two GEMMs as well
]


@pytest.mark.parametrize("shape0,shape1,K", PAIRS)
@pytest.mark.parametrize("accumulate", [(False, False), (True, False), (True, True)])
def test_two_weight_gradients_in_one_launch(B, shape0, shape1, K, accumulate):
    """alpha_gemm_tn_pair: both products against f64, C += where asked, three launches bit for bit."""
    r = rng(K + shape0[0] + 7 * shape1[1])
    ops, refs, c0s = [], [], []
    for (M, N), accu in zip((shape0, shape1), accumulate):
        a = bf16_round(r.standard_normal((K, M)) * 0.05)
        b = bf16_round(r.standard_normal((K, N)) * 0.05)
        c0 = r.standard_normal((M, N)).astype(f32) if accu else None
        ops.append((B.upload(a, "bf16"), B.upload(b, "bf16")))
        c0s.append(c0)
        refs.append(a.astype(np.float64).T @ b.astype(np.float64) + (0 if c0 is None else c0))
    scale = float(np.sqrt(K)) * 0.05 * 0.05
    outs = []
    for rep in range(3):
        intos = [None if c0 is None else B.upload(c0, "f32") for c0 in c0s]
        got = B.matmulTransposedAPair((ops[0][0], ops[0][1], intos[0]), (ops[1][0], ops[1][1], intos[1]))
        outs.append([np.array(t.data) for t in got])
        for t, into in zip(got, intos):
            assert into is None or t is into
    for o, ref in zip(outs[0], refs):
        assert o.dtype == f32 and float(np.abs(o - ref).max()) < scale * 1e-5 * 16 + 2e-6
    for o in outs[1:]:
        assert all(np.array_equal(x, y) for x, y in zip(o, outs[0]))
    B.checkAsyncError()


K_BALANCED = [
    # (layout, M, N, K, out): few output tiles, long K -> K is split
    ("tn", 2304, 768, 16384, "f32"), ("tn", 768, 768, 16384, "f32"), ("tn", 768, 3072, 8192, "f32"),
    ("tn", 1000, 520, 8200, "f32"),            # ragged M, N (rows and columns beyond the matrix in the last tiles), ragged K
    ("nt", 512, 512, 16384, "bf16"),           # bf16 output through the scalar reduce path
    ("nn", 300, 264, 12288, "f32"),
    ("tn", 128, 768, 16384, "f32"),            # M <= 128: single-CTA kernel, 128 x 256 tiles
    ("tn", 768, 128, 16384, "f32"),            # N <= 128: 128 x 128 tiles
]


@pytest.mark.parametrize("layout,M,N,K,out", K_BALANCED)
@pytest.mark.parametrize("accumulate", [0, 1])
def test_gemm_split_over_k_adds_partials_in_a_fixed_order(B, layout, M, N, K, out, accumulate):
    """The weight-gradient GEMMs split K across the device: partial products meet in an fp32
    workspace and are added in split order.  Result against the f64 product; five launches must
    agree bit for bit; accumulate adds to what C held; a different split shape in between must
    not disturb anything."""
    from alpha2_b200 import _lib as L
    from alpha2_b200._lib import check
    r = rng(M + 3 * N + K)
    sa, sb = shapes_for(layout, M, N, K)
    a = bf16_round(r.standard_normal(sa) * 0.05)
    b = bf16_round(r.standard_normal(sb) * 0.05)
    c0 = bf16_round(r.standard_normal((M, N))) if accumulate else np.zeros((M, N), f32)
    A, Bm = B.upload(a, "bf16"), B.upload(b, "bf16")
    code = {"nt": L.GEMM_NT, "nn": L.GEMM_NN, "tn": L.GEMM_TN}[layout]
    ref = c0.astype(np.float64) + gemm_ref(layout, a, b)
    outs = []
    other = B.upload(bf16_round(r.standard_normal((4096, 256)) * 0.05), "bf16")
    for rep in range(5):
        Cm = B.upload(c0, out)
        check(B.lib.alpha_gemm(code, A.ptr, Bm.ptr, Cm.ptr, M, N, K, sa[1], sb[1], N, L.BF16, L.DTYPE_CODE[out],
                               L.EPI_NONE, 0, 0, accumulate))
        Cm.invalidate_host()
        outs.append(np.array(Cm.data))
        if rep == 1:
            B.matmulTransposedA(other, other)                # [256, 256] from K = 4096: one shared tile
    scale = float(np.sqrt(K)) * 0.05 * 0.05
    tol = (scale * 1e-5 * 16 + 1e-12) if out == "f32" else (2 ** -7 * (float(np.abs(ref).max()) + scale))
    assert float(np.abs(outs[0] - ref).max()) < tol
    for o in outs[1:]:
        assert np.array_equal(o, outs[0])
    B.checkAsyncError()


# ── attention ───────────────────────────────────────────────────────────────
@pytest.mark.parametrize("cfg", [(3, 64, 16, 30.0), (2, 100, 64, 30.0), (2, 256, 64, 0.0), (1, 130, 32, 2.0),
                                 (1, 192, 128, 30.0),
                                 (2, 640, 64, 30.0),    # 5 key/query blocks: the 4-stage rings wrap
                                 (1, 300, 64, 2.0),     # tight cap: tanh arguments beyond the polynomial range
                                 (1, 1024, 64, 0.0),
                                 (1, 2048, 64, 30.0),   # the 350M configuration's context: 16 blocks per item
                                 (1, 1990, 64, 0.0)])   # ragged, long, running-maximum path
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_flash_attention_contract(B, cfg, dtype):
    """Backend.flashAttention / flashAttentionBackward on [B*H, T, D] (interfaces.ts:127-135)."""
    BH, T, D, cap = cfg
    r = rng(T + D)
    q, k, v, do = (r.standard_normal((BH, T, D)).astype(f32) for _ in range(4))
    tol = 3e-5
    if dtype == "bf16":
        q, k, v, do = (bf16_round(t) for t in (q, k, v, do))
        tol = 2e-2
    scale = 1 / math.sqrt(D)
    o_ref, lse_ref = flash_attention_dense(q, k, v, T, scale, cap)
    Q, K, V, dO = (B.upload(t, dtype) for t in (q, k, v, do))
    res = B.flashAttention(Q, K, V, T, scale, cap)
    assert rel_err(res["output"].data, o_ref) < tol
    assert rel_err(res["lse"].data, lse_ref) < (1e-5 if dtype == "f32" else 1e-3)
    o_used = res["output"].data
    dq, dk, dv = flash_attention_dense_backward(q, k, v, o_used, do, res["lse"].data, T, scale, cap)
    g = B.flashAttentionBackward(Q, K, V, res["output"], dO, res["lse"], T, scale, cap)
    for name, ref in (("dQ", dq), ("dK", dk), ("dV", dv)):
        assert rel_err(g[name].data, ref) < tol * 2, name


@pytest.mark.parametrize("geom", [(2, 96, 4, 16), (2, 200, 3, 64), (1, 512, 2, 64)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_attention_on_fused_qkv(B, dtype, geom):
    """q/k/v read in place from [B*T, 3E]; output head-merged; gradients land in [B*T, 3E].
    Head dim 64 in bf16 is the tensor-core path (ragged T = 200 included)."""
    Bn, T, H, D = geom
    E = H * D
    r = rng(21)
    qkv = r.standard_normal((Bn * T, 3 * E)).astype(f32)
    dout = r.standard_normal((Bn * T, E)).astype(f32)
    tol = 3e-5
    if dtype == "bf16":
        qkv, dout = bf16_round(qkv), bf16_round(dout)
        tol = 2e-2
    split = lambda m: m.reshape(Bn, T, H, D).transpose(0, 2, 1, 3).reshape(Bn * H, T, D)
    merge = lambda m: m.reshape(Bn, H, T, D).transpose(0, 2, 1, 3).reshape(Bn * T, E)
    q, k, v = (split(qkv[:, i * E:(i + 1) * E]) for i in range(3))
    scale = 1 / math.sqrt(D)
    o_ref, lse_ref = flash_attention_dense(q, k, v, T, scale, 30.0)
    QKV = B.upload(qkv, dtype)
    out, lse = B.attentionQkv(QKV, Bn, T, H, scale, 30.0)
    assert rel_err(out.data, merge(o_ref)) < tol
    dq, dk, dv = flash_attention_dense_backward(q, k, v, split(out.data), split(dout), lse.data, T, scale, 30.0)
    dqkv = B.attentionQkvBackward(QKV, out, B.upload(dout, dtype), lse, Bn, T, H, scale, 30.0).data
    ref = np.concatenate([merge(dq), merge(dk), merge(dv)], axis=1)
    assert rel_err(dqkv, ref) < tol * 2


@pytest.mark.parametrize("geom", [(2, 128, 2, 192), (3, 200, 12, 768), (16, 1024, 12, 768)])
def test_rowdot_gemm_feeds_attention_backward(B, geom):
    """dO = G @ Wo with the row-dots dO.O taken in the GEMM's epilogue (one per row and head of 64
    columns), and attention's backward fed with them: dO equals the plain GEMM bit for bit, the
    row-dots equal the f64 products of the rounded values, and the gradients equal those of the
    backward that computes the row-dots itself."""
    Bn, T, H, K = geom
    E, N = 64 * H, Bn * T
    r = rng(Bn * 7 + T)
    g = bf16_round(r.standard_normal((N, K)) * 0.1)
    w = bf16_round(r.standard_normal((K, E)) * 0.1)
    qkv = bf16_round(r.standard_normal((N, 3 * E)))
    G, W, QKV = B.upload(g, "bf16"), B.upload(w, "bf16"), B.upload(qkv, "bf16")
    scale = 1 / math.sqrt(64)
    out, lse = B.attentionQkv(QKV, Bn, T, H, scale, 30.0)
    dO, delta = B.matmulRowdot(G, W, out, T, H)
    plain = B.matmul(G, W)
    assert np.array_equal(dO.data, plain.data)
    want = (plain.data.astype(np.float64) * out.data.astype(np.float64)).reshape(Bn, T, H, 64).sum(-1).transpose(0, 2, 1)
    assert delta.shape == (Bn, H, T)
    assert float(np.max(np.abs(delta.data - want))) < 1e-5 * max(1.0, float(np.max(np.abs(want))))
    a = B.attentionQkvBackward(QKV, out, dO, lse, Bn, T, H, scale, 30.0, delta=delta).data
    b = B.attentionQkvBackward(QKV, out, dO, lse, Bn, T, H, scale, 30.0).data
    assert float(np.max(np.abs(a - b))) <= 2 ** -7 * float(np.max(np.abs(b)))
    B.checkAsyncError()


def test_rope_matches_oracle_and_inverts(B):
    from oracle import autograd as oag
    from oracle.autograd import Ctx, Tape, Variable
    Bn, T, H, D = 2, 33, 3, 16
    E = H * D
    r = rng(31)
    x = r.standard_normal((Bn, T, E)).astype(f32)
    ref = oag.rope(Ctx(Tape(), O), Variable(x, True), H).data
    buf = np.zeros((Bn * T, 3 * E), f32)
    buf[:, E:2 * E] = x.reshape(Bn * T, E)
    X = B.upload(buf)
    B.rope(X, Bn, T, H, D, 3 * E, E)
    got = X.data
    assert rel_err(got[:, E:2 * E], ref.reshape(Bn * T, E)) < 3e-6
    assert np.all(got[:, :E] == 0) and np.all(got[:, 2 * E:] == 0)
    B.rope(X, Bn, T, H, D, 3 * E, E, inverse=True)
    assert rel_err(X.data[:, E:2 * E], x.reshape(Bn * T, E)) < 3e-6


@pytest.mark.parametrize("geom", [(2, 33, 3, 16), (1, 2048, 2, 64), (2, 40, 2, 6)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_rope_qkv_matches_oracle_and_inverts(B, geom, dtype):
    """q and k blocks of a fused [B*T, 3E] activation rotated, v passed through, out of place;
    head dim 6 takes the scalar kernel (pairs are not a multiple of 16 bytes)."""
    from oracle import autograd as oag
    from oracle.autograd import Ctx, Tape, Variable
    Bn, T, H, D = geom
    E = H * D
    qkv = rng(32).standard_normal((Bn * T, 3 * E)).astype(f32)
    if dtype == "bf16":
        qkv = bf16_round(qkv)
    ref = qkv.copy()
    for blk in range(2):
        xb = np.ascontiguousarray(qkv[:, blk * E:(blk + 1) * E]).reshape(Bn, T, E)
        ref[:, blk * E:(blk + 1) * E] = oag.rope(Ctx(Tape(), O), Variable(xb, True), H).data.reshape(Bn * T, E)
    X = B.upload(qkv, dtype)
    Y = B.ropeQkv(X, Bn, T, H)
    tol = 3e-6 if dtype == "f32" else 6e-3
    assert rel_err(Y.data, ref) < tol
    assert np.array_equal(Y.data[:, 2 * E:], qkv[:, 2 * E:]) and np.array_equal(X.data, qkv)
    back = B.ropeQkv(Y, Bn, T, H, inverse=True)
    assert rel_err(back.data, qkv) < 2 * tol


def test_allocator_reuses_blocks(B):
    B.syncGpu()
    for _ in range(3):
        t = B.zeros([1000, 100]); del t
    s0 = B.gpuMemStats()
    for _ in range(50):
        t = B.zeros([1000, 100]); del t
    s1 = B.gpuMemStats()
    assert s1["deviceMallocs"] == s0["deviceMallocs"] and s1["allocs"] >= s0["allocs"] + 50
    assert s1["bytesInUse"] == s0["bytesInUse"]


def test_async_scalar_read(B):
    """alpha_d2h_async + event: the value is that of the tensor when the read was enqueued."""
    t = B.full((), 3.5)
    h = B.readScalarAsync(t)
    B.scaleInplace(t, 2.0)                  # enqueued after the read
    assert h.get() == 3.5 and h.get() == 3.5
    assert t.item() == 7.0
