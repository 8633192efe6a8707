"""Data loader (packages/train/src/data.ts), evaluation (eval.ts) and sampling (sample.ts)."""
import math

import numpy as np
import pytest

from alpha2_b200.data import DataLoader
from alpha2_b200.eval import evaluate, next_token, sample_tokens
from oracle.cpu_ref import SeededRng as OracleRng
from oracle.data import OracleLoader


def _tokens(n, vocab=50, seed=1):
    return np.random.default_rng(seed).integers(0, vocab, n).astype(np.int32)


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("n,B,T", [(1000, 4, 16), (97, 3, 16), (40, 2, 33)])
def test_loader_equals_restatement(packed, n, B, T):
    tok = _tokens(n)
    a = DataLoader(tok, OracleRng(11), B, T, packed)
    b = OracleLoader(tok, OracleRng(11), B, T, packed)
    for _ in range(12):                                   # long enough for the packed cursors to wrap
        ia, ta = a.nextBatch()
        ib, tb = b.nextBatch()
        assert np.array_equal(ia, ib) and np.array_equal(ta, tb)
    assert a.stepsPerEpoch == n // (B * T)


def test_packed_wraps_like_the_reference_by_hand():
    ld = DataLoader(np.arange(10, dtype=np.int32), None, 2, 4, packed=True)
    i1, t1 = (x.copy() for x in ld.nextBatch())
    assert i1.tolist() == [[0, 1, 2, 3], [5, 6, 7, 8]] and t1.tolist() == [[1, 2, 3, 4], [6, 7, 8, 9]]
    i2, t2 = ld.nextBatch()
    assert i2.tolist() == [[4, 5, 6, 7], [9, 0, 1, 2]]
    assert t2.tolist() == [[5, 6, 7, 8], [0, 1, 2, 3]]    # the corpus' last token is followed by its first


def test_random_mode_needs_more_tokens_than_the_block():
    with pytest.raises(ValueError):
        DataLoader(np.arange(8, dtype=np.int32), OracleRng(1), 2, 8).nextBatch()


@pytest.mark.parametrize("packed", [False, True])
def test_ranks_partition_the_global_batch(packed):
    tok, B, T, world = _tokens(777), 3, 8, 2
    whole = DataLoader(tok, OracleRng(5), B * world, T, packed)
    parts = [DataLoader(tok, OracleRng(5), B, T, packed, rank=r, world=world) for r in range(world)]
    for _ in range(6):
        iw, tw = whole.nextBatch()
        got_i = np.concatenate([p.nextBatch()[0] for p in parts])
        # nextBatch returns the ring buffer: take targets from a second loader pass
        assert np.array_equal(got_i, iw)
    whole = DataLoader(tok, OracleRng(5), B * world, T, packed)
    parts = [DataLoader(tok, OracleRng(5), B, T, packed, rank=r, world=world) for r in range(world)]
    for _ in range(6):
        tw = whole.nextBatch()[1]
        assert np.array_equal(np.concatenate([p.nextBatch()[1] for p in parts]), tw)


def test_two_buffers_alternate():
    ld = DataLoader(_tokens(200), OracleRng(2), 2, 8)
    a = ld.nextBatch()[0]
    keep = a.copy()
    b = ld.nextBatch()[0]
    assert a is not b and np.array_equal(a, keep)          # still intact after one more call
    c = ld.nextBatch()[0]
    assert c is a                                           # reused on the call after next


class SeqRng:
    def __init__(self, vals):
        self.vals, self.i = list(vals), 0

    def next(self):
        v = self.vals[self.i]
        self.i += 1
        return v


def test_next_token_rules():
    logits = np.log(np.array([0.1, 0.2, 0.7], np.float32))
    assert next_token(logits, SeqRng([]), 0.0, 0, None) == 2                     # greedy
    assert next_token(np.array([1, 3, 3], np.float32), SeqRng([]), 0, 0, None) == 1   # first maximum
    assert next_token(logits, SeqRng([0.05]), 1.0, 0, None) == 0                  # cumulative 0.1 / 0.3 / 1.0
    assert next_token(logits, SeqRng([0.25]), 1.0, 0, None) == 1
    assert next_token(logits, SeqRng([0.95]), 1.0, 0, None) == 2
    assert next_token(logits, SeqRng([0.0]), 1.0, 1, None) == 2                   # top-1 keeps only the maximum
    assert next_token(logits, SeqRng([0.99]), 1.0, 2, None) == 2                  # top-2 = {1, 2}: 0.2/0.9, 0.7/0.9
    assert next_token(logits, SeqRng([0.1]), 1.0, 2, None) == 1
    assert next_token(logits, SeqRng([0.999]), 1.0, 0, 0.5) == 2                  # nucleus 0.5 = {2}
    assert next_token(logits, SeqRng([0.9]), 1.0, 0, 0.8) == 1                    # nucleus 0.8 = {2, 1}; r*0.9 = 0.81 > 0.7
    # temperature sharpens: at T = 0.25 token 2 holds 0.7^4 / (0.1^4 + 0.2^4 + 0.7^4) = 0.993 of the mass
    assert next_token(logits, SeqRng([0.5]), 0.25, 0, None) == 2


def _host_model(attention="fused"):
    from alpha2_b200.gpt import ModelConfig, initGPT
    from alpha2_b200.rng import SeededRng
    from tests.fake_backend import NumpyBackend
    mc = ModelConfig(vocabSize=32, blockSize=12, nLayer=2, nEmbd=16, nHead=2, tied=True, init="plain")
    B = NumpyBackend()
    return mc, B, initGPT(mc, B, SeededRng(9))


def test_evaluate_is_the_mean_batch_loss_on_the_host_backend():
    from alpha2_b200.autograd import Tape
    from alpha2_b200.gpt import gptForward
    from tests.fake_backend import T
    mc, B, P = _host_model()
    tok = _tokens(300, 32)
    res = evaluate(mc, P, B, DataLoader(tok, OracleRng(4), 2, 12), nBatches=3)
    ld = DataLoader(tok, OracleRng(4), 2, 12)
    losses = []
    for _ in range(3):
        i, t = ld.nextBatch()
        losses.append(float(np.asarray(gptForward(mc, P, B, Tape(), T(i.copy(), "i32"), T(t.copy(), "i32"))["loss"].data.data).reshape(-1)[0]))
    assert abs(res["loss"] - sum(losses) / 3) < 1e-6 and res["nBatches"] == 3
    assert abs(res["perplexity"] - math.exp(res["loss"])) < 1e-9


def test_sampling_loop_on_the_host_backend():
    mc, B, P = _host_model()
    out = sample_tokens(mc, P, B, OracleRng(1), [3, 4, 5], steps=20, temperature=0.0)
    assert out.size == mc.blockSize and out[:3].tolist() == [3, 4, 5]            # stops at a full context
    again = sample_tokens(mc, P, B, OracleRng(1), [3, 4, 5], steps=20, temperature=0.0)
    assert np.array_equal(out, again)
    a = sample_tokens(mc, P, B, OracleRng(7), [1], steps=5, temperature=0.9, topk=8, topp=0.9)
    b = sample_tokens(mc, P, B, OracleRng(7), [1], steps=5, temperature=0.9, topk=8, topp=0.9)
    assert a.size == 6 and np.array_equal(a, b) and a.max() < mc.vocabSize


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [("f32", 2e-5), ("bf16", 2e-2)])
def test_evaluate_and_last_row_logits_on_the_device(dtype, tol):
    """Device evaluation against the oracle's forward on the same batches; the last-row
    projection against the full projection."""
    from alpha2_b200.autograd import Tape
    from alpha2_b200.backend import CudaBackend
    from alpha2_b200.gpt import ModelConfig, gptForward, initGPT
    from alpha2_b200.rng import SeededRng
    from oracle import gpt as ogpt
    from oracle.autograd import Tape as OTape
    from oracle.cpu_ref import CpuRef
    B = CudaBackend(0)
    kw = dict(vocabSize=96, blockSize=32, nLayer=2, nEmbd=64, nHead=1, tied=True, init="plain")
    mc = ModelConfig(**kw, compute_dtype=dtype)
    P = initGPT(mc, B, SeededRng(5))
    tok = _tokens(500, 96)
    res = evaluate(mc, P, B, DataLoader(tok, OracleRng(3), 2, 32, backend=B), nBatches=2)
    ocfg = ogpt.ModelConfig(**kw)
    OP = ogpt.init_gpt(ocfg, OracleRng(5))
    ld = OracleLoader(tok, OracleRng(3), 2, 32)
    want = 0.0
    for _ in range(2):
        i, t = ld.nextBatch()
        want += float(ogpt.gpt_forward(ocfg, OP, CpuRef(), OTape(), i, t)[1].data) / 2
    assert abs(res["loss"] - want) / want < tol
    ctx = tok[:20].reshape(1, -1)
    full = gptForward(mc, P, B, Tape(), B.upload(ctx, "i32"), None)["logits"].data.data
    last = gptForward(mc, P, B, Tape(), B.upload(ctx, "i32"), None, lastOnly=True)["logits"].data.data
    assert last.shape == (1, 1, 96)
    assert np.allclose(np.asarray(last, np.float32).reshape(-1), np.asarray(full, np.float32)[0, -1], rtol=1e-2 if dtype == "bf16" else 1e-5, atol=1e-2 if dtype == "bf16" else 1e-5)
    out = sample_tokens(mc, P, B, OracleRng(2), ctx[0, :5], steps=6, temperature=0.0)
    assert out.size == 11
    B.checkAsyncError()


@pytest.mark.gpu
@pytest.mark.parametrize("packed", [False, True])
def test_pinned_loader_feeds_the_device_while_earlier_work_is_still_queued(packed):
    """Seven batches are requested back to back from a two-slot page-locked ring while tens of
    milliseconds of kernels are still queued in front of the copies; every device batch must
    equal the host loader's, and the tensors must not alias the ring."""
    import time
    from alpha2_b200.backend import CudaBackend
    B = CudaBackend(0)
    tok = _tokens(300000, 50257, seed=3)
    ld = DataLoader(tok, OracleRng(21), 16, 1024, packed, backend=B, pin=True)
    ref = DataLoader(tok, OracleRng(21), 16, 1024, packed)
    x = B.upload(np.random.default_rng(0).standard_normal((2048, 2048)).astype(np.float32))
    B.matmul(x, x)                                           # first launch of the kernel: module load, attributes
    B.syncGpu()
    t0 = time.perf_counter()
    for _ in range(24):                                      # fp32 FMA GEMMs: a long queue
        x2 = B.matmul(x, x)
    queued = time.perf_counter() - t0
    got = [ld.nextDeviceBatch() for _ in range(7)]
    B.syncGpu()
    busy = time.perf_counter() - t0
    assert busy > 2 * queued                                 # the requests really ran ahead of the device
    for i, t in got:
        wi, wt = ref.nextBatch()
        assert i._host is None and np.array_equal(i.data, wi) and np.array_equal(t.data, wt)
    ld.close()
    B.checkAsyncError()
