"""Train-step parity at the full stated shapes, against fixtures the CPU oracle produced.

The oracle takes minutes per step at these sizes, so ``tests/golden/make_step_fixtures.py`` ran
it once and its losses, gradient norms and parameter samples are committed
(``tests/golden/step_*.npz``).  Here the CUDA library replays the same seeded weights and the
same seeded batches:

* small GPT (vocab 4096, 6 layers, width 384, context 256) at batch 32 for 100 steps,
* the GPT-2-124M shape (12 layers, width 768, vocab 50257, context 1024, tied head), 3 steps,
* the 350M shape (24 layers, width 1024, context 2048, RMSNorm, SwiGLU, RoPE, untied head) on
  sequences of 1024 tokens with two accumulated micro-steps, 2 steps,

each in fp32 and in bf16 (fp32 master weights and AdamW state).  Tolerances, with what the
committed build measures in brackets: fp32 — loss within 1e-5 relative at every step [8.9e-8
over the 100 steps, 1.9e-7 at the 124M shape], gradient norm within 5e-4 relative [4.1e-5,
3.1e-6], every parameter tensor's sample within 1e-4 relative (L2) plus the absolute floor the
other step tests use (AdamW moves an element whose gradient is rounding noise by up to about
lr); bf16 — loss within 2e-3 relative at every step [1.9e-4 over the 100 steps, 4.7e-4 at the
124M shape], gradient norm within 1e-1 relative in runs of up to ten steps [7.6e-3] and, over
the 100-step run, where the norm itself falls to 0.2 and jitters by a factor of two from step
to step, within 2e-1 at every step [0.109 at step 65] and 5e-2 on average [0.019].  The
reference's own criterion for this comparison is a final-loss difference below 0.01
(apps/cli/src/commands/bench.ts:381-382); it is asserted as well [2.3e-5 in bf16].
"""
import math
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from tests.golden.make_step_fixtures import CASES, case_batches, sample_index

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def B():
    from alpha2_b200.backend import CudaBackend
    b = CudaBackend(0)
    yield b
    b.checkAsyncError()


def _sampled(tr, name):
    flat = np.asarray(tr.params[name].data.data, np.float32).reshape(-1)
    return flat, flat[sample_index(flat.size)]


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("case", list(CASES))
def test_step_trajectory_against_the_oracle_fixture(B, case, dtype):
    from alpha2_b200.gpt import ModelConfig
    from alpha2_b200.trainer import TrainConfig, Trainer
    path = os.path.join(GOLDEN, f"step_{case}.npz")
    if not os.path.exists(path):
        pytest.fail(f"fixture {path} is missing; run tests/golden/make_step_fixtures.py {case}")
    fx = np.load(path)
    spec = CASES[case]
    batches = case_batches(spec)
    assert np.array_equal(fx["batch_token_sums"], [int(t.sum()) + int(g.sum()) for t, g in batches])
    tr = Trainer(B, ModelConfig(**spec["model"], compute_dtype=dtype), TrainConfig(**spec["train"]))
    names = [str(n) for n in fx["param_names"]]
    assert names == [n for n, _ in tr.entries]
    for n in names:                                           # same seeded init, bit for bit
        _, got = _sampled(tr, n)
        assert np.array_equal(got, fx[f"init/{n}/sample"]), n
    f32_run = dtype == "f32"
    long_run = spec["steps"] > 10
    loss_tol, gn_tol = (1e-5, 5e-4) if f32_run else (2e-3, 2e-1 if long_run else 1e-1)
    acc = spec["accum"]
    worst_loss = worst_gn = sum_gn = 0.0
    for s in range(spec["steps"]):
        micro = [(B.upload(t, "i32"), B.upload(g, "i32")) for t, g in batches[s * acc:(s + 1) * acc]]
        r = tr.train_step(micro)
        assert math.isfinite(r["loss"]) and math.isfinite(r["gradNorm"])
        want_loss, want_gn = float(fx["loss"][s]), float(fx["gradNorm"][s])
        el, eg = abs(r["loss"] - want_loss) / abs(want_loss), abs(r["gradNorm"] - want_gn) / want_gn
        worst_loss, worst_gn, sum_gn = max(worst_loss, el), max(worst_gn, eg), sum_gn + eg
        assert el < loss_tol, (case, dtype, s, r["loss"], want_loss)
        assert eg < gn_tol, (case, dtype, s, r["gradNorm"], want_gn)
        assert abs(r["lr"] - float(fx["lr"][s])) < 1e-12
        if f32_run and (s + 1) in spec["snapshots"]:
            lr = spec["train"]["lr"]
            for n in names:
                flat, got = _sampled(tr, n)
                want = fx[f"step{s + 1}/{n}/sample"].astype(np.float64)
                err = np.linalg.norm(got.astype(np.float64) - want)
                bound = 1e-4 * np.linalg.norm(want) + 4 * lr * 1e-3 * math.sqrt(want.size)
                assert err < bound, (case, s, n, err, bound)
                full = float(np.linalg.norm(flat.astype(np.float64)))
                assert abs(full - float(fx[f"step{s + 1}/{n}/norm"])) <= 1e-4 * full + 4 * lr * 1e-3 * math.sqrt(flat.size)
    assert abs(r["loss"] - float(fx["loss"][-1])) < 0.01     # bench.ts:381-382
    assert f32_run or sum_gn / spec["steps"] < 5e-2
    print(f"{case} {dtype}: worst relative loss error {worst_loss:.2e}, gradient norm {worst_gn:.2e}")
    B.checkAsyncError()
    del tr
    B.purgeBufferPools()
