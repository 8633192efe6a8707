"""Train-step parity on the GPU: the CUDA backend against the oracle on identical seeded
weights and tokens (the tiny byte-level GPT and the small GPT, plus reduced-size stand-ins of
the GPT-2-124M and 350M shapes; the full shapes are in tests/test_gpu_step_golden.py).

Tolerances (north star): fp32 path — loss within 1e-4 relative per step; every parameter
tensor within 1e-4 relative (L2) plus an absolute floor of a few learning-rate quanta
(AdamW moves an element whose gradient is reduction-order noise by up to ~lr in either
direction, so a pure relative bound per element is not meaningful).  bf16 path — loss
within 2e-2 relative.
"""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from oracle import gpt as ogpt
from oracle import train as otrain


@pytest.fixture(scope="module")
def B():
    from alpha2_b200.backend import CudaBackend
    b = CudaBackend(0)
    yield b
    b.checkAsyncError()


def oracle_cfg(mc):
    return ogpt.ModelConfig(**{k: getattr(mc, k) for k in
                               ("vocabSize", "blockSize", "nLayer", "nEmbd", "nHead", "ffnActivation", "ffnDim",
                                "softCap", "tied", "norm", "rope", "init")})


def run_parity(B, mc, tc_kwargs, batches, route, fused, steps, loss_rtol, param_rtol, dtype="f32", check_params=True):
    from alpha2_b200.gpt import ModelConfig
    from alpha2_b200.trainer import TrainConfig, Trainer
    mc = ModelConfig(**{**mc, "compute_dtype": dtype})
    tc = TrainConfig(**tc_kwargs)
    ref = otrain.Trainer(oracle_cfg(mc), otrain.TrainConfig(**tc_kwargs))
    tr = Trainer(B, mc, tc, attention=route, fused=fused)
    for n, v in ref.P.items():
        assert np.array_equal(v.data, tr.params[n].data.data), n      # same seeded init, bit for bit
    worst = 0.0
    for i in range(steps):
        tok, tgt = batches[i % len(batches)]
        a = tr.train_step([(B.upload(tok, "i32"), B.upload(tgt, "i32"))])
        b = ref.train_step([(tok, tgt)])
        assert math.isfinite(a["loss"])
        rel = abs(a["loss"] - b["loss"]) / abs(b["loss"])
        worst = max(worst, rel)
        assert rel < loss_rtol, (i, a["loss"], b["loss"])
        assert abs(a["gradNorm"] - b["gradNorm"]) < max(loss_rtol * 20, 2e-4) * max(1.0, b["gradNorm"]), (i, a, b)
        assert abs(a["lr"] - b["lr"]) < 1e-12
        if check_params and (i == 0 or i == steps - 1 or i % 5 == 4):
            atol_scale = 4 * tc.lr
            for n, v in ref.P.items():
                got = tr.params[n].data.data.astype(np.float64)
                want = v.data.astype(np.float64)
                err = np.linalg.norm(got - want)
                bound = param_rtol * np.linalg.norm(want) + atol_scale * 1e-3 * math.sqrt(want.size)
                assert err < bound, (i, n, err, bound)
    B.checkAsyncError()
    return worst


C1 = dict(vocabSize=256, blockSize=64, nLayer=2, nEmbd=64, nHead=4)
C1_TRAIN = dict(iters=20, batchSize=4, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, weightDecay=0.1, gradClip=1.0, seed=42)


@pytest.mark.parametrize("route,fused", [("fused", True), ("standard", False), ("flash", False)])
def test_config1_fp32_20_steps(B, route, fused):
    """The tiny byte-level GPT (vocab 256, 2 layers, width 64, 4 heads, context 64, batch 4),
    reference-faithful: untied head, soft cap 30, residual-scaled init."""
    batches = otrain.uniform_batches(123, 20, 4, 64, 256)
    run_parity(B, C1, C1_TRAIN, batches, route, fused, 20, 1e-4, 1e-4)


def test_config1_literal_tied_head(B):
    """The tiny byte-level GPT with N(0, 0.02) everywhere and tied embeddings."""
    batches = otrain.uniform_batches(124, 20, 4, 64, 256)
    run_parity(B, {**C1, "tied": True, "init": "plain"}, C1_TRAIN, batches, "fused", True, 20, 1e-4, 1e-4)


def test_config1_learns_a_repeated_batch(B):
    """A fixed small set of batches: the loss must fall, and fall the same way on both sides;
    also exercises clipping (gradClip 0.25 triggers on every step)."""
    batches = otrain.uniform_batches(7, 2, 4, 64, 256)
    train = {**C1_TRAIN, "iters": 30, "lr": 3e-3, "gradClip": 0.25}
    run_parity(B, C1, train, batches, "fused", True, 30, 2e-4, 5e-4)


def test_grad_accumulation_and_release(B):
    from alpha2_b200.gpt import ModelConfig
    from alpha2_b200.trainer import TrainConfig, Trainer
    mc = ModelConfig(**C1)
    tr = Trainer(B, mc, TrainConfig(**C1_TRAIN))
    ref = otrain.Trainer(oracle_cfg(mc), otrain.TrainConfig(**C1_TRAIN))
    bs = otrain.uniform_batches(9, 4, 4, 64, 256)
    for s in range(2):
        pair = bs[2 * s:2 * s + 2]
        a = tr.train_step([(B.upload(t, "i32"), B.upload(g, "i32")) for t, g in pair])
        b = ref.train_step(pair)
        assert abs(a["loss"] - b["loss"]) < 1e-4 * b["loss"] and abs(a["gradNorm"] - b["gradNorm"]) < 2e-4
    # steady state: no new device allocations from one step to the next, nothing leaks
    tr.train_step([(B.upload(bs[0][0], "i32"), B.upload(bs[0][1], "i32"))])
    B.syncGpu()
    s0 = B.gpuMemStats()
    for _ in range(3):
        tr.train_step([(B.upload(bs[0][0], "i32"), B.upload(bs[0][1], "i32"))])
    B.syncGpu()
    s1 = B.gpuMemStats()
    assert s1["deviceMallocs"] == s0["deviceMallocs"], (s0, s1)
    assert s1["bytesInUse"] == s0["bytesInUse"], (s0, s1)


C3 = dict(vocabSize=4096, blockSize=256, nLayer=6, nEmbd=384, nHead=6, tied=True, init="plain")
C3_TRAIN = dict(iters=100, batchSize=32, lr=3e-4, seed=42)


def test_config3_fp32(B):
    """The small GPT (vocab 4096, 6 layers, width 384, context 256) in fp32 against the oracle
    run at test time: batch reduced to 4 rows so that the CPU oracle finishes in seconds.  Batch
    32 for 100 steps is compared with a committed oracle trajectory in test_gpu_step_golden.py."""
    batches = otrain.zipf_batches(5, 3, 4, 256, 4096)
    run_parity(B, C3, C3_TRAIN, batches, "fused", True, 3, 1e-4, 1e-4)


def test_config3_bf16_loss(B):
    batches = otrain.zipf_batches(5, 4, 4, 256, 4096)
    worst = run_parity(B, C3, C3_TRAIN, batches, "fused", True, 4, 2e-2, 0, dtype="bf16", check_params=False)
    assert worst < 2e-2


def test_config4_shape_small_bf16(B):
    """GPT-2-small's vocabulary (50257: not a multiple of any tile), head dim 64, learned
    positions, tied head — two layers, short context, bf16, loss against the fp32 oracle."""
    mc = dict(vocabSize=50257, blockSize=128, nLayer=2, nEmbd=768, nHead=12, tied=True, init="plain")
    batches = otrain.zipf_batches(6, 2, 2, 128, 50257)
    run_parity(B, mc, dict(iters=10, batchSize=2, seed=1), batches, "fused", True, 2, 2e-2, 0, dtype="bf16",
               check_params=False)


def test_config5_shape_small(B):
    """RMSNorm + SwiGLU + RoPE + untied head (the 350M configuration's ingredients), small,
    fp32 for parameters and bf16 for the loss."""
    mc = dict(vocabSize=512, blockSize=64, nLayer=2, nEmbd=128, nHead=2, ffnActivation="swiglu", ffnDim=352,
              norm="rms", rope=True, softCap=0.0)
    batches = otrain.zipf_batches(8, 3, 4, 64, 512)
    tcfg = dict(iters=10, batchSize=4, seed=3)
    run_parity(B, mc, tcfg, batches, "fused", True, 3, 1e-4, 1e-4)
    run_parity(B, mc, tcfg, batches, "fused", True, 3, 2e-2, 0, dtype="bf16", check_params=False)


@pytest.mark.gpu
@pytest.mark.parametrize("arch", ["gpt2", "rms_rope_swiglu"])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_activation_checkpointing_on_the_device(B, dtype, arch):
    """Every block recomputed during backward (packages/autograd/src/checkpoint.ts): same
    losses and parameters as the plain run, bit for bit (the kernels are deterministic).  The
    second architecture rotates q and k in place on the projection's output, which the
    recompute has to produce afresh."""
    from alpha2_b200.gpt import ModelConfig
    from alpha2_b200.trainer import TrainConfig, Trainer
    extra = dict(tied=True) if arch == "gpt2" else dict(tied=False, ffnActivation="swiglu", ffnDim=352, norm="rms",
                                                        rope=True, softCap=0.0)
    mc = ModelConfig(vocabSize=512, blockSize=128, nLayer=3, nEmbd=128, nHead=2, init="plain",
                     compute_dtype=dtype, **extra)
    batches = otrain.zipf_batches(9, 3, 4, 128, 512)
    runs = []
    for ck in (False, True):
        tr = Trainer(B, mc, TrainConfig(iters=10, batchSize=4, gradClip=1.0, seed=11), activationCheckpointing=ck)
        losses = [tr.train_step([(B.upload(t, "i32"), B.upload(g, "i32"))])["loss"] for t, g in batches]
        runs.append((losses, {n: np.array(v.data.data) for n, v in tr.entries}))
    assert runs[0][0] == runs[1][0]
    for n in runs[0][1]:
        assert np.array_equal(runs[0][1][n], runs[1][1][n]), n
