"""The oracle's forward/backward against an independent float64 torch.autograd model.

The reference holds no step-level golden values (its tests pin single ops only), so the
oracle's composite graph is cross-checked here against textbook float64 math computed by
torch.autograd: standard causal multi-head attention with tanh soft-capping, LayerNorm,
tanh-GELU, mean cross-entropy — and the RMSNorm / RoPE / SwiGLU / tied-head extensions.
"""
import math

import numpy as np
import pytest
import torch

from oracle.autograd import Tape
from oracle.cpu_ref import CpuRef, SeededRng
from oracle.gpt import (ModelConfig, flash_attention_dense, flash_attention_dense_backward,
                        gpt_forward, init_gpt)
from oracle.train import TrainConfig, Trainer, lr_at, no_decay_names, uniform_batches


def torch_model_loss(cfg: ModelConfig, P: dict, tokens, targets):
    t = {n: torch.tensor(v.data.astype(np.float64), requires_grad=True) for n, v in P.items()}
    Bn, T = tokens.shape
    E, H = cfg.nEmbd, cfg.nHead
    D = E // H
    tok = torch.tensor(tokens.astype(np.int64))

    def norm(x, pre):
        if cfg.norm == "rms":
            return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5) * t[f"{pre}.weight"]
        return torch.nn.functional.layer_norm(x, (E,), t[f"{pre}.weight"], t[f"{pre}.bias"], 1e-5)

    def rope(x):
        half = D // 2
        inv = 10000.0 ** (-torch.arange(half, dtype=torch.float64) * 2.0 / D)
        ang = torch.arange(T, dtype=torch.float64)[:, None] * inv[None]
        c, s = torch.cos(ang)[None, :, None], torch.sin(ang)[None, :, None]
        x4 = x.reshape(Bn, T, H, D)
        a, b = x4[..., :half], x4[..., half:]
        return torch.cat([a * c - b * s, b * c + a * s], -1).reshape(Bn, T, E)

    x = t["wte"][tok]
    if not cfg.rope:
        x = x + t["wpe"][torch.arange(T)][None]
    cap = 30.0 if cfg.softCap is None else cfg.softCap
    for i in range(cfg.nLayer):
        pre = f"layer.{i}"
        qkv = norm(x, f"{pre}.ln1") @ t[f"{pre}.attn.wqkv"].T
        q, k, v = qkv.split(E, dim=-1)
        if cfg.rope:
            q, k = rope(q), rope(k)
        q, k, v = (z.reshape(Bn, T, H, D).transpose(1, 2) for z in (q, k, v))
        s = q @ k.transpose(-1, -2) / math.sqrt(D)
        if cap > 0:
            s = torch.tanh(s / cap) * cap
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), -1e9)
        o = (torch.softmax(s, -1) @ v).transpose(1, 2).reshape(Bn, T, E)
        x = x + o @ t[f"{pre}.attn.wo"].T
        h = norm(x, f"{pre}.ln2")
        if cfg.ffnActivation == "swiglu":
            m = torch.nn.functional.silu(h @ t[f"{pre}.mlp.fc_gate"].T) * (h @ t[f"{pre}.mlp.fc_up"].T)
            x = x + m @ t[f"{pre}.mlp.fc_proj"].T
        else:
            m = torch.nn.functional.gelu(h @ t[f"{pre}.mlp.fc1"].T, approximate="tanh")
            x = x + m @ t[f"{pre}.mlp.fc2"].T
    x = norm(x, "lnF")
    head = t["wte"] if cfg.tied else t["lmHead"]
    logits = x @ head.T
    loss = torch.nn.functional.cross_entropy(logits.reshape(-1, cfg.vocabSize),
                                             torch.tensor(targets.reshape(-1).astype(np.int64)))
    loss.backward()
    return float(loss.detach()), {n: v.grad.numpy() for n, v in t.items()}


CASES = {
    "reference": ModelConfig(vocabSize=96, blockSize=16, nLayer=2, nEmbd=32, nHead=4),
    "tied_plain": ModelConfig(vocabSize=96, blockSize=16, nLayer=2, nEmbd=32, nHead=4, tied=True, init="plain"),
    "rms_rope_swiglu": ModelConfig(vocabSize=96, blockSize=16, nLayer=2, nEmbd=32, nHead=4, norm="rms",
                                   rope=True, ffnActivation="swiglu", ffnDim=48, softCap=0.0),
}


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_grads_match_float64_autograd(name):
    cfg = CASES[name]
    P = init_gpt(cfg, SeededRng(3))
    # larger weights than the 0.02 init so that every path carries signal
    for n, v in P.items():
        if v.data.ndim == 2:
            v.data *= np.float32(5.0)
    tokens, targets = uniform_batches(11, 1, 3, 16, 96)[0]
    B, tape = CpuRef(), Tape()
    _, loss = gpt_forward(cfg, P, B, tape, tokens, targets)
    tape.backward(loss, B)
    ref_loss, ref_g = torch_model_loss(cfg, P, tokens, targets)
    assert abs(float(loss.data) - ref_loss) < 2e-6 * max(1, abs(ref_loss))
    for n, v in P.items():
        g, r = v.grad.astype(np.float64), ref_g[n]
        err = np.linalg.norm(g - r) / max(np.linalg.norm(r), 1e-30)
        assert err < 5e-6, (n, err)


def test_init_order_and_std():
    """gpt.ts:73-151: draw order and the residual-scaled std of wo / fc2."""
    cfg = ModelConfig(vocabSize=50, blockSize=8, nLayer=2, nEmbd=16, nHead=2)
    P = init_gpt(cfg, SeededRng(42))
    r = SeededRng(42)
    assert np.array_equal(P["wte"].data, r.fill_gauss((50, 16), 0.02))
    assert np.array_equal(P["wpe"].data, r.fill_gauss((8, 16), 0.02))
    for i in range(2):
        assert np.array_equal(P[f"layer.{i}.mlp.fc1"].data, r.fill_gauss((64, 16), 0.02))
        assert np.array_equal(P[f"layer.{i}.mlp.fc2"].data, r.fill_gauss((16, 64), 0.02 / 2))
        assert np.array_equal(P[f"layer.{i}.attn.wqkv"].data, r.fill_gauss((48, 16), 0.02))
        assert np.array_equal(P[f"layer.{i}.attn.wo"].data, r.fill_gauss((16, 16), 0.02 / 2))
    assert np.array_equal(P["lmHead"].data, r.fill_gauss((50, 16), 0.02))
    assert list(P)[:5] == ["wte", "wpe", "lmHead", "lnF.weight", "lnF.bias"]   # gpt.ts:435-439
    assert np.all(P["lnF.weight"].data == 1) and np.all(P["layer.0.ln1.bias"].data == 0)


def test_lr_schedule():
    """trainer.ts:1088-1096,1150-1158: 20 iterations => 4 warm-up steps, lrMin = lr/10."""
    tc = TrainConfig(iters=20, lr=3e-4)
    lrs = [lr_at(tc, s) for s in range(20)]
    assert abs(lrs[0] - (3e-5 + 2.7e-4 * 1 / 4)) < 1e-12
    assert abs(lrs[3] - 3e-4) < 1e-12 and abs(lrs[4] - 3e-4) < 1e-12
    assert all(a >= b for a, b in zip(lrs[4:], lrs[5:]))
    assert abs(lr_at(TrainConfig(iters=20, lr=3e-4, warmupIters=-1), 0) - 3e-4) < 1e-12


def test_no_decay_set():
    s = no_decay_names(ModelConfig(nLayer=2))
    assert "wte" in s and "layer.1.ln2.bias" in s and "lmHead" not in s and "layer.0.attn.wo" not in s


def test_flash_hook_equals_standard_branch_math():
    """The fused-attention contract (interfaces.ts:127-135) against dense float64 autograd."""
    rng = np.random.default_rng(0)
    BH, T, D = 3, 12, 8
    q, k, v, do = (rng.standard_normal((BH, T, D)).astype(np.float32) for _ in range(4))
    for cap in (30.0, 0.0, 2.0):
        o, lse = flash_attention_dense(q, k, v, T, 1 / math.sqrt(D), cap)
        tq, tk, tv = (torch.tensor(z.astype(np.float64), requires_grad=True) for z in (q, k, v))
        s = tq @ tk.transpose(-1, -2) / math.sqrt(D)
        if cap > 0:
            s = torch.tanh(s / cap) * cap
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        to = torch.softmax(s, -1) @ tv
        np.testing.assert_allclose(o, to.detach().numpy(), rtol=2e-6, atol=2e-6)
        np.testing.assert_allclose(lse, torch.logsumexp(s, -1).detach().numpy(), rtol=2e-6, atol=2e-6)
        to.backward(torch.tensor(do.astype(np.float64)))
        dq, dk, dv = flash_attention_dense_backward(q, k, v, o, do, lse, T, 1 / math.sqrt(D), cap)
        for got, ref in ((dq, tq.grad), (dk, tk.grad), (dv, tv.grad)):
            np.testing.assert_allclose(got, ref.numpy(), rtol=1e-4, atol=2e-6)


def test_trainer_runs_and_clips():
    mc = ModelConfig(vocabSize=64, blockSize=16, nLayer=1, nEmbd=16, nHead=2)
    tc = TrainConfig(iters=6, batchSize=2, gradClip=0.5, seed=1)
    tr = Trainer(mc, tc)
    bs = uniform_batches(5, 2, 2, 16, 64)
    first = tr.train_step([bs[0]])
    assert first["clipCoef"] < 1.0 and abs(first["clipCoef"] - 0.5 / first["gradNorm"]) < 1e-12
    losses = [tr.train_step([bs[0]])["loss"] for _ in range(5)]
    assert losses[-1] < first["loss"]                 # same batch repeated: loss must fall
    acc = Trainer(mc, tc).train_step([bs[0], bs[1]])  # two micro-steps (trainer.ts:1188-1273)
    assert np.isfinite(acc["loss"]) and acc["gradNorm"] > 0
