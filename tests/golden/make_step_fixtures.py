"""Writes the train-step fixtures ``tests/golden/step_<case>.npz`` by running the CPU oracle.

    python tests/golden/make_step_fixtures.py [case ...]      (no argument: every case)

The oracle needs minutes per step at these sizes (f64 arithmetic with an f32 store after every
op, standard attention with its full [B, H, T, T] score tensors), far too long to repeat inside
a GPU test, so it is run once, here, and what it produced is committed.  The GPU tests
(``tests/test_gpu_step_golden.py``) replay the same seeded weights and batches through the CUDA
library and compare.  Every case is a model at its full stated shape:

* ``small_gpt_b32_100steps`` — vocab 4096, 6 layers, width 384, 6 heads, context 256, tied
  head, batch 32, Zipf(1.1) tokens, 100 optimizer steps.
* ``gpt2_124m_3steps`` — vocab 50257, 12 layers, width 768, 12 heads, context 1024, learned
  positions, GELU MLP 3072, tied head; one sequence of 1024 tokens per step, 3 steps.
* ``gpt_350m_accum2_2steps`` — vocab 32768, 24 layers, width 1024, 16 heads, context 2048,
  RMSNorm, SwiGLU 2816, RoPE, untied head; one sequence of 1024 tokens per micro-step (the
  oracle keeps every layer's dense [heads, T, T] score tensors for its backward pass: at 2048
  tokens that is more host memory than the 62 GB this was generated with), two accumulated
  micro-steps per optimizer step, 2 steps.

A fixture holds, per step: loss, gradient norm, learning rate, clip coefficient; at the
snapshot steps, for every parameter tensor: its L2 norm (f64) and a strided sample of at most
2048 elements (``sample_index``); the same sample of the initial weights; and the sum of every
batch's token ids, so that a reader can tell that it regenerated the same batches.
"""
from __future__ import annotations

import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SAMPLES = 2048

CASES = {
    "small_gpt_b32_100steps": dict(
        model=dict(vocabSize=4096, blockSize=256, nLayer=6, nEmbd=384, nHead=6, tied=True, init="plain"),
        train=dict(iters=100, batchSize=32, lr=3e-4, seed=42), data_seed=5, batch=32, accum=1, steps=100,
        snapshots=(1, 50, 100)),
    "gpt2_124m_3steps": dict(
        model=dict(vocabSize=50257, blockSize=1024, nLayer=12, nEmbd=768, nHead=12, tied=True, init="plain"),
        train=dict(iters=100, batchSize=1, lr=3e-4, seed=42), data_seed=6, batch=1, accum=1, steps=3,
        snapshots=(1, 3)),
    "gpt_350m_accum2_2steps": dict(
        model=dict(vocabSize=32768, blockSize=2048, nLayer=24, nEmbd=1024, nHead=16, tied=False,
                   ffnActivation="swiglu", ffnDim=2816, norm="rms", rope=True, init="plain"),
        train=dict(iters=100, batchSize=1, lr=3e-4, seed=42), data_seed=7, batch=1, accum=2, steps=2,
        snapshots=(1, 2), seq_len=1024),
}


def sample_index(n: int) -> np.ndarray:
    """Which flat elements of an n-element tensor a fixture keeps."""
    k = min(n, SAMPLES)
    return (np.arange(k, dtype=np.int64) * (n // k)).astype(np.int64)


def case_batches(case: dict):
    """The case's micro-batches, in order: ``steps * accum`` pairs of int32 [batch, T]."""
    from oracle import train as otrain
    m = case["model"]
    return otrain.zipf_batches(case["data_seed"], case["steps"] * case["accum"], case["batch"],
                               case.get("seq_len", m["blockSize"]), m["vocabSize"])


def snapshot(P: dict) -> dict:
    out = {}
    for name, v in P.items():
        flat = np.asarray(v.data, np.float32).reshape(-1)
        out[f"{name}/norm"] = np.float64(np.linalg.norm(flat.astype(np.float64)))
        out[f"{name}/sample"] = flat[sample_index(flat.size)].copy()
    return out


def generate(name: str) -> str:
    from oracle import gpt as ogpt
    from oracle import train as otrain
    case = CASES[name]
    tr = otrain.Trainer(ogpt.ModelConfig(**case["model"]), otrain.TrainConfig(**case["train"]))
    batches = case_batches(case)
    out = {"batch_token_sums": np.array([int(t.sum()) + int(g.sum()) for t, g in batches], np.int64)}
    for k, v in snapshot(tr.P).items():
        out[f"init/{k}"] = v
    rows = []
    acc = case["accum"]
    for s in range(case["steps"]):
        t0 = time.time()
        r = tr.train_step(batches[s * acc:(s + 1) * acc])
        rows.append([r["loss"], r["gradNorm"], r["lr"], r["clipCoef"]])
        print(f"{name}: step {s + 1}/{case['steps']} loss {r['loss']:.6f} gradNorm {r['gradNorm']:.6f} "
              f"({time.time() - t0:.0f} s)", flush=True)
        if s + 1 in case["snapshots"]:
            for k, v in snapshot(tr.P).items():
                out[f"step{s + 1}/{k}"] = v
    rows = np.array(rows, np.float64)
    out.update(loss=rows[:, 0], gradNorm=rows[:, 1], lr=rows[:, 2], clipCoef=rows[:, 3],
               param_names=np.array(list(tr.P.keys())))
    path = os.path.join(HERE, f"step_{name}.npz")
    np.savez_compressed(path, **out)
    return path


if __name__ == "__main__":
    for n in (sys.argv[1:] or list(CASES)):
        print(generate(n), flush=True)
