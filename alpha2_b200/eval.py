"""Evaluation and sampling on the train-step kernels (forward only).

``evaluate`` mirrors packages/train/src/eval.ts:16-61: the mean loss over ``nBatches``
batches of a loader and its perplexity, with the tape cleared and the batch released after
every forward.  ``sample_tokens`` / ``sample`` mirror packages/train/src/sample.ts:22-201:
greedy for temperature <= 0, otherwise temperature scaling, top-k filtering, nucleus (top-p)
sampling or plain multinomial sampling, all on the host over the last position's logits
with the same order of operations and the same use of the random stream (one ``rng.next()``
per sampled token).  The device computes only that last row of logits (``lastOnly``).
"""
from __future__ import annotations

import math

import numpy as np

from .autograd import Tape
from .gpt import gptForward


def evaluate(config, params, backend, loader, nBatches: int = 50, attention: str = "fused") -> dict:
    release = getattr(backend, "releaseGpuTensor", None)
    flush = getattr(backend, "flush", None)
    total = 0.0
    for i in range(nBatches):
        inputs, targets = loader.nextBatch()
        ti, tt = backend.upload(inputs, "i32"), backend.upload(targets, "i32")
        tape = Tape()
        out = gptForward(config, params, backend, tape, ti, tt, training=False, attention=attention, release=release)
        loss = out["loss"]
        if loss is not None:
            total += float(np.asarray(loss.data.data, dtype=np.float32).reshape(-1)[0])   # eval.ts:43
            if release:
                release(loss.data)
        tape.clear(release)
        if release:
            release(ti)
            release(tt)
        if flush and (i & 7) == 7:
            flush()
    if flush:
        flush()
    avg = total / nBatches
    return {"loss": avg, "perplexity": math.exp(avg), "nBatches": nBatches}


def next_token(lastLogits: np.ndarray, rng, temperature: float, topk: int, topp: float | None) -> int:
    """One sampling decision over a row of logits (sample.ts:62-196); ``lastLogits`` is the raw
    row, float32."""
    vocab = lastLogits.shape[0]
    topP = min(1.0, max(0.0, topp)) if (topp is not None and math.isfinite(topp)) else 1.0
    if temperature <= 0:                                   # greedy: first maximum wins (:86-98)
        return int(np.argmax(lastLogits))
    logits = (lastLogits.astype(np.float64) / temperature).astype(np.float32)
    if 0 < topk < vocab:                                   # :107-114
        threshold = np.sort(logits)[::-1][topk - 1]
        logits = np.where(logits < threshold, np.float32(-np.inf), logits)
    if 0 < topP < 1:                                       # :117-168
        maxVal = float(np.max(logits))
        if math.isfinite(maxVal):
            finite = np.isfinite(logits)
            probs = np.zeros(vocab, np.float32)
            probs[finite] = np.exp(logits[finite].astype(np.float64) - maxVal).astype(np.float32)
            active = np.nonzero(finite)[0]
            sumExp = float(np.sum(probs[active].astype(np.float64)))
            if sumExp > 0 and active.size > 0:
                order = active[np.argsort(-probs[active], kind="stable")]
                target = sumExp * topP
                keptMass, keepCount = 0.0, 0
                while keepCount < order.size:
                    keptMass += float(probs[order[keepCount]])
                    if keptMass >= target:
                        keepCount += 1
                        break
                    keepCount += 1
                if keepCount <= 0:
                    keepCount = 1
                if keptMass <= 0:
                    keptMass = float(probs[order[0]])
                r = rng.next() * keptMass
                cum = 0.0
                sampled = int(order[keepCount - 1])
                for k in range(keepCount):
                    cum += float(probs[order[k]])
                    if r < cum:
                        sampled = int(order[k])
                        break
                return sampled
    maxVal = float(np.max(logits))                         # :171-195
    probs = np.exp(logits.astype(np.float64) - maxVal).astype(np.float32)
    sumExp = 0.0
    for p in probs:
        sumExp += float(p)
    probs = (probs.astype(np.float64) / sumExp).astype(np.float32)
    r = rng.next()
    cumsum = 0.0
    for v in range(vocab):
        cumsum += float(probs[v])
        if r < cumsum:
            return v
    return 0


def sample_tokens(config, params, backend, rng, promptTokens, steps: int, temperature: float = 1.0, topk: int = 0,
                  topp: float | None = None, attention: str = "fused") -> np.ndarray:
    """Token-level generation loop (sample.ts:36-199): the context is the tokens so far (at
    most blockSize of them); generation stops at ``steps`` new tokens or a full context."""
    release = getattr(backend, "releaseGpuTensor", None)
    flush = getattr(backend, "flush", None)
    prompt = np.asarray(promptTokens, dtype=np.int32).reshape(-1)
    maxLen = min(prompt.size + steps, config.blockSize)
    tokens = np.zeros(maxLen, np.int32)
    tokens[:min(prompt.size, maxLen)] = prompt[:maxLen]
    cur = min(prompt.size, maxLen)
    i = 0
    while i < steps and cur < config.blockSize:
        start = max(0, cur - config.blockSize)
        ctx = np.ascontiguousarray(tokens[start:cur]).reshape(1, -1)
        td = backend.upload(ctx, "i32")
        tape = Tape()
        out = gptForward(config, params, backend, tape, td, None, training=False, attention=attention,
                         release=release, lastOnly=(attention == "fused"))
        logits = np.asarray(out["logits"].data.data, dtype=np.float32).reshape(-1, config.vocabSize)[-1]
        tape.clear(release)
        if release:
            release(out["logits"].data)
            release(td)
        if flush and (i & 7) == 7:
            flush()
        nxt = next_token(logits, rng, temperature, topk, topp)
        if cur < maxLen:
            tokens[cur] = nxt
            cur += 1
        i += 1
    return tokens[:cur]


def sample(config, params, backend, rng, encode, decode, prompt: str, sampleConfig: dict, attention: str = "fused"):
    """sample.ts:22-33 signature: text in, text out, through the caller's tokenizer functions."""
    toks = sample_tokens(config, params, backend, rng, encode(prompt), int(sampleConfig.get("steps", 0)),
                         float(sampleConfig.get("temperature", 1.0)), int(sampleConfig.get("topk", 0)),
                         sampleConfig.get("topp"), attention)
    return decode(toks)
