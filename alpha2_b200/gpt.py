"""GPT model — host-side mirror of ``packages/model/src/gpt.ts`` driving the CUDA backend.

``initGPT`` (:73-151) draws the reference's weights for a seed: wte, wpe, then per layer
the MLP matrices *before* wqkv and wo, finally lmHead; std 0.02, residual projections
0.02/sqrt(2L).  ``gptForward`` (:344-427) has three attention routes:

* ``attention="standard"`` — the op sequence of the reference's CPU path (:256-279):
  head split by reshape/transpose, QK^T, scale, softCap, maskedFill, softmax, PV, merge.
* ``attention="flash"``    — the reference's fused-hook route (:248-254) with the head
  split done correctly ([B,T,H,D] -> [B,H,T,D] before the hook).  The reference feeds the
  hook a raw reshape of [B,T,E] to [B*H,T,D] with no transpose, which computes a different
  function from its own CPU path and lets queries see future tokens; that literal behaviour
  is available as ``attention="flash_raw_reshape"`` for interface tests only.
* ``attention="fused"``    — this backend's route: QKV read in place, no split/merge
  copies, GELU and residual adds in GEMM epilogues, fused head + loss.

Extensions asked for by the benchmark configurations and absent from the reference:
tied head (``tied``), RMSNorm (``norm="rms"``), RoPE (``rope``), bf16 compute with f32
master weights (``compute_dtype="bf16"``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

from . import autograd as ag
from .autograd import Ctx, Param, Tape, Variable
from .backend import CudaBackend, TensorData
from .rng import SeededRng


@dataclass
class ModelConfig:
    """packages/core/src/types.ts:51-64 (+ extension switches)."""
    vocabSize: int = 256
    blockSize: int = 256
    nLayer: int = 6
    nEmbd: int = 256
    nHead: int = 8
    dropout: float = 0.0
    ffnActivation: str = "gelu"
    ffnDim: int | None = None
    softCap: float | None = None      # None -> 30.0 (gpt.ts:244); 0 disables
    tied: bool = False
    norm: str = "layer"
    rope: bool = False
    init: str = "reference"           # "plain": every matrix N(0, 0.02)
    compute_dtype: str = "f32"        # "bf16": bf16 activations/weight shadows, f32 masters

    def ffn_dim(self) -> int:
        if self.ffnDim is not None:
            return self.ffnDim
        if self.ffnActivation == "swiglu":
            return int(math.ceil((8 / 3) * self.nEmbd / 64) * 64)
        return 4 * self.nEmbd


class GPTParams:
    """name -> Param in the order of collectParamEntries (gpt.ts:433-468)."""

    def __init__(self):
        self.entries: dict[str, Param] = {}

    def __getitem__(self, k: str) -> Param:
        return self.entries[k]

    def items(self):
        return self.entries.items()

    def values(self):
        return self.entries.values()


def _make_param(backend: CudaBackend, name: str, host: np.ndarray, cfg: ModelConfig, matrix: bool) -> Param:
    td = backend.upload(host, "f32")
    shadow = None
    if cfg.compute_dtype == "bf16" and matrix:
        shadow = backend.castDtype(td, "bf16")
    return Param(td, name, shadow)


def initGPT(cfg: ModelConfig, backend: CudaBackend, rng: SeededRng, host_params: dict | None = None) -> GPTParams:
    """gpt.ts:73-151.  ``host_params`` (name -> float32 array) overrides the draw, e.g. to
    start from weights produced elsewhere."""
    V, T, L, E = cfg.vocabSize, cfg.blockSize, cfg.nLayer, cfg.nEmbd
    F = cfg.ffn_dim()
    std = 0.02
    rstd = std / math.sqrt(2 * L) if cfg.init == "reference" else std
    drawn: dict[str, np.ndarray] = {}

    def w(name, shape, s):
        drawn[name] = rng.fill_gauss(shape, s)

    w("wte", (V, E), std)
    if not cfg.rope:
        w("wpe", (T, E), std)
    for i in range(L):
        if cfg.ffnActivation == "swiglu":
            w(f"layer.{i}.mlp.fc_gate", (F, E), std)
            w(f"layer.{i}.mlp.fc_up", (F, E), std)
            w(f"layer.{i}.mlp.fc_proj", (E, F), rstd)
        else:
            w(f"layer.{i}.mlp.fc1", (F, E), std)
            w(f"layer.{i}.mlp.fc2", (E, F), rstd)
        w(f"layer.{i}.attn.wqkv", (3 * E, E), std)
        w(f"layer.{i}.attn.wo", (E, E), rstd)
    if not cfg.tied:
        w("lmHead", (V, E), std)

    order = ["wte"] + ([] if cfg.rope else ["wpe"]) + ([] if cfg.tied else ["lmHead"])
    norm_suffixes = ["weight"] if cfg.norm == "rms" else ["weight", "bias"]
    order += [f"lnF.{s}" for s in norm_suffixes]
    for i in range(L):
        order += [f"layer.{i}.ln1.{s}" for s in norm_suffixes]
        order += [f"layer.{i}.attn.wqkv", f"layer.{i}.attn.wo"]
        order += [f"layer.{i}.ln2.{s}" for s in norm_suffixes]
        if cfg.ffnActivation == "swiglu":
            order += [f"layer.{i}.mlp.fc_gate", f"layer.{i}.mlp.fc_up", f"layer.{i}.mlp.fc_proj"]
        else:
            order += [f"layer.{i}.mlp.fc1", f"layer.{i}.mlp.fc2"]

    P = GPTParams()
    for name in order:
        if name in drawn:
            host = drawn[name]
        elif name.endswith(".weight"):
            host = np.ones(E, np.float32)
        else:
            host = np.zeros(E, np.float32)
        if host_params is not None:
            host = np.ascontiguousarray(host_params[name], dtype=np.float32).reshape(host.shape)
        P.entries[name] = _make_param(backend, name, host, cfg, matrix=name in drawn)
    return P


def collectParamEntries(params: GPTParams):
    return list(params.items())


def countParams(params: GPTParams) -> int:
    return sum(p.data.size for p in params.values())


# ── forward caches (gpt.ts:196-206) ───────────────────────────────────────────
_pos_cache: dict = {}
_mask_cache: dict = {}


def clearForwardCache():
    _pos_cache.clear()
    _mask_cache.clear()


def _norm(ctx, cfg, x, P, prefix):
    if cfg.norm == "rms":
        return ag.rmsNorm(ctx, x, P[f"{prefix}.weight"], 1e-5)
    return ag.layerNorm(ctx, x, P[f"{prefix}.weight"], P[f"{prefix}.bias"], 1e-5)


def _lin(ctx, x, w):
    """matmulTransposed against the compute copy of a parameter."""
    return ag.linear(ctx, x, w)


def _block_reference(ctx: Ctx, cfg: ModelConfig, x: Variable, P: GPTParams, i: int, Bn: int, T: int,
                     mask: TensorData, attention: str, training: bool) -> Variable:
    """gpt.ts:220-333 op for op."""
    E, H = cfg.nEmbd, cfg.nHead
    D = E // H
    pre = f"layer.{i}"
    cap = 30.0 if cfg.softCap is None else cfg.softCap
    ln1 = _norm(ctx, cfg, x, P, f"{pre}.ln1")
    q3d = ag.reshape(ctx, ln1, (Bn * T, E))
    qkv = _lin(ctx, q3d, P[f"{pre}.attn.wqkv"])
    if cfg.rope:
        qkv = ag.ropeQk(ctx, qkv, Bn, T, H)
    qf, kf, vf = ag.sliceQkv(ctx, qkv)
    q = ag.reshape(ctx, qf, (Bn, T, E))
    k = ag.reshape(ctx, kf, (Bn, T, E))
    v = ag.reshape(ctx, vf, (Bn, T, E))
    scale_ = 1 / math.sqrt(D)
    if attention == "flash_raw_reshape":                      # gpt.ts:248-254, literally
        qFA, kFA, vFA = (ag.reshape(ctx, t, (Bn * H, T, D)) for t in (q, k, v))
        att = ag.flashAttention(ctx, qFA, kFA, vFA, T, scale_, cap)
        concat = ag.reshape(ctx, ag.transpose(ctx, ag.reshape(ctx, att, (Bn, H, T, D)), 1, 2), (Bn * T, E))
    elif attention == "flash":
        split = lambda t: ag.reshape(ctx, ag.transpose(ctx, ag.reshape(ctx, t, (Bn, T, H, D)), 1, 2), (Bn * H, T, D))
        att = ag.flashAttention(ctx, split(q), split(k), split(v), T, scale_, cap)
        concat = ag.reshape(ctx, ag.transpose(ctx, ag.reshape(ctx, att, (Bn, H, T, D)), 1, 2), (Bn * T, E))
    else:                                                      # gpt.ts:256-279
        qH = ag.transpose(ctx, ag.reshape(ctx, q, (Bn, T, H, D)), 1, 2)
        kH = ag.transpose(ctx, ag.reshape(ctx, k, (Bn, T, H, D)), 1, 2)
        vH = ag.transpose(ctx, ag.reshape(ctx, v, (Bn, T, H, D)), 1, 2)
        kT = ag.transpose(ctx, kH, 2, 3)
        scores = ag.scale(ctx, ag.matmul(ctx, qH, kT), scale_)
        if cap > 0:
            scores = ag.softCap(ctx, scores, cap)
        masked = Variable(ctx.backend.maskedFill(scores.data, mask, -1e9), True)
        ctx.tape.record(masked, [scores], lambda g, B, rel, n: [B.maskedFill(g, mask, 0)])
        attw = ag.dropout(ctx, ag.softmax(ctx, masked, -1), cfg.dropout, training)
        out = ag.matmul(ctx, attw, vH)
        concat = ag.reshape(ctx, ag.transpose(ctx, out, 1, 2), (Bn * T, E))
    proj = ag.reshape(ctx, _lin(ctx, concat, P[f"{pre}.attn.wo"]), (Bn, T, E))
    x = ag.residualDropoutAdd(ctx, x, proj, cfg.dropout, training)

    ln2 = _norm(ctx, cfg, x, P, f"{pre}.ln2")
    flat = ag.reshape(ctx, ln2, (Bn * T, E))
    if cfg.ffnActivation == "swiglu":
        gate = _lin(ctx, flat, P[f"{pre}.mlp.fc_gate"])
        up = _lin(ctx, flat, P[f"{pre}.mlp.fc_up"])
        h = _lin(ctx, ag.siluMul(ctx, gate, up), P[f"{pre}.mlp.fc_proj"])
    else:
        h = _lin(ctx, ag.linearGelu(ctx, flat, P[f"{pre}.mlp.fc1"]), P[f"{pre}.mlp.fc2"])
    return ag.residualDropoutAdd(ctx, x, ag.reshape(ctx, h, (Bn, T, E)), cfg.dropout, training)


def _block_fused(ctx: Ctx, cfg: ModelConfig, x: Variable, P: GPTParams, i: int, Bn: int, T: int) -> Variable:
    """Same math as gpt.ts:220-333 on [B*T, E] activations with this backend's fused ops."""
    E, H = cfg.nEmbd, cfg.nHead
    D = E // H
    pre = f"layer.{i}"
    cap = 30.0 if cfg.softCap is None else cfg.softCap
    ln1 = _norm(ctx, cfg, x, P, f"{pre}.ln1")
    x = ag.attentionBlock(ctx, ln1, P[f"{pre}.attn.wqkv"], P[f"{pre}.attn.wo"], x, Bn, T, H, 1 / math.sqrt(D), cap,
                          ropeTheta=10000.0 if cfg.rope else None)
    ln2 = _norm(ctx, cfg, x, P, f"{pre}.ln2")
    if cfg.ffnActivation == "swiglu":
        gate = ag.linear(ctx, ln2, P[f"{pre}.mlp.fc_gate"])
        up = ag.linear(ctx, ln2, P[f"{pre}.mlp.fc_up"])
        return ag.linearAdd(ctx, ag.siluMul(ctx, gate, up), P[f"{pre}.mlp.fc_proj"], x)
    return ag.mlpGelu(ctx, ln2, P[f"{pre}.mlp.fc1"], P[f"{pre}.mlp.fc2"], x)


def gptForward(cfg: ModelConfig, params: GPTParams, backend: CudaBackend, tape: Tape, tokens: TensorData,
               targets: TensorData | None = None, training: bool = False, attention: str = "fused",
               dropoutRng=None, release=None, lossGradScale: float = 1.0, lastOnly: bool = False,
               activationCheckpointing: bool = False):
    """gpt.ts:344-427.  tokens/targets: int32 [B, T].  Returns {"logits": Variable|None, "loss": Variable|None}.
    ``lastOnly`` (fused route, no targets): project only each sequence's last position —
    logits [B, 1, V], what sampling reads (sample.ts:62-72) — instead of all T rows.
    ``activationCheckpointing`` (with ``training``): every transformer block becomes one
    checkpointed segment (gpt.ts:393-403), recomputed during backward."""
    ctx = Ctx(tape, backend, dropoutRng, release)
    Bn, T = tokens.shape
    E = cfg.nEmbd
    P = params
    head = P["wte"] if cfg.tied else P["lmHead"]
    dt = cfg.compute_dtype

    if attention == "fused":
        if cfg.dropout != 0 and training:
            raise ValueError("the fused route is built for dropout 0 (all benchmark configurations)")
        if cfg.rope:
            wte_c = P["wte"].shadow if P["wte"].shadow is not None else P["wte"].data
            vocab = cfg.vocabSize
            emb = backend.reshape(backend.embedding(wte_c, tokens), (Bn * T, E))
            x = ag._record(ctx, emb, [P["wte"]], lambda g, B, rel, n: [B.embeddingBackward(tokens, g, vocab)])
        else:
            x = ag.embeddingPos(ctx, P["wte"], P["wpe"], tokens)      # [B*T, E]
        for i in range(cfg.nLayer):
            if activationCheckpointing and training:
                x = ag.checkpoint(ctx, lambda c, xi, i=i: _block_fused(c, cfg, xi, P, i, Bn, T), x)
            else:
                x = _block_fused(ctx, cfg, x, P, i, Bn, T)
        x = _norm(ctx, cfg, x, P, "lnF")
        if targets is not None:
            tflat = backend.reshape(targets, (Bn * T,))
            return {"logits": None, "loss": ag.lmHeadLoss(ctx, x, head, tflat, lossGradScale)}
        if lastOnly:
            idx = backend.upload(np.arange(Bn, dtype=np.int32) * T + (T - 1), "i32")
            last = backend.embedding(x.data, idx)                  # row gather: [B, E]
            logits = backend.matmulTransposed(last, ag._compute_weight(head))
            backend.releaseGpuTensor(idx)
            backend.releaseGpuTensor(last)
            return {"logits": ag.Variable(backend.reshape(logits, (Bn, 1, cfg.vocabSize)), False), "loss": None}
        return {"logits": ag.reshape(ctx, ag.linear(ctx, x, head), (Bn, T, cfg.vocabSize)), "loss": None}

    # reference-shaped routes
    if dt != "f32":
        raise ValueError("the reference-shaped routes run in f32; use attention='fused' for bf16")
    tok_emb = ag.embedding(ctx, P["wte"], tokens)
    if cfg.rope:
        x = tok_emb
    else:
        key = (Bn, T, backend.device)
        pos = _pos_cache.get(key)
        if pos is None:
            pos = backend.upload(np.tile(np.arange(T, dtype=np.int32), (Bn, 1)), "i32")
            _pos_cache[key] = pos
        x = ag.add(ctx, tok_emb, ag.embedding(ctx, P["wpe"], pos))
    mask = _mask_cache.get((T, backend.device))
    if mask is None:
        mask = backend.causalMask(T)
        _mask_cache[(T, backend.device)] = mask
    for i in range(cfg.nLayer):
        if activationCheckpointing and training:
            x = ag.checkpoint(ctx, lambda c, xi, i=i: _block_reference(c, cfg, xi, P, i, Bn, T, mask, attention,
                                                                       training), x)
        else:
            x = _block_reference(ctx, cfg, x, P, i, Bn, T, mask, attention, training)
    x = _norm(ctx, cfg, x, P, "lnF")
    flat = ag.reshape(ctx, x, (Bn * T, E))
    logits = ag.reshape(ctx, _lin(ctx, flat, head), (Bn, T, cfg.vocabSize))
    loss = None
    if targets is not None:
        lv = ag.reshape(ctx, logits, (Bn * T, cfg.vocabSize))
        loss = ag.crossEntropy(ctx, lv, backend.reshape(targets, (Bn * T,)))
    return {"logits": logits, "loss": loss}
