"""GPT model of the reference, restated on the oracle tape.  TEST INFRASTRUCTURE ONLY.

Follows ``packages/model/src/gpt.ts``: ``initGPT`` (:73-151, draw order wte, wpe, then per
layer the MLP weights *before* wqkv and wo, finally lmHead; std 0.02, and 0.02/sqrt(2L) for
wo / fc2 / fc_proj), ``transformerBlock`` (:220-333) and ``gptForward`` (:344-427).  The
attention is the *standard* branch (:256-279), which is what the reference runs on its CPU
backend (cpu_ref has no flashAttention hook).  ``flash_attention_dense`` restates the
contract of the optional hook (``packages/core/src/interfaces.ts:127-135``) for op-level
tests, including the raw-reshape head layout of gpt.ts:250-254.

EXTENSIONS (needed by the benchmarked model shapes, absent from the reference):
``tied`` (lm head shares wte; follows the reference's own written plan in
docs/GPT2-PLAN.md:68-88), ``norm="rms"``, ``rope``, and ``init="plain"`` (every linear and
embedding weight N(0, 0.02) without the residual-scaled std).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np

from . import autograd as ag
from .autograd import Ctx, Tape, Variable
from .cpu_ref import CpuRef, SeededRng, f32, f64


@dataclass
class ModelConfig:
    """packages/core/src/types.ts:51-64 plus the EXTENSION switches."""
    vocabSize: int = 256
    blockSize: int = 256
    nLayer: int = 6
    nEmbd: int = 256
    nHead: int = 8
    dropout: float = 0.0
    ffnActivation: str = "gelu"          # "gelu" | "swiglu"
    ffnDim: int | None = None
    softCap: float | None = None         # None -> 30.0 (gpt.ts:244); 0 disables (EXTENSION)
    tied: bool = False                   # EXTENSION
    norm: str = "layer"                  # EXTENSION: "layer" | "rms"
    rope: bool = False                   # EXTENSION
    init: str = "reference"              # "reference" | "plain" (EXTENSION)

    def ffn_dim(self) -> int:
        if self.ffnDim is not None:
            return self.ffnDim
        if self.ffnActivation == "swiglu":
            return int(math.ceil((8 / 3) * self.nEmbd / 64) * 64)
        return 4 * self.nEmbd


def init_gpt(cfg: ModelConfig, rng: SeededRng) -> dict:
    """gpt.ts:73-151.  Returns an ordered dict name -> Variable using the names of
    collectParamEntries (:433-468)."""
    V, T, L, E = cfg.vocabSize, cfg.blockSize, cfg.nLayer, cfg.nEmbd
    F = cfg.ffn_dim()
    std = 0.02
    rstd = std / math.sqrt(2 * L) if cfg.init == "reference" else std

    def w(shape, s):
        return Variable(rng.fill_gauss(shape, s), True)

    def norm_params():
        p = {"weight": Variable(np.ones(E, f32), True)}
        if cfg.norm == "layer":
            p["bias"] = Variable(np.zeros(E, f32), True)
        return p

    drawn = {"wte": w((V, E), std)}
    if not cfg.rope:
        drawn["wpe"] = w((T, E), std)
    layers = []
    for _ in range(L):
        lp = {}
        if cfg.ffnActivation == "swiglu":
            lp["mlp.fc_gate"] = w((F, E), std)
            lp["mlp.fc_up"] = w((F, E), std)
            lp["mlp.fc_proj"] = w((E, F), rstd)
        else:
            lp["mlp.fc1"] = w((F, E), std)
            lp["mlp.fc2"] = w((E, F), rstd)
        lp["ln1"] = norm_params()
        lp["attn.wqkv"] = w((3 * E, E), std)
        lp["attn.wo"] = w((E, E), rstd)
        lp["ln2"] = norm_params()
        layers.append(lp)
    lnF = norm_params()
    lm_head = drawn["wte"] if cfg.tied else w((V, E), std)

    # entry order of collectParamEntries (gpt.ts:433-468)
    P: dict[str, Variable] = {"wte": drawn["wte"]}
    if not cfg.rope:
        P["wpe"] = drawn["wpe"]
    if not cfg.tied:
        P["lmHead"] = lm_head
    for k, v in lnF.items():
        P[f"lnF.{k}"] = v
    for i, lp in enumerate(layers):
        for k, v in lp["ln1"].items():
            P[f"layer.{i}.ln1.{k}"] = v
        P[f"layer.{i}.attn.wqkv"] = lp["attn.wqkv"]
        P[f"layer.{i}.attn.wo"] = lp["attn.wo"]
        for k, v in lp["ln2"].items():
            P[f"layer.{i}.ln2.{k}"] = v
        for k in ("mlp.fc_gate", "mlp.fc_up", "mlp.fc_proj", "mlp.fc1", "mlp.fc2"):
            if k in lp:
                P[f"layer.{i}.{k}"] = lp[k]
    return P


def _norm(ctx, cfg, x, P, prefix):
    if cfg.norm == "rms":
        return ag.rmsNorm(ctx, x, P[f"{prefix}.weight"], 1e-5)
    return ag.layerNorm(ctx, x, P[f"{prefix}.weight"], P[f"{prefix}.bias"], 1e-5)


def _block(ctx: Ctx, cfg: ModelConfig, x: Variable, P: dict, i: int, Bn: int, T: int, mask) -> Variable:
    """gpt.ts:220-333, standard-attention branch."""
    E, H = cfg.nEmbd, cfg.nHead
    D = E // H
    pre = f"layer.{i}"
    ln1 = _norm(ctx, cfg, x, P, f"{pre}.ln1")
    q3d = ag.reshape(ctx, ln1, (Bn * T, E))
    qkv = ag.matmulTransposed(ctx, q3d, P[f"{pre}.attn.wqkv"])
    qf, kf, vf = ag.sliceQkv(ctx, qkv)
    q = ag.reshape(ctx, qf, (Bn, T, E))
    k = ag.reshape(ctx, kf, (Bn, T, E))
    v = ag.reshape(ctx, vf, (Bn, T, E))
    if cfg.rope:
        q = ag.rope(ctx, q, H)
        k = ag.rope(ctx, k, H)
    cap = 30.0 if cfg.softCap is None else cfg.softCap

    qH = ag.transpose(ctx, ag.reshape(ctx, q, (Bn, T, H, D)), 1, 2)
    kH = ag.transpose(ctx, ag.reshape(ctx, k, (Bn, T, H, D)), 1, 2)
    vH = ag.transpose(ctx, ag.reshape(ctx, v, (Bn, T, H, D)), 1, 2)
    kT = ag.transpose(ctx, kH, 2, 3)
    scores = ag.scale(ctx, ag.matmul(ctx, qH, kT), 1 / math.sqrt(D))
    if cap and cap > 0:
        scores = ag.softCap(ctx, scores, cap)
    masked = ag.maskedFillEntry(ctx, scores, mask, -1e9)
    att = ag.softmax(ctx, masked, -1)
    out = ag.matmul(ctx, att, vH)
    concat = ag.reshape(ctx, ag.transpose(ctx, out, 1, 2), (Bn * T, E))
    proj = ag.reshape(ctx, ag.matmulTransposed(ctx, concat, P[f"{pre}.attn.wo"]), (Bn, T, E))
    x = ag.add(ctx, x, proj)

    ln2 = _norm(ctx, cfg, x, P, f"{pre}.ln2")
    flat = ag.reshape(ctx, ln2, (Bn * T, E))
    if cfg.ffnActivation == "swiglu":
        gate = ag.matmulTransposed(ctx, flat, P[f"{pre}.mlp.fc_gate"])
        up = ag.matmulTransposed(ctx, flat, P[f"{pre}.mlp.fc_up"])
        h = ag.matmulTransposed(ctx, ag.siluMul(ctx, gate, up), P[f"{pre}.mlp.fc_proj"])
    else:
        h = ag.matmulTransposed(ctx, ag.matmulTransposedGelu(ctx, flat, P[f"{pre}.mlp.fc1"]),
                                P[f"{pre}.mlp.fc2"])
    return ag.add(ctx, x, ag.reshape(ctx, h, (Bn, T, E)))


def gpt_forward(cfg: ModelConfig, P: dict, B: CpuRef, tape: Tape, tokens: np.ndarray,
                targets: np.ndarray | None = None):
    """gpt.ts:344-427.  tokens/targets: int32 [B, T].  Returns (logits Variable, loss Variable|None)."""
    ctx = Ctx(tape, B)
    Bn, T = tokens.shape
    E = cfg.nEmbd
    x = ag.embedding(ctx, P["wte"], tokens)
    if not cfg.rope:
        pos = np.tile(np.arange(T, dtype=np.int32), (Bn, 1))
        x = ag.add(ctx, x, ag.embedding(ctx, P["wpe"], pos))
    mask = B.causalMask(T)
    for i in range(cfg.nLayer):
        x = _block(ctx, cfg, x, P, i, Bn, T, mask)
    x = _norm(ctx, cfg, x, P, "lnF")
    flat = ag.reshape(ctx, x, (Bn * T, E))
    head = P["wte"] if cfg.tied else P["lmHead"]
    logits = ag.reshape(ctx, ag.matmulTransposed(ctx, flat, head), (Bn, T, cfg.vocabSize))
    loss = None
    if targets is not None:
        lv = ag.reshape(ctx, logits, (Bn * T, cfg.vocabSize))
        loss = ag.crossEntropy(ctx, lv, targets.reshape(-1))
    return logits, loss


# ── the optional fused-attention hook, as a dense f64 computation ──────────────
def flash_attention_dense(q, k, v, T, scale, soft_cap):
    """Contract of Backend.flashAttention (interfaces.ts:127-135; kernel semantics in
    packages/helios/src/kernels/attention.ts:427-450,552-558): per [BH] slice
    s = scale*q.k ; optional s = tanh(s/cap)*cap ; causal mask ; softmax ; O = P v ;
    LSE = max + ln(sum).  q,k,v: [BH,T,D] float32.  Returns (O f32, LSE f32)."""
    q64, k64, v64 = q.astype(f64), k.astype(f64), v.astype(f64)
    s = np.einsum("bid,bjd->bij", q64, k64) * scale
    if soft_cap and soft_cap > 0:
        s = np.tanh(s / soft_cap) * soft_cap
    causal = np.triu(np.ones((T, T), dtype=bool), 1)
    s = np.where(causal[None], -np.inf, s)
    m = s.max(-1, keepdims=True)
    e = np.exp(s - m)
    l = e.sum(-1, keepdims=True)
    o = np.einsum("bij,bjd->bid", e / l, v64)
    return o.astype(f32), (m + np.log(l))[..., 0].astype(f32)


def flash_attention_dense_backward(q, k, v, o, do, lse, T, scale, soft_cap):
    """Contract of Backend.flashAttentionBackward (interfaces.ts:130-135; math in
    packages/helios/src/kernels/attention.ts:1217-1231,1411-1427): P is rebuilt from LSE,
    D_i = dO_i . O_i, dS = P*(dP - D_i) times the softcap derivative 1 - tanh^2."""
    q64, k64, v64, do64 = (t.astype(f64) for t in (q, k, v, do))
    raw = np.einsum("bid,bjd->bij", q64, k64) * scale
    if soft_cap and soft_cap > 0:
        th = np.tanh(raw / soft_cap)
        s, dcap = th * soft_cap, 1 - th * th
    else:
        s, dcap = raw, 1.0
    causal = np.triu(np.ones((T, T), dtype=bool), 1)
    p = np.where(causal[None], 0.0, np.exp(s - lse.astype(f64)[..., None]))
    dv = np.einsum("bij,bid->bjd", p, do64)
    dp = np.einsum("bid,bjd->bij", do64, v64)
    di = (do64 * o.astype(f64)).sum(-1, keepdims=True)
    ds = p * (dp - di) * dcap * scale
    dq = np.einsum("bij,bjd->bid", ds, k64)
    dk = np.einsum("bij,bid->bjd", ds, q64)
    return dq.astype(f32), dk.astype(f32), dv.astype(f32)
