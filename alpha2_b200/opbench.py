"""Op microbenchmark over the C ABI (the train-step ops alone, at the GPT-2-124M step's shapes).

    python -m alpha2_b200.opbench [--op NAME ...] [--iters 10] [--json] [--cublas]

Ops and shapes (bf16 inputs, fp32 accumulation): GEMM forward / dX / dW at
[16384x768]x[768x{2304,3072}], [16384x3072]x[3072x768] and the lm head [16384x768]x[768x50257]
with A, B ~ N(0, 0.02); causal flash attention forward+backward at B=8, H=12, T=1024, D=64
with q, k, v, dO ~ N(0, 1); fused softmax-cross-entropy on logits [16384, 50257] ~ N(0, 1);
plus LayerNorm, AdamW and the embedding scatter-add at the train-step sizes.

Every launch is timed alone with CUDA events on the library's stream after 3 warm-up
launches; a 256 MiB buffer is overwritten between launches so that each one starts with a
cold L2 (``--flush read`` reads it instead: the lines a kernel evicts are then clean, while
with the default they are dirty and their write-back is part of what the kernel waits for).  Printed per op: mean device time, achieved TFLOP/s or GB/s from the algorithmic
work, and the fraction of the measured peak (MEASURED_PEAKS.json: burst figures, since the
kernel runs alone).

``--cublas`` adds a yardstick column for the GEMM rows: ``torch.matmul`` (cuBLAS) on the same
shape, layout and leading dimensions, timed the same way (CUDA events, cold L2).  It is there
only to say what a library GEMM reaches on that shape on that GPU; nothing in the library or
the train step calls it.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os

import numpy as np

from . import _lib as L
from ._lib import check
from .backend import CudaBackend

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["bf16_tflops"], d["hbm_gbs"], "measured"
    return 1590.0, 6650.0, "fallback"


class Bench:
    def __init__(self, iters: int, cublas: bool = False, flush: str = "write"):
        self.cublas = cublas
        self.flush = flush
        self.B = CudaBackend(0)
        self.lib = self.B.lib
        self.iters = iters
        buf = C.c_uint64()
        check(self.lib.alpha_alloc(256 << 20, C.byref(buf)))
        self.flush_ptr = buf.value
        self.ev = [C.c_uint64(), C.c_uint64()]
        for e in self.ev:
            check(self.lib.alpha_event_create(C.byref(e)))
        self.rng = np.random.default_rng(0)
        self.scalar = self.B._new((), "f32")

    def flush_l2(self):
        """write: L2 ends up full of dirty lines of another buffer (what a kernel meets inside a
        train step, where its predecessor's output is still dirty in L2: its own traffic then
        also pays for writing those lines back).  read: full of clean lines."""
        if self.flush == "write":
            check(self.lib.alpha_memset(self.flush_ptr, 1, 256 << 20))
        else:
            check(self.lib.alpha_check_finite(self.flush_ptr, (256 << 20) // 4, L.F32, self.scalar.ptr))

    def normal(self, shape, std, dtype="bf16"):
        n = int(np.prod(shape))
        # large tensors: tile a 4M-element block (the statistics are what matters here)
        block = (self.rng.standard_normal(min(n, 1 << 22)) * std).astype(np.float32)
        reps = -(-n // block.size)
        arr = np.tile(block, reps)[:n].reshape(shape)
        return self.B.upload(arr, dtype)

    def time(self, fn) -> float:
        for _ in range(3):
            fn()
        total = 0.0
        for _ in range(self.iters):
            self.flush_l2()
            check(self.lib.alpha_event_record(self.ev[0].value))
            fn()
            check(self.lib.alpha_event_record(self.ev[1].value))
            check(self.lib.alpha_event_sync(self.ev[1].value))
            ms = C.c_float()
            check(self.lib.alpha_event_elapsed_ms(self.ev[0].value, self.ev[1].value, C.byref(ms)))
            total += ms.value
        self.B.checkAsyncError()
        return total / self.iters


def gemm_case(b: Bench, layout: str, M: int, N: int, K: int, out_dtype: str = "bf16", epilogue: int = L.EPI_NONE):
    """Operands are allocated with leading dimensions padded to a multiple of 64 elements (as
    the train step lays out the logits), the logical extents stay M, N, K."""
    B = b.B
    pad = lambda n: (n + 63) // 64 * 64
    logical = {"nt": ((M, K), (N, K)), "nn": ((M, K), (K, N)), "tn": ((K, M), (K, N))}[layout]
    lda, ldb, ldc = pad(logical[0][1]), pad(logical[1][1]), pad(N)
    A, Bm = b.normal((logical[0][0], lda), 0.02), b.normal((logical[1][0], ldb), 0.02)
    Cc = B._new((M, ldc), out_dtype)
    aux = B._new((M, ldc), out_dtype) if epilogue != L.EPI_NONE else None
    code = {"nt": L.GEMM_NT, "nn": L.GEMM_NN, "tn": L.GEMM_TN}[layout]

    def fn():
        check(B.lib.alpha_gemm(code, A.ptr, Bm.ptr, Cc.ptr, M, N, K, lda, ldb, ldc, L.BF16, L.DTYPE_CODE[out_dtype],
                               epilogue, aux.ptr if aux is not None else 0, ldc, 0))
    ms = b.time(fn)
    r = {"ms": ms, "work": 2.0 * M * N * K, "kind": "flop"}
    if b.cublas and epilogue == L.EPI_NONE:
        r["cublas_ms"] = cublas_gemm_ms(b, layout, M, N, K, lda, ldb, out_dtype)
    return r


def cublas_gemm_ms(b: Bench, layout: str, M: int, N: int, K: int, lda: int, ldb: int, out_dtype: str) -> float:
    """torch.matmul on strided views with the same leading dimensions; fp32 output where the
    library's GEMM writes fp32 (weight gradients) if this torch offers it, else bf16."""
    import torch
    dev = torch.device("cuda", 0)
    rows_a, rows_b = (K if layout == "tn" else M), (N if layout == "nt" else K)
    a = (torch.randn(rows_a, lda, device=dev) * 0.02).to(torch.bfloat16)
    bm = (torch.randn(rows_b, ldb, device=dev) * 0.02).to(torch.bfloat16)
    A = a[:, :M].t() if layout == "tn" else a[:, :K]
    Bm = bm[:, :K].t() if layout == "nt" else bm[:, :N]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    fn = lambda: torch.matmul(A, Bm)
    if out_dtype == "f32":
        try:
            torch.mm(A, Bm, out_dtype=torch.float32)
            fn = lambda: torch.mm(A, Bm, out_dtype=torch.float32)
        except Exception:
            pass
    for _ in range(3):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total = 0.0
    for _ in range(b.iters):
        flush.fill_(1)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        total += e0.elapsed_time(e1)
    return total / b.iters


def dw_pair_case(b: Bench, s0, s1, K):
    """Two weight gradients A_i^T B_i over one K in one launch (alpha_gemm_tn_pair), as the MLP's backward issues them."""
    B = b.B
    ops = [(b.normal((K, M), 0.02), b.normal((K, N), 0.02), B._new((M, N), "f32")) for M, N in (s0, s1)]
    ms = b.time(lambda: B.matmulTransposedAPair(*ops))
    return {"ms": ms, "work": 2.0 * K * (s0[0] * s0[1] + s1[0] * s1[1]), "kind": "flop"}


def attn_case(b: Bench, Bn=16, H=12, T=1024, D=64, backward=False, dtype="bf16", cap=30.0):
    B = b.B
    E = H * D
    qkv = b.normal((Bn * T, 3 * E), 1.0, dtype)
    dout = b.normal((Bn * T, E), 1.0, dtype)
    scale = 1 / math.sqrt(D)
    out, lse = B.attentionQkv(qkv, Bn, T, H, scale, cap)
    if not backward:
        ms = b.time(lambda: B.attentionQkv(qkv, Bn, T, H, scale, cap))
        return {"ms": ms, "work": 4.0 * Bn * H * T * T * D, "kind": "flop"}
    ms = b.time(lambda: B.attentionQkvBackward(qkv, out, dout, lse, Bn, T, H, scale, cap))
    return {"ms": ms, "work": 8.0 * Bn * H * T * T * D, "kind": "flop"}


def ce_case(b: Bench, N=16384, V=50257):
    B = b.B
    ld = (V + 63) // 64 * 64
    logits = b.normal((N, ld), 1.0)
    targets = B.upload(b.rng.integers(0, V, N).astype(np.int32), "i32")
    loss = B._new((), "f32")

    def fn():
        check(B.lib.alpha_softmax_ce_fwd_bwd(logits.ptr, targets.ptr, logits.ptr, loss.ptr, N, V, ld, 1.0, L.BF16))
    return {"ms": b.time(fn), "work": 2.0 * N * V * 2, "kind": "byte"}


def layernorm_case(b: Bench, rows=16384, dim=768, backward=False):
    B = b.B
    x, g = b.normal((rows, dim), 1.0), b.normal((rows, dim), 1.0)
    w, bias = B.ones((dim,)), B.zeros((dim,))
    if not backward:
        return {"ms": b.time(lambda: B.layerNorm(x, w, bias, 1e-5)), "work": 2.0 * rows * dim * 2, "kind": "byte"}
    return {"ms": b.time(lambda: B.layerNormBackward(x, w, g, 1e-5)), "work": 3.0 * rows * dim * 2, "kind": "byte"}


def rmsnorm_case(b: Bench, rows=16384, dim=1024, backward=False):
    B = b.B
    x, g = b.normal((rows, dim), 1.0), b.normal((rows, dim), 1.0)
    w = B.ones((dim,))
    if not backward:
        return {"ms": b.time(lambda: B.rmsNorm(x, w, 1e-5)), "work": 2.0 * rows * dim * 2, "kind": "byte"}
    return {"ms": b.time(lambda: B.rmsNormBackward(x, w, g, 1e-5)), "work": 3.0 * rows * dim * 2, "kind": "byte"}


def swiglu_case(b: Bench, rows=16384, F=2816, backward=False):
    B = b.B
    gate, up, g = (b.normal((rows, F), 1.0) for _ in range(3))
    if not backward:
        return {"ms": b.time(lambda: B.siluMul(gate, up)), "work": 3.0 * rows * F * 2, "kind": "byte"}
    return {"ms": b.time(lambda: B.siluMulBackward(gate, up, g)), "work": 5.0 * rows * F * 2, "kind": "byte"}


def rope_case(b: Bench, Bn=8, T=2048, H=16, D=64):
    """Rotation of the q and k column blocks of a fused [B*T, 3E] activation, in place (what the
    train step does; v is not touched)."""
    B = b.B
    E = H * D
    qkv = b.normal((Bn * T, 3 * E), 1.0)
    return {"ms": b.time(lambda: B.rope(qkv, Bn, T, 2 * H, D, 3 * E)), "work": 2.0 * Bn * T * 2 * E * 2, "kind": "byte"}


def adamw_case(b: Bench, n=124_000_000):
    B = b.B
    p, m, v = B.zeros((n,)), B.zeros((n,)), B.zeros((n,))
    g = B.zeros((n,))
    sh = B.zeros((n,), "bf16")
    fn = lambda: B.adamwStepMulti([(p, g, m, v, 0.1, sh)], 3e-4, 0.9, 0.95, 1e-8, 0.1, 0.05, 1.0)
    return {"ms": b.time(fn), "work": 30.0 * n, "kind": "byte"}


def embedding_bwd_case(b: Bench, N=16384, V=50257, E=768):
    B = b.B
    p = 1.0 / np.power(np.arange(1, V + 1, dtype=np.float64), 1.1)
    cdf = np.cumsum(p / p.sum())
    idx = B.upload(np.minimum(np.searchsorted(cdf, b.rng.random(N)), V - 1).astype(np.int32), "i32")
    g = b.normal((N, E), 1.0)
    return {"ms": b.time(lambda: B.embeddingBackward(idx, g, V, out=None)), "work": N * E * 2.0 + V * E * 4.0,
            "kind": "byte"}


M = 16384
CASES = {
    "gemm_fwd_qkv": lambda b: gemm_case(b, "nt", M, 2304, 768),
    "gemm_fwd_fc1": lambda b: gemm_case(b, "nt", M, 3072, 768),
    "gemm_fwd_fc1_gelu": lambda b: gemm_case(b, "nt", M, 3072, 768, epilogue=L.EPI_GELU),
    "gemm_fwd_fc2": lambda b: gemm_case(b, "nt", M, 768, 3072),
    "gemm_fwd_head": lambda b: gemm_case(b, "nt", M, 50257, 768),
    "gemm_dx_qkv": lambda b: gemm_case(b, "nn", M, 768, 2304),
    "gemm_dx_fc1": lambda b: gemm_case(b, "nn", M, 768, 3072),
    "gemm_dx_fc2": lambda b: gemm_case(b, "nn", M, 3072, 768),
    "gemm_dx_head": lambda b: gemm_case(b, "nn", M, 768, 50257),
    "gemm_dw_qkv": lambda b: gemm_case(b, "tn", 2304, 768, M, "f32"),
    "gemm_dw_fc1": lambda b: gemm_case(b, "tn", 3072, 768, M, "f32"),
    "gemm_dw_fc2": lambda b: gemm_case(b, "tn", 768, 3072, M, "f32"),
    "gemm_dw_head": lambda b: gemm_case(b, "tn", 50257, 768, M, "f32"),
    "gemm_dw_fc1_fc2_pair": lambda b: dw_pair_case(b, (3072, 768), (768, 3072), M),
    "attn_fwd": lambda b: attn_case(b),
    "attn_bwd": lambda b: attn_case(b, backward=True),
    "attn_fwd_b8": lambda b: attn_case(b, Bn=8),
    "attn_bwd_b8": lambda b: attn_case(b, Bn=8, backward=True),
    "attn_fwd_nocap_b8": lambda b: attn_case(b, Bn=8, cap=0.0),
    "attn_bwd_nocap_b8": lambda b: attn_case(b, Bn=8, backward=True, cap=0.0),
    "softmax_ce": lambda b: ce_case(b),
    "layernorm_fwd": lambda b: layernorm_case(b),
    "layernorm_bwd": lambda b: layernorm_case(b, backward=True),
    "rmsnorm_fwd_1024": lambda b: rmsnorm_case(b),
    "rmsnorm_bwd_1024": lambda b: rmsnorm_case(b, backward=True),
    "swiglu_fwd": lambda b: swiglu_case(b),
    "swiglu_bwd": lambda b: swiglu_case(b, backward=True),
    "rope_qk": lambda b: rope_case(b),
    "gemm_fwd_gate_350m": lambda b: gemm_case(b, "nt", M, 2816, 1024),
    "gemm_dx_gate_350m": lambda b: gemm_case(b, "nn", M, 1024, 2816),
    "gemm_dw_gate_350m": lambda b: gemm_case(b, "tn", 2816, 1024, M, "f32"),
    "adamw": lambda b: adamw_case(b),
    "embedding_bwd": lambda b: embedding_bwd_case(b),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", action="append", choices=sorted(CASES), help="default: all")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--cublas", action="store_true", help="time torch.matmul beside every plain GEMM row")
    ap.add_argument("--flush", choices=["write", "read"], default="write",
                    help="how L2 is emptied before each launch: by writing (dirty lines, default) or reading (clean lines) 256 MiB")
    args = ap.parse_args()
    tf_peak, gb_peak, src = _peaks()
    b = Bench(args.iters, args.cublas, args.flush)
    rows = []
    for name in (args.op or list(CASES)):
        r = CASES[name](b)
        if r["kind"] == "flop":
            ach = r["work"] / (r["ms"] * 1e-3) / 1e12
            rows.append({"op": name, "ms": r["ms"], "achieved": ach, "unit": "TFLOP/s", "frac": ach / tf_peak})
            if "cublas_ms" in r:
                rows[-1]["cublas_ms"] = r["cublas_ms"]
                rows[-1]["cublas_tflops"] = r["work"] / (r["cublas_ms"] * 1e-3) / 1e12
        else:
            ach = r["work"] / (r["ms"] * 1e-3) / 1e9
            rows.append({"op": name, "ms": r["ms"], "achieved": ach, "unit": "GB/s", "frac": ach / gb_peak})
    if args.json:
        print(json.dumps({"peaks": src, "rows": rows}))
    else:
        print(f"# peaks: {src} (bf16 {tf_peak} TFLOP/s burst, HBM {gb_peak} GB/s)")
        for r in rows:
            extra = ""
            if "cublas_ms" in r:
                extra = f"   | cuBLAS {r['cublas_ms']:8.4f} ms {r['cublas_tflops']:8.1f} TFLOP/s  (ours/cuBLAS {r['achieved'] / r['cublas_tflops']:.2f})"
            print(f"{r['op']:20s} {r['ms']:9.4f} ms  {r['achieved']:9.1f} {r['unit']:8s} {100 * r['frac']:5.1f}% of peak{extra}")


if __name__ == "__main__":
    main()
