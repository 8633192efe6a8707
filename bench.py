"""Train-step benchmark: tokens/s of the GPT train step at the GPT-2-124M shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" = one optimizer step of the hot path (forward, loss, backward, gradient norm /
clip, AdamW) over one batch of synthetic tokens (Zipf s=1.1 over the vocabulary, seeded;
random-init weights of the named shape).  Under torchrun (N > 1) every rank runs the step on
its own micro-batch and gradients are all-reduced with NCCL (weak scaling); rank 0 prints
one JSON line.

Keys: ``value`` — whole-job tokens/s with every step's tokens already resident in HBM,
device-timed with CUDA events on the library's stream, max over ranks; ``e2e`` — the same
steps driven through the public API with host buffers: per step the product's DataLoader
draws the batch on the host into page-locked memory, tokens and targets are copied to the
device and the loss is read back; ``comm`` (N > 1) — step time with and without the gradient
exchange, i.e. how much of it is exposed; ``roofline`` — the dominant
kernel family (tensor-core GEMM) timed with events around its launches in a third pass over
the same steps (events between kernels would stop the launch overlap of the two timed regions,
which run first, back to back); ``cpu_baseline``
— the CPU oracle (a port of the reference's cpu_ref path) timed on the host cores on a
bounded sample; ``clocks`` — nvidia-smi samples taken during the timed regions.

``--impl reference`` times the CPU oracle alone on the same configuration (rank 0 only).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # GPT-2-small shape (124M), micro-batch 16 per GPU — the shape the headline metric is quoted on
    "gpt2-124m": dict(model=dict(vocabSize=50257, blockSize=1024, nLayer=12, nEmbd=768, nHead=12, tied=True,
                                 init="plain"), micro_batch=16, dtype="bf16"),
    # small GPT: vocab 4096, 6 layers, width 384, context 256, batch 32
    "small-gpt": dict(model=dict(vocabSize=4096, blockSize=256, nLayer=6, nEmbd=384, nHead=6, tied=True,
                                 init="plain"), micro_batch=32, dtype="bf16"),
    # GPT 350M shape: RMSNorm, SwiGLU, RoPE, untied head, 4 accumulated micro-batches of 8 per step
    "gpt-350m": dict(model=dict(vocabSize=32768, blockSize=2048, nLayer=24, nEmbd=1024, nHead=16, tied=False,
                                ffnActivation="swiglu", ffnDim=2816, norm="rms", rope=True, init="plain"),
                     micro_batch=8, accum=4, dtype="bf16"),
    # a seconds-long case for checking the script itself
    "tiny": dict(model=dict(vocabSize=256, blockSize=64, nLayer=2, nEmbd=64, nHead=4), micro_batch=4, dtype="bf16"),
}


def flops_per_token(m: dict) -> float:
    """6*P_mm + 12*L*E*T with P_mm = L*(4E^2 + 2EF) + V*E (3EF for SwiGLU; model FLOPs, no causal
    discount)."""
    E, L, V, T = m["nEmbd"], m["nLayer"], m["vocabSize"], m["blockSize"]
    swiglu = m.get("ffnActivation") == "swiglu"
    F = m.get("ffnDim") or (4 * E)
    return 6.0 * (L * (4 * E * E + (3 if swiglu else 2) * E * F) + V * E) + 12.0 * L * E * T


def measured_peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [x.strip() for x in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
                except ValueError:
                    continue
                for n, v in zip(names, parts[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        # samples under load only (idle samples before/after the region would drag the median)
        busy = [c for c, p in zip(sm, power) if p > 0.5 * max(power)] if power else sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def oracle_step_rate(model: dict, sample_T: int, steps: int, warmup: int) -> dict:
    """Tokens/s of the CPU oracle on one sequence of ``sample_T`` tokens per step."""
    from oracle import gpt as ogpt
    from oracle import train as otrain
    m = dict(model)
    mc = ogpt.ModelConfig(**m)
    tr = otrain.Trainer(mc, otrain.TrainConfig(iters=1000, batchSize=1, seed=42))
    batches = otrain.zipf_batches(11, steps + warmup, 1, sample_T, m["vocabSize"])
    for i in range(warmup):
        tr.train_step([batches[i]])
    t0 = time.perf_counter()
    for i in range(warmup, warmup + steps):
        tr.train_step([batches[i]])
    dt = time.perf_counter() - t0
    return {"tokens_per_s": steps * sample_T / dt, "seconds": dt, "ms_per_step": 1e3 * dt / steps}


def profiled_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, taken
    from the ncu summary committed under profiles/ (the MLP up-projection forward GEMM,
    16384 x 3072 x 768).  (None, None) when the summary is missing."""
    import re
    name = "gemm_tc_pair_kernel_fc1_fwd_16384x3072x768.md"
    try:
        text = open(os.path.join(ROOT, "profiles", name)).read()
        rd = float(re.search(r"dram__bytes_read\.sum\s*\|\s*([0-9.]+)\s*MB", text).group(1))
        wr = float(re.search(r"dram__bytes_write\.sum\s*\|\s*([0-9.]+)\s*MB", text).group(1))
        return (rd + wr) * 1e6, f"profiles/{name}"
    except Exception:
        return None, None


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def run_reference(args, wl) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    model = wl["model"]
    total = max(1, args.steps + args.warmup)
    # One sequence per step, as long as the in-run cpu_baseline's (256 tokens) when the whole
    # --steps/--warmup run then stays near four minutes: ~18 ms per token per step for the 124M
    # shape on 16 host threads, scaled by the model's FLOPs per token.
    per_tok = 0.018 * flops_per_token(model) / flops_per_token(WORKLOADS["gpt2-124m"]["model"])
    T = min(256, model["blockSize"])
    while T > 32 and total * T * per_tok > 240.0:
        T //= 2
    try:                                         # torchrun exports OMP_NUM_THREADS=1; the CPU arm may use every core
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=host_threads())
    except Exception:
        pass
    r = oracle_step_rate(model, T, args.steps, args.warmup)
    sample = f"1 sequence x {T} tokens per step, full {model['nLayer']}-layer model, fp32 storage / f64 accumulate"
    line = {
        "impl": "reference", "metric": "train tokens/s", "value": r["tokens_per_s"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, **{k: model[k] for k in ("vocabSize", "nLayer", "nEmbd", "nHead", "blockSize")},
                   "parallelism": "cpu"},
        "cpu_baseline": {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": host_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": r["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU oracle: a numpy/C port of the reference's cpu_ref train step (no JavaScript runtime exists "
                "here to run the reference itself); matmuls use multi-threaded BLAS in f64",
    }
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gpt2-124m", choices=sorted(WORKLOADS))
    ap.add_argument("--micro-batch", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--wire", default="f32", choices=["f32", "bf16"], help="element type of the gradient exchange (N > 1)")
    ap.add_argument("--repeats", type=int, default=3, help="timed repetitions of the resident-token region (median reported)")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, wl)
        return
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local))

    from alpha2_b200 import _lib as L
    from alpha2_b200._lib import check
    from alpha2_b200.backend import CudaBackend, TensorData, _DeviceBuffer
    from alpha2_b200.gpt import ModelConfig
    from alpha2_b200.trainer import DataParallel, TrainConfig, Trainer

    B = CudaBackend(local)
    lib = B.lib
    dp = None
    if world > 1:
        ids = [DataParallel.new_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        dp = DataParallel(B, world, rank, ids[0], wire=args.wire)

    model = wl["model"]
    mb = args.micro_batch or wl["micro_batch"]
    T = model["blockSize"]
    mc = ModelConfig(**model, compute_dtype=wl["dtype"])
    accum = int(wl.get("accum", 1))
    tr = Trainer(B, mc, TrainConfig(iters=100000, batchSize=mb, warmupIters=100, seed=42, gradAccumSteps=accum), dp=dp)

    # synthetic tokens: Zipf(1.1) over the vocabulary, a different seeded stream per rank
    from alpha2_b200.data import zipf_batches
    n_batches = (args.steps + args.warmup) * accum
    host_batches = zipf_batches(1000 + rank, n_batches, mb, T, model["vocabSize"])
    tok_bytes = mb * T * 4
    pinned = []
    for tok, tgt in host_batches:
        pair = []
        for arr in (tok, tgt):
            p = C.c_void_p()
            check(lib.alpha_host_alloc(tok_bytes, C.byref(p)))
            C.memmove(p, arr.ctypes.data, tok_bytes)
            pair.append(p)
        pinned.append(pair)

    def device_tokens(step):
        """The ``accum`` micro-batches of one optimizer step, copied from pinned host memory."""
        micro = []
        for i in range(step * accum, (step + 1) * accum):
            out = []
            for p in pinned[i]:
                td = TensorData((mb, T), "i32", _DeviceBuffer(tok_bytes))
                check(lib.alpha_h2d(td.ptr, p, tok_bytes))
                out.append(td)
            micro.append(tuple(out))
        return micro

    def barrier():
        B.syncGpu()
        if dist is not None:
            dist.barrier()
        B.syncGpu()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        import torch
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ev0, ev1 = C.c_uint64(), C.c_uint64()
    check(lib.alpha_event_create(C.byref(ev0)))
    check(lib.alpha_event_create(C.byref(ev1)))

    def timed(fn) -> float:
        barrier()
        check(lib.alpha_event_record(ev0.value))
        fn()
        check(lib.alpha_event_record(ev1.value))
        check(lib.alpha_event_sync(ev1.value))
        ms = C.c_float()
        check(lib.alpha_event_elapsed_ms(ev0.value, ev1.value, C.byref(ms)))
        barrier()
        return max_over_ranks(float(ms.value))

    # ── warm-up (end to end, so pools, tensor maps and NCCL are all primed) ─────────────
    for i in range(args.warmup):
        tr.train_step(device_tokens(i), read_back=True)
    B.checkAsyncError()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()

    # ── region A: tokens resident in HBM, nothing read back inside the region ───────────
    resident = [device_tokens(args.warmup + i) for i in range(args.steps)]
    launches0 = B.launch_count()
    last = {}

    def region_a():
        for i in range(args.steps):
            last["r"] = tr.train_step(resident[i], read_back=False)
    ms_a = timed(region_a)
    launches = B.launch_count() - launches0
    final_loss = last["r"]["lossTensor"].item()

    # more runs of the same region: the figure reported is the median (single regions of a few
    # hundred milliseconds move by a percent or so with the clock)
    runs_a = [ms_a]
    for _ in range(max(0, args.repeats - 1)):
        runs_a.append(timed(region_a))
    ms_a = statistics.median(runs_a)

    # ── region B: end to end through the public API with host buffers ───────────────────
    # Batches come from the product's DataLoader over a synthetic token stream in page-locked
    # memory (two slots, guarded by events): per step it draws the windows on the host, copies
    # tokens and targets to the device asynchronously and the step consumes them.
    from alpha2_b200.data import DataLoader
    from alpha2_b200.rng import SeededRng
    corpus = np.concatenate([t.reshape(-1) for t, _ in host_batches[:64]])
    loader = DataLoader(corpus, SeededRng(7 + rank), mb, T, backend=B, pin=True)

    def loader_tokens():
        return [loader.nextDeviceBatch() for _ in range(accum)]
    losses = []

    def region_b():
        # every step: tokens from pinned host memory, loss copied back to the host.  The copy
        # of step i is enqueued behind step i and collected after step i+1 has been enqueued,
        # so the host never stalls the device (the last one is collected inside the region).
        pending = None
        for i in range(args.steps):
            out = tr.train_step(loader_tokens(), read_back=False)
            nxt = B.readScalarAsync(out["lossTensor"])
            if pending is not None:
                losses.append(pending.get())
            pending = nxt
        losses.append(pending.get())
    region_b_warm = tr.train_step(loader_tokens(), read_back=True)     # first use of the loader's buffers, untimed
    ms_b = timed(region_b)
    loader.close()
    clocks = sampler.stop() if rank == 0 else {}
    # ── region P: the steps of region A once more with per-kernel-family event timing switched
    # on (kept out of regions A and B: an event record between two kernels stops their overlap;
    # run last, after the clock sampling has stopped) ────
    check(lib.alpha_profile_enable(1))
    ms_p = timed(region_a)
    check(lib.alpha_profile_enable(0))
    prof = (L.ProfileEntry * len(L.PROFILE_CATEGORIES))()
    check(lib.alpha_profile_read(prof, len(L.PROFILE_CATEGORIES)))
    # ── region C (multi-GPU only, last: the replicas drift apart in it): the steps of region A
    # with the gradient exchange switched off, so that "step time minus compute-only step time"
    # says how much of the exchange is exposed ──
    ms_c = None
    if dp is not None:
        ms_c_ref = timed(region_a)                 # with the exchange, directly before
        dp.enabled = False
        ms_c = timed(region_a)
        dp.enabled = True

    del resident

    B.checkAsyncError()

    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    tokens_per_step = mb * T * accum * world
    value = tokens_per_step * args.steps / (ms_a / 1e3)
    e2e = tokens_per_step * args.steps / (ms_b / 1e3)
    peaks = measured_peaks()
    fpt = flops_per_token(model)
    gemm = prof[0]
    achieved = (gemm.work / 1e12) / (gemm.ms / 1e3) if gemm.ms > 0 else None
    peak_tf = peaks["bf16_tflops_sustained"]
    profile = {}
    for name, e in zip(L.PROFILE_CATEGORIES, prof):
        if e.launches:
            profile[name] = {"ms_per_step": e.ms / args.steps, "launches_per_step": e.launches / args.steps,
                             "work_per_step": e.work / args.steps}
    traffic, traffic_src = (profiled_traffic() if args.workload == "gpt2-124m" else (None, None))
    line = {
        "metric": "train tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_a / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
        "config": {"workload": args.workload, "shape": {k: model[k] for k in ("vocabSize", "nLayer", "nEmbd", "nHead", "blockSize")},
                   "micro_batch_per_gpu": mb, "grad_accum_steps": accum, "tokens_per_step": tokens_per_step, "tied_embeddings": bool(model.get("tied")),
                   "precision": "bf16 activations and weight shadows, fp32 master weights and AdamW state",
                   "parallelism": f"dp{world}", "gradient_exchange": (f"NCCL all-reduce, {args.wire} on the wire" if world > 1 else "none"), "l2": "inputs larger than L2 (each step streams >10 GB of activations and weights)",
                   "tokens": "Zipf(s=1.1), seeded per rank",
                   "attention": "causal, scores soft-capped at 30*tanh(s/30) as in the reference model (gpt.ts:244)"
                   if model.get("softCap", None) in (None, 30.0) else f"causal, softCap {model.get('softCap')}",
                   "timed_region": f"{args.steps} steps, median of {len(runs_a)} repetitions"},
        "ms_per_step_runs": [m / args.steps for m in runs_a],
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": 2 * tok_bytes * accum, "d2h_bytes_per_step": 4,
                "ms_per_step": ms_b / args.steps},
        "gpu_launches": launches,
        "clocks": clocks,
        "mfu": {"flops_per_token": fpt, "of_burst_peak": value / world * fpt / (peaks["bf16_tflops"] * 1e12),
                "of_sustained_peak": value / world * fpt / (peak_tf * 1e12), "peaks": peaks["source"]},
        "roofline": {"bound": "tensor", "kernel": "gemm_tc_pair_kernel (bf16 tcgen05 GEMM, CTA pairs, all layouts)",
                     "achieved": achieved,
                     "peak": peak_tf, "unit": "TFLOP/s", "frac": (achieved / peak_tf) if achieved else None,
                     # DRAM bytes of one profiled launch, read from the committed ncu summary of that launch
                     "traffic": traffic, "traffic_launch": traffic_src,
                     "peak_source": f"{peaks['source']} cuBLAS bf16, sustained",
                     "launches_per_step": gemm.launches / args.steps, "ms_per_step": gemm.ms / args.steps},
        "profile": profile, "profile_pass_ms_per_step": ms_p / args.steps,
        "comm": ({"compute_only_ms_per_step": ms_c / args.steps,
                  "exposed_ms_per_step": (ms_c_ref - ms_c) / args.steps,
                  "note": "the timed region run once more with the exchange, minus the same steps with the "
                          "gradient exchange switched off directly after it"} if ms_c is not None else None),
        "final_loss": final_loss,
    }
    if world == 1 and not args.no_cpu_baseline:
        sample_T = min(256, T)
        r = oracle_step_rate({k: v for k, v in model.items()}, sample_T, 1, 0)
        line["cpu_baseline"] = {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": host_threads(), "kind": "port",
                                "sample": f"1 step on 1 sequence x {sample_T} tokens, full model, {r['seconds']:.1f} s of CPU work"}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
