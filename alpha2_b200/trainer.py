"""Train step — host-side mirror of the step body of ``packages/train/src/trainer.ts``.

Per optimizer step (trainer.ts:1146-1784): learning-rate schedule (:1088-1096,
:1150-1158); micro-step loop = forward, backward, tape clear (:1188-1273), the loss kept on
the device when accumulating (:1210-1226); gradient norm from one ``totalSumOfSquares``
(:1346-1350); clip folded into the optimizer's ``gradScale`` with the gradients left
untouched (:1297, :1650-1656); ``optimizer.stepParamEntries`` (:1761-1762); zero-grad by
dropping the buffers (:1776-1780).

Two ways to finish a step:
* ``fused=False`` — the reference's order of host reads: loss, then the squared norm, then
  the clip coefficient on the host and one ``adamwStep`` per tensor.
* ``fused=True``  — nothing is read back inside the step: the squared norm stays on the
  device, one multi-tensor AdamW launch derives the clip coefficient from it, and the
  loss / norm scalars are returned as device tensors that the caller may read later.

Data parallel (no reference counterpart): with a ``DataParallel`` object every rank runs
the same step on its own batch; gradients are summed across ranks as they become final
during backward, 1/world is folded into ``gradScale`` next to 1/accum.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

from .autograd import Param, Tape
from .backend import CudaBackend, TensorData
from .gpt import ModelConfig, collectParamEntries, gptForward, initGPT
from .optimizers import AdamW
from .rng import SeededRng


@dataclass
class TrainConfig:
    """packages/core/src/types.ts:66-142 (fields the step uses) with the reference defaults."""
    iters: int = 1000
    batchSize: int = 64
    lr: float = 3e-4
    lrMin: float = 0.0
    warmupIters: int = 0
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weightDecay: float = 0.1
    gradClip: float = 1.0
    seed: int = 42
    gradAccumSteps: int = 1


def noDecayNames(cfg: ModelConfig) -> set:
    """apps/cli/src/commands/train.ts:320-331 (``lmHead`` is decayed: the set names the
    non-existent ``lmHead.weight``)."""
    s = {"wte", "wpe", "lnF.weight", "lnF.bias", "lmHead.weight"}
    for i in range(cfg.nLayer):
        for ln in ("ln1", "ln2"):
            s.add(f"layer.{i}.{ln}.weight")
            s.add(f"layer.{i}.{ln}.bias")
    return s


def learningRate(tc: TrainConfig, step: int) -> float:
    """trainer.ts:1088-1096,1150-1158; ``step`` is 0-based."""
    total = tc.iters
    warmup = tc.warmupIters if tc.warmupIters > 0 else (0 if tc.warmupIters < 0 else min(2000, total // 5))
    lr_min = tc.lr / 10 if (tc.lrMin or 0) == 0 else tc.lrMin
    denom = max(1, total - warmup)
    if step < warmup:
        base = lr_min + (tc.lr - lr_min) * (step + 1) / warmup
    else:
        decay = (step - warmup) / denom
        base = lr_min + (tc.lr - lr_min) * 0.5 * (1 + math.cos(math.pi * decay))
    return max(lr_min * 0.1, base)


class CollectiveError(RuntimeError):
    """The gradient exchange failed (NCCL reported an asynchronous error) or did not finish
    within the host's deadline.  The communicator has been aborted; the step is void."""


class PeerLeftError(RuntimeError):
    """Another rank announced that it has left the job; raised before anything is launched."""


class DataParallel:
    """One rank of a data-parallel job: NCCL communicator inside the library, gradients
    all-reduced on its side stream as soon as backward has finalised them.

    Failure handling, all on the host (the reference is single-device and has none):
    * ``store`` — any key-value store shared by the ranks with ``set(key, value)`` and
      ``check([keys]) -> bool`` (``torch.distributed.TCPStore`` fits).  A rank that stops
      between steps calls ``leave()``; the others see it in ``assert_peers()``, which the
      trainer calls at the top of every step, before any kernel or collective of that step is
      enqueued, and raise ``PeerLeftError`` instead of entering a collective that would wait for
      ever.
    * ``sync(timeout_s)`` — waits on the host for the collectives enqueued so far, polling the
      device and NCCL's asynchronous error state; on an error or when the deadline passes it
      aborts the communicator (``ncclCommAbort`` releases collectives stuck on a missing peer)
      and raises ``CollectiveError``.  ``wait()`` stays the cheap stream-order form used inside
      the step.
    """

    def __init__(self, backend: CudaBackend, world: int, rank: int, unique_id: bytes, store=None,
                 wire: str = "f32"):
        import ctypes as C
        from ._lib import check
        if wire not in ("f32", "bf16"):
            raise ValueError("wire must be 'f32' or 'bf16'")
        self.backend, self.world, self.rank, self.store = backend, world, rank, store
        #: element type on the wire.  "f32": the fp32 gradient buffers themselves are reduced, so
        #: data-parallel and single-GPU runs differ only in the order of one fp32 sum per element.
        #: "bf16": every fp32 gradient is rounded to bf16 into a side buffer, the side buffers
        #: are reduced (half the bytes over NVLink, bf16 sums across ranks) and converted back
        #: before the norm — two extra passes over the gradients and 8 bits less of them.
        self.wire = wire
        buf = C.create_string_buffer(unique_id, 128)
        check(backend.lib.alpha_comm_init_rank(world, rank, buf))

    @staticmethod
    def new_unique_id() -> bytes:
        import ctypes as C
        from . import _lib as L
        from ._lib import check
        buf = C.create_string_buffer(128)
        check(L.load().alpha_comm_unique_id(buf))
        return buf.raw

    #: gradients are handed to NCCL in groups of about this many bytes (one collective launch each)
    bucket_bytes = 32 << 20
    #: False turns every exchange into a no-op (each rank then trains on its own gradients):
    #: a measuring aid for "how much of the exchange is hidden behind backward", nothing else
    enabled = True

    def allreduce(self, grad: TensorData) -> None:
        from ._lib import check
        if not self.enabled:
            return
        check(self.backend.lib.alpha_comm_allreduce_sum(grad.ptr, grad.size, self.backend._code(grad.dtype)))

    def allreduce_bucket(self, grads: list) -> None:
        """Sum-allreduce several gradient tensors of one dtype as a single NCCL group."""
        import ctypes as C
        from ._lib import check
        if not grads or not self.enabled:
            return
        n = len(grads)
        ptrs = (C.c_uint64 * n)(*[g.ptr for g in grads])
        counts = (C.c_int64 * n)(*[g.size for g in grads])
        check(self.backend.lib.alpha_comm_allreduce_sum_bucket(ptrs, counts, n, self.backend._code(grads[0].dtype)))

    def wait(self) -> None:
        from ._lib import check
        if self.enabled:
            check(self.backend.lib.alpha_comm_wait())

    # ── failure handling ──────────────────────────────────────────────────────
    def leave(self) -> None:
        """Announce that this rank will enqueue no further collectives (call between steps)."""
        if self.store is not None:
            self.store.set(f"alpha_dp/left/{self.rank}", b"1")

    def peers_gone(self) -> list:
        if self.store is None:
            return []
        return [r for r in range(self.world) if r != self.rank and self.store.check([f"alpha_dp/left/{r}"])]

    def assert_peers(self) -> None:
        gone = self.peers_gone()
        if gone:
            raise PeerLeftError(f"rank {self.rank}: rank(s) {gone} left the job; not entering the next exchange")

    def sync(self, timeout_s: float = 30.0, poll_s: float = 0.0005) -> None:
        """Wait on the host until every collective enqueued so far has completed."""
        import ctypes as C
        import time
        from ._lib import check
        lib = self.backend.lib
        pending, err = C.c_int(0), C.c_int(0)
        deadline = time.monotonic() + float(timeout_s)
        while True:
            check(lib.alpha_comm_query(C.byref(pending), C.byref(err)))
            if err.value != 0:
                lib.alpha_comm_abort()
                raise CollectiveError(f"rank {self.rank}: NCCL reported asynchronous error {err.value}; "
                                      "communicator aborted")
            if not pending.value:
                return
            if time.monotonic() > deadline:
                lib.alpha_comm_abort()
                raise CollectiveError(f"rank {self.rank}: gradient exchange did not finish within {timeout_s} s; "
                                      "communicator aborted")
            time.sleep(poll_s)


class Trainer:
    def __init__(self, backend: CudaBackend, modelConfig: ModelConfig, trainConfig: TrainConfig,
                 params=None, attention: str = "fused", fused: bool = True, dp: DataParallel | None = None,
                 release: bool = True, activationCheckpointing: bool = False):
        self.B, self.mc, self.tc = backend, modelConfig, trainConfig
        if params is None:
            rng = SeededRng(trainConfig.seed)
            params = initGPT(modelConfig, backend, rng)
        self.params = params
        self.entries = collectParamEntries(params)
        self.opt = AdamW(backend, lr=trainConfig.lr, beta1=trainConfig.beta1, beta2=trainConfig.beta2,
                         eps=trainConfig.eps, weightDecay=trainConfig.weightDecay,
                         noDecayNames=noDecayNames(modelConfig))
        self.tape = Tape()
        self.attention, self.fused, self.dp = attention, fused, dp
        self.activationCheckpointing = activationCheckpointing      # trainer.ts:559,1203
        self.step_index = 0
        self._wire_pairs: list = []
        self.releaseFn = backend.releaseGpuTensor if release else None

    # ── one optimizer step ────────────────────────────────────────────────────
    def train_step(self, batches, read_back: bool = True) -> dict:
        """batches: one (tokens, targets) pair of int32 [B, T] TensorData per micro-step.
        Returns loss / gradNorm / lr / clipCoef — floats when ``read_back``, else the loss
        and squared-norm device tensors under "lossTensor" / "sumSqTensor"."""
        B, tc = self.B, self.tc
        accum = len(batches)
        world = self.dp.world if self.dp else 1
        if self.dp is not None and hasattr(self.dp, "assert_peers"):
            self.dp.assert_peers()                             # before anything of this step is enqueued
        lr = learningRate(tc, self.step_index)
        self.opt.setLr(lr)
        B.resetStepOps()
        loss_acc = None
        loss_td = None
        mark = getattr(B, "rangePush", None)        # phase ranges for timeline tools (trainer.ts:1189-1264 times the same phases)
        unmark = getattr(B, "rangePop", None)
        for mi, (tokens, targets) in enumerate(batches):
            if mark:
                mark("forward")
            out = gptForward(self.mc, self.params, B, self.tape, tokens, targets, training=True,
                             attention=self.attention, release=self.releaseFn,
                             activationCheckpointing=self.activationCheckpointing)
            if mark:
                unmark()
            loss = out["loss"]
            if accum > 1:                                      # trainer.ts:1210-1226
                scaled = B.scale(loss.data, 1 / accum)
                if loss_acc is None:
                    loss_acc = scaled
                else:
                    B.addInplace(loss_acc, scaled)
            else:
                loss_td = B.clone(loss.data) if self.releaseFn else loss.data
            last = mi == accum - 1
            if mark:
                mark("backward")
            self._backward(loss, allreduce=last and self.dp is not None)
            self.tape.clear(self.releaseFn)
            if mark:
                unmark()
        if accum > 1:
            loss_td = loss_acc
        if self.dp is not None:
            self.dp.wait()
            for g, w in self._wire_pairs:                      # bf16 wire: the reduced copies back into the gradients
                B.castInto(w, g)
                if self.releaseFn is not None:
                    self.releaseFn(w)
            self._wire_pairs.clear()

        if mark:
            mark("optimizer")
        grad_scale = 1.0 / (accum * world)
        grads = [v.grad for _, v in self.entries if v.grad is not None]
        sumsq = B.totalSumOfSquares(grads)
        result = {"lr": lr}
        if self.fused:
            self.opt.stepParamEntries(self.entries, grad_scale, fused=True,
                                      clipSumSq=sumsq if tc.gradClip > 0 else None, maxNorm=tc.gradClip)
            if read_back:
                gnorm = math.sqrt(float(sumsq.item())) * abs(grad_scale)
                if not math.isfinite(gnorm):               # the kernel left p, m, v untouched
                    self.opt.undoStep()
                    result["skipped"] = True
                result.update(loss=loss_td.item(), gradNorm=gnorm,
                              clipCoef=(tc.gradClip / gnorm if tc.gradClip > 0 and gnorm > tc.gradClip else 1.0))
            else:
                result.update(lossTensor=loss_td, sumSqTensor=sumsq)
        else:
            loss_val = loss_td.item()                          # trainer.ts:1247
            gnorm = math.sqrt(float(sumsq.item())) * abs(grad_scale)   # :1348-1349
            clip, eff = 1.0, grad_scale
            if tc.gradClip > 0 and gnorm > tc.gradClip:       # :1650-1656
                clip = tc.gradClip / gnorm
                eff *= clip
            if math.isfinite(loss_val) and math.isfinite(gnorm):
                self.opt.stepParamEntries(self.entries, eff)
            result.update(loss=loss_val, gradNorm=gnorm, clipCoef=clip)
        if mark:
            unmark()
        if read_back and hasattr(B, "checkAsyncError"):
            # The host has just waited for the step's scalars, so asking the library whether a
            # tensor-core kernel gave up a bounded wait costs one 4-byte read.  Such a step
            # produced garbage; the error must not pass silently into the next one.
            B.checkAsyncError()
        for _, v in self.entries:                              # trainer.ts:1776-1780
            v.grad = None
        self.step_index += 1
        result["gpuOps"] = B.gpuOpsThisStep
        return result

    def _backward(self, loss, allreduce: bool) -> None:
        if not allreduce:
            self.tape.backward(loss, self.B, self.releaseFn)
            return
        # Count how many tape entries feed each parameter: its gradient is final once the
        # last of them has run, and can be handed to the collective while backward goes on.
        pending: dict[int, int] = {}
        by_id: dict[int, Param] = {}
        for e in self.tape.entries:
            for v in e.inputs:
                if isinstance(v, Param):
                    pending[v.id] = pending.get(v.id, 0) + 1
                    by_id[v.id] = v
        dp = self.dp
        # Finished gradients collect in a bucket (in the order backward finalises them: head and
        # last layers first); a full bucket goes to the collective as one group while backward
        # continues.  A communicator without bucket support gets them one by one.
        bucketed = hasattr(dp, "allreduce_bucket")
        limit = getattr(dp, "bucket_bytes", 32 << 20)
        bucket: list = []
        fill = [0]
        bf16_wire = getattr(dp, "wire", "f32") == "bf16"
        B = self.B

        def on_wire(g):
            """The tensor that goes to the collective for gradient g."""
            if bf16_wire and g.dtype == "f32":
                t = B.castDtype(g, "bf16")
                self._wire_pairs.append((g, t))
                return t
            return g

        def flush():
            if bucket:
                by_dtype: dict = {}
                for g in bucket:
                    by_dtype.setdefault(g.dtype, []).append(g)
                for gs in by_dtype.values():
                    dp.allreduce_bucket(gs)
                bucket.clear()
                fill[0] = 0

        def on_entry_done(entry):
            for v in entry.inputs:
                if isinstance(v, Param) and v.id in pending:
                    pending[v.id] -= 1
                    if pending[v.id] == 0 and v.grad is not None:
                        w = on_wire(v.grad)
                        if bucketed:
                            bucket.append(w)
                            fill[0] += w.size * (2 if w.dtype == "bf16" else 4)
                            if fill[0] >= limit:
                                flush()
                        else:
                            dp.allreduce(w)
                        del pending[v.id]
        self.tape.backward(loss, self.B, self.releaseFn, onEntryDone=on_entry_done)
        flush()

    # ── state exchange with the host (checkpointing needs exactly this) ───────
    def host_params(self) -> dict:
        return {n: np.array(v.data.data, dtype=np.float32) for n, v in self.entries}

    def load_param(self, name: str, host: np.ndarray) -> None:
        """Replace one parameter's fp32 master by host values (and rebuild its bf16 compute copy)."""
        v = dict(self.entries)[name]
        old, old_shadow = v.data, getattr(v, "shadow", None)
        v.data = self.B.upload(np.ascontiguousarray(host, dtype=np.float32).reshape(old.shape), "f32")
        if old_shadow is not None:
            v.shadow = self.B.castDtype(v.data, old_shadow.dtype)
        if self.releaseFn is not None:
            self.releaseFn(old)
            if old_shadow is not None:
                self.releaseFn(old_shadow)
