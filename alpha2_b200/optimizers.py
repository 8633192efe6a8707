"""AdamW — host-side mirror of ``packages/train/src/optimizers.ts:21-234``.

Same update rule (:84-92), bias corrections from running beta powers (:107-115), per-name
weight-decay switch (``noDecayNames``), lazily created moment buffers that live on the
device (:166-199), ``stateDict`` / ``loadStateDict`` (:201-229).  ``stepParamEntries``
(:54-94) calls ``backend.adamwStep`` per tensor like the reference, or — ``fused=True`` —
hands every tensor to one multi-tensor launch and lets the kernel derive the clip
coefficient from the device-resident sum of squared gradients.
"""
from __future__ import annotations

import numpy as np

from .backend import CudaBackend, TensorData


class AdamW:
    name = "adamw"

    def __init__(self, backend: CudaBackend, lr: float = 3e-4, beta1: float = 0.9, beta2: float = 0.999,
                 eps: float = 1e-8, weightDecay: float = 0.01, noDecayNames: set | None = None):
        self.backend = backend
        self.lr, self.beta1, self.beta2, self.eps, self.weightDecay = lr, beta1, beta2, eps, weightDecay
        self.noDecayNames = noDecayNames or set()
        self._step = 0
        self._beta1Pow = 1.0
        self._beta2Pow = 1.0
        self._prev = None
        self._m: dict[str, TensorData] = {}
        self._v: dict[str, TensorData] = {}

    def setLr(self, lr: float) -> None:
        self.lr = lr

    def _next_bias_corrections(self):
        self._prev = (self._step, self._beta1Pow, self._beta2Pow)
        self._step += 1
        self._beta1Pow *= self.beta1
        self._beta2Pow *= self.beta2
        return 1 - self._beta1Pow, 1 - self._beta2Pow

    def undoStep(self) -> None:
        """Take back the last advance of the step count and the running beta powers.  The fused
        update skips itself on the device when the gradient norm is not finite; a host that
        learns of that afterwards (it reads the norm with the loss) calls this so that the
        bias corrections continue as if the optimizer had not been called — which is what the
        reference does for such a step (trainer.ts:1495-1527,1750)."""
        if self._prev is not None:
            self._step, self._beta1Pow, self._beta2Pow = self._prev
            self._prev = None

    def _moments(self, name: str, param: TensorData):
        if name not in self._m:
            self._m[name] = self.backend.zeros(param.shape, "f32")
            self._v[name] = self.backend.zeros(param.shape, "f32")
        return self._m[name], self._v[name]

    def stepParamEntries(self, entries, gradScale: float = 1.0, fused: bool = False,
                         clipSumSq: TensorData | None = None, maxNorm: float = 0.0) -> None:
        """entries: iterable of (name, Variable-like with .data/.grad[/.shadow])."""
        bc1, bc2 = self._next_bias_corrections()
        B = self.backend
        if fused:
            batch = []
            for name, var in entries:
                if var.grad is None:
                    continue
                m, v = self._moments(name, var.data)
                wd = 0.0 if name in self.noDecayNames else self.weightDecay
                batch.append((var.data, var.grad, m, v, wd, getattr(var, "shadow", None)))
            if batch:
                B.adamwStepMulti(batch, self.lr, self.beta1, self.beta2, self.eps, bc1, bc2, gradScale,
                                 clipSumSq, maxNorm)
            return
        for name, var in entries:
            if var.grad is None:
                continue
            m, v = self._moments(name, var.data)
            wd = 0.0 if name in self.noDecayNames else self.weightDecay
            B.adamwStep(var.data, var.grad, m, v, self.lr, self.beta1, self.beta2, self.eps, wd, bc1, bc2,
                        gradScale, getattr(var, "shadow", None))

    def step(self, params: dict, grads: dict, gradScale: float = 1.0) -> None:
        """optimizers.ts:96-105: name -> TensorData maps."""
        bc1, bc2 = self._next_bias_corrections()
        for name, p in params.items():
            g = grads.get(name)
            if g is None:
                continue
            m, v = self._moments(name, p)
            wd = 0.0 if name in self.noDecayNames else self.weightDecay
            self.backend.adamwStep(p, g, m, v, self.lr, self.beta1, self.beta2, self.eps, wd, bc1, bc2, gradScale)

    def stateDict(self) -> dict:
        buffers = {}
        for name, m in self._m.items():
            buffers[f"{name}.m"] = np.array(m.data, dtype=np.float32).reshape(-1)
            buffers[f"{name}.v"] = np.array(self._v[name].data, dtype=np.float32).reshape(-1)
        return {"step": self._step, "buffers": buffers}

    def loadStateDict(self, state: dict, shapes: dict | None = None) -> None:
        self._step = int(state["step"])
        self._beta1Pow = self.beta1 ** self._step
        self._beta2Pow = self.beta2 ** self._step
        self._m.clear()
        self._v.clear()
        for key, arr in state["buffers"].items():
            name, kind = key[:-2], key[-1]
            a = np.asarray(arr, dtype=np.float32)
            if shapes and name in shapes:
                a = a.reshape(shapes[name])
            (self._m if kind == "m" else self._v)[name] = self.backend.upload(a, "f32")
