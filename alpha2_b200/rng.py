"""SeededRng of the reference (packages/core/src/rng.ts:6-68), implemented by the host-side
generator inside libalpha_cuda.so (alpha_rng_*), so that ``initGPT`` draws the reference's
weights for a given seed."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L


class SeededRng:
    def __init__(self, seed: int = 42):
        self._st = L.HostRng()
        self._lib = L.load()
        self.seed(seed)

    def seed(self, s: int) -> None:
        self._seed = int(s)
        self._lib.alpha_rng_seed(C.byref(self._st), C.c_uint32(self._seed & 0xFFFFFFFF))

    def state(self) -> int:
        return self._seed

    def setState(self, s: int) -> None:
        self.seed(s)

    def next(self) -> float:
        return self._lib.alpha_rng_next(C.byref(self._st))

    def nextGauss(self) -> float:
        return self._lib.alpha_rng_gauss(C.byref(self._st))

    def fill_gauss(self, shape, std: float) -> np.ndarray:
        """``data[i] = float32(nextGauss() * std)`` for every element in order (gpt.ts:53-58)."""
        out = np.empty(shape, dtype=np.float32)
        self._lib.alpha_rng_fill_gauss(C.byref(self._st), out.ctypes.data, out.size, float(std))
        return out
