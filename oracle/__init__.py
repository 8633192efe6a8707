"""CPU oracle for the alpha GPT train step.  TEST INFRASTRUCTURE ONLY.

This package restates, in numpy plus a little C, the reference's own CPU path for one
training step: ``packages/tensor/src/cpu_ref.ts`` (op numerics), ``packages/autograd/src``
(tape and backward formulas), ``packages/model/src/gpt.ts`` (init order and forward graph),
``packages/train/src/optimizers.ts`` (AdamW) and the step body of
``packages/train/src/trainer.ts``.  It is the checker that the CUDA library is compared
with; nothing in the product package imports it, and it never runs on the product path.

Parity status: the op-level numerics are pinned against every known-answer test the
reference holds for this path (``packages/tests/src/{tensor,autograd,optimizer}.test.ts``,
see ``tests/test_oracle_golden.py``).  Step-level parity (loss trajectory, parameters after
N steps, the RNG stream) is *unpinned*: the reference's tests hold no such literal values
and no JavaScript runtime exists here to produce them, so it rests on this restatement
following the cited lines.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
_BUILD = os.path.join(_HERE, "_build")
_SO = os.path.join(_BUILD, "liboracle.so")
_lock = threading.Lock()
_lib = None


def build(force: bool = False) -> str:
    """Compile oracle/rng.c into oracle/_build/liboracle.so with gcc."""
    src = os.path.join(_HERE, "rng.c")
    with _lock:
        if (not force and os.path.exists(_SO)
                and os.path.getmtime(_SO) >= os.path.getmtime(src)):
            return _SO
        os.makedirs(_BUILD, exist_ok=True)
        tmp = _SO + ".tmp.%d" % os.getpid()
        subprocess.check_call(["gcc", "-O2", "-fPIC", "-shared", "-ffp-contract=off",
                               "-o", tmp, src, "-lm"])
        os.replace(tmp, _SO)
    return _SO


class _Rng(ctypes.Structure):
    _fields_ = [("s0", ctypes.c_uint32), ("s1", ctypes.c_uint32),
                ("has_spare", ctypes.c_int32), ("spare", ctypes.c_double)]


def lib():
    global _lib
    if _lib is None:
        L = ctypes.CDLL(build())
        P = ctypes.POINTER(_Rng)
        L.alpha_rng_seed.argtypes = [P, ctypes.c_uint32]
        L.alpha_rng_next.argtypes = [P]
        L.alpha_rng_next.restype = ctypes.c_double
        L.alpha_rng_gauss.argtypes = [P]
        L.alpha_rng_gauss.restype = ctypes.c_double
        L.alpha_rng_fill_gauss_f32.argtypes = [P, ctypes.c_void_p, ctypes.c_int64, ctypes.c_double]
        L.alpha_rng_fill_uniform_i32.argtypes = [P, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32]
        d = ctypes.c_double
        L.alpha_oracle_adamw_f32.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64] + [d] * 8
        L.alpha_oracle_embedding_bwd_f32.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int64] * 2
        L.alpha_oracle_matmul_f32.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int64] * 3
        L.alpha_oracle_layernorm_bwd_f32.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int64] * 2 + [d]
        _lib = L
    return _lib
