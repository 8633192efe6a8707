"""CudaBackend: the reference's ``Backend`` interface on top of libalpha_cuda.so.

Mirror of ``packages/core/src/interfaces.ts:38-151`` (same method names, argument meaning
and error behaviour), standing where the reference has ``HeliosBackend``
(``packages/helios/src/backend.ts:1221``).  A TypeScript host would bind the same C ABI with
bun:ffi; this file is that host layer written in Python because no JavaScript runtime
exists on the build or GPU machines.

Tensors: ``TensorData`` keeps ``shape``/``dtype``/``data`` like the reference's plain
objects (interfaces.ts:31-35).  Device residence follows helios: outputs live on the GPU
and ``.data`` reads them back on demand (backend.ts:1143-1171); host-created tensors upload
on first use (:298-313); ``reshape`` shares the buffer (:4528-4538); in-place ops
invalidate the cached host copy (:706-729); ``releaseGpuTensor`` frees explicitly (:688-699)
and garbage collection is the backstop (:629-639).

There is no CPU fallback: every method runs a CUDA kernel through the C ABI, and a missing
library or device raises.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Iterable, Sequence

import numpy as np

from . import _lib as L
from ._lib import AlphaCudaError, check

_NP = {"f32": np.float32, "i32": np.int32}


def _size(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


class _DeviceBuffer:
    """One allocation from the library's caching pool; freed when the last owner lets go."""
    __slots__ = ("ptr", "nbytes", "__weakref__")

    def __init__(self, nbytes: int):
        out = C.c_uint64()
        check(L.load().alpha_alloc(max(int(nbytes), 1), C.byref(out)))
        self.ptr = out.value
        self.nbytes = int(nbytes)

    def free(self):
        if self.ptr:
            lib = L._lib
            if lib is not None:
                lib.alpha_free(self.ptr)
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def bf16_to_f32(raw_u16: np.ndarray) -> np.ndarray:
    return (raw_u16.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even conversion to bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + 0x7FFF + ((u >> 16) & 1)
    nan = np.isnan(x)
    out = (rounded >> 16).astype(np.uint16)
    out[nan] = 0x7FC0
    return out


class TensorData:
    """``{shape, dtype, data}`` (interfaces.ts:31-35) with lazy device residence."""
    __slots__ = ("shape", "dtype", "_buf", "_host", "_released", "__weakref__")

    def __init__(self, shape, dtype: str = "f32", buf: _DeviceBuffer | None = None, host: np.ndarray | None = None):
        self.shape = tuple(int(d) for d in shape)
        self.dtype = dtype
        self._buf = buf
        self._host = host
        self._released = False

    @classmethod
    def from_host(cls, array: np.ndarray, dtype: str | None = None) -> "TensorData":
        if dtype is None:
            dtype = "i32" if np.issubdtype(array.dtype, np.integer) else "f32"
        arr = np.ascontiguousarray(array, dtype=_NP["i32" if dtype == "i32" else "f32"])
        return cls(arr.shape, dtype, None, arr)

    @property
    def size(self) -> int:
        return _size(self.shape)

    @property
    def nbytes(self) -> int:
        return self.size * L.DTYPE_SIZE[self.dtype]

    @property
    def ptr(self) -> int:
        """Device address; uploads a host-created tensor on first use."""
        if self._buf is None:
            if self._host is None:
                raise AlphaCudaError("tensor has neither device nor host storage (released?)")
            self._buf = _DeviceBuffer(self.nbytes)
            src = self._host
            if self.dtype == "bf16":
                src = f32_to_bf16_bits(src)
            src = np.ascontiguousarray(src)
            check(L.load().alpha_h2d(self._buf.ptr, src.ctypes.data, src.nbytes))
        return self._buf.ptr

    @property
    def data(self) -> np.ndarray:
        """Host copy (float32 / int32 numpy array); reads the device buffer back and waits."""
        if self._host is None:
            if self._buf is None:
                raise AlphaCudaError("tensor was released")
            if self.dtype == "bf16":
                raw = np.empty(self.shape, dtype=np.uint16)
                check(L.load().alpha_d2h(raw.ctypes.data, self._buf.ptr, raw.nbytes))
                self._host = bf16_to_f32(raw)
            else:
                arr = np.empty(self.shape, dtype=_NP[self.dtype])
                check(L.load().alpha_d2h(arr.ctypes.data, self._buf.ptr, arr.nbytes))
                self._host = arr
        return self._host

    def invalidate_host(self):
        self._host = None

    def item(self) -> float:
        return float(self.data.reshape(-1)[0])


class AsyncScalar:
    """A pending device-to-host read of one f32 / i32 element (see CudaBackend.readScalarAsync).
    Pinned slots and events are recycled through the backend: no allocation per read."""

    def __init__(self, backend: "CudaBackend", t: TensorData):
        if t.dtype == "bf16":
            raise AlphaCudaError("readScalarAsync: f32 or i32 tensors only")
        self._b = backend
        self._int = t.dtype == "i32"
        self._slot = backend._scalar_slot()
        arr, pin, ev = self._slot
        check(backend.lib.alpha_d2h_async(pin, t.ptr, 4))
        check(backend.lib.alpha_event_record(ev.value))
        self._val = None

    def get(self) -> float:
        if self._val is None:
            arr, pin, ev = self._slot
            check(self._b.lib.alpha_event_sync(ev.value))
            self._val = float(arr.view(np.int32)[0]) if self._int else float(arr[0])
            self._b._scalar_free.append(self._slot)
            self._slot = None
        return self._val


class CudaBackend:
    """interfaces.ts:38-151 on a B200.  ``dtype`` strings: "f32", "bf16", "i32"."""

    name = "alpha_cuda"

    def __init__(self, device: int = 0):
        self.lib = L.load()
        check(self.lib.alpha_init(int(device)))
        self.device = int(device)
        self._ops_mark = self.launch_count()
        self._rng = None

    # ── helpers ──────────────────────────────────────────────────────────────
    def _new(self, shape, dtype) -> TensorData:
        shape = tuple(int(d) for d in shape)
        return TensorData(shape, dtype, _DeviceBuffer(_size(shape) * L.DTYPE_SIZE[dtype]))

    @staticmethod
    def _code(dtype: str) -> int:
        return L.DTYPE_CODE[dtype]

    @staticmethod
    def _same(a: TensorData, b: TensorData, what: str):
        if a.shape != b.shape:
            raise AlphaCudaError(f"{what}: shape mismatch {a.shape} vs {b.shape}")
        if a.dtype != b.dtype:
            raise AlphaCudaError(f"{what}: dtype mismatch {a.dtype} vs {b.dtype}")

    def launch_count(self) -> int:
        out = C.c_uint64()
        check(self.lib.alpha_launch_count(C.byref(out)))
        return out.value

    # ── duck-typed extras probed by the trainer/CLI (trainer.ts:998-1044; train.ts:284-318)
    def releaseGpuTensor(self, td: TensorData) -> None:
        if td is not None and td._buf is not None:
            td._buf = None          # the buffer frees itself when its last sharer lets go
            td._host = None

    def flush(self) -> None:        # work is already enqueued on the stream
        return None

    def syncGpu(self) -> None:
        check(self.lib.alpha_stream_sync())

    def rangePush(self, name: str) -> None:
        """Open a named NVTX range on the host timeline (see alpha_range_push)."""
        self.lib.alpha_range_push(name.encode())

    def rangePop(self) -> None:
        self.lib.alpha_range_pop()

    def checkAsyncError(self) -> None:
        check(self.lib.alpha_check_async_error())

    def purgeBufferPools(self) -> None:
        check(self.lib.alpha_purge_pools())

    def gpuMemStats(self) -> dict:
        s = L.MemStats()
        check(self.lib.alpha_mem_stats(C.byref(s)))
        return {"bytesInUse": s.bytes_in_use, "bytesCached": s.bytes_cached, "peakInUse": s.peak_in_use,
                "deviceMallocs": s.n_device_mallocs, "allocs": s.n_allocs}

    def getDeviceInfo(self) -> dict:
        d = L.DeviceInfo()
        check(self.lib.alpha_device_info(C.byref(d)))
        return {"deviceName": d.name.decode(), "vendorId": d.vendor_id, "smCount": d.sm_count,
                "computeCapability": (d.cc_major, d.cc_minor), "totalMem": d.total_mem, "l2Bytes": d.l2_bytes}

    def resetStepOps(self) -> None:
        self._ops_mark = self.launch_count()

    @property
    def gpuOpsThisStep(self) -> int:
        return self.launch_count() - self._ops_mark

    def smokeTest(self) -> bool:
        a = self.fromArray([1, 2, 3, 4], [2, 2])
        b = self.fromArray([5, 6, 7, 8], [2, 2])
        return [round(float(v)) for v in self.matmul(a, b).data.reshape(-1)] == [19, 22, 43, 50]

    # ── creation (interfaces.ts:42-46) ───────────────────────────────────────
    def zeros(self, shape, dtype: str = "f32") -> TensorData:
        t = self._new(shape, dtype)
        check(self.lib.alpha_memset(t.ptr, 0, t.nbytes))
        return t

    def full(self, shape, value: float, dtype: str = "f32") -> TensorData:
        t = self._new(shape, dtype)
        check(self.lib.alpha_fill(t.ptr, t.size, float(value), self._code(dtype)))
        return t

    def ones(self, shape, dtype: str = "f32") -> TensorData:
        return self.full(shape, 1.0, dtype)

    def randn(self, shape, dtype: str = "f32") -> TensorData:
        """cpu_ref.ts:134-140: Gaussian samples from the backend's own SeededRng(42)."""
        from .rng import SeededRng
        if self._rng is None:
            self._rng = SeededRng(42)
        return self.upload(self._rng.fill_gauss(shape, 1.0), dtype)

    def fromArray(self, data, shape, dtype: str = "f32") -> TensorData:
        arr = np.asarray(data, dtype=np.int32 if dtype == "i32" else np.float32)
        if arr.size != _size(shape):
            raise AlphaCudaError(f"Data length {arr.size} does not match shape size {_size(shape)}")
        return self.upload(arr.reshape(shape), dtype)

    def upload(self, array: np.ndarray, dtype: str | None = None) -> TensorData:
        t = TensorData.from_host(array, dtype)
        t.ptr  # upload now
        if t.dtype == "bf16":
            t._host = None
        return t

    def uploadAsync(self, array: np.ndarray, dtype: str = "i32") -> TensorData:
        """Enqueue a copy of ``array`` (page-locked memory from ``pinned_array``, i32 or f32)
        into a new device tensor and return at once.  The caller must not write ``array``
        again before an event recorded after this call has completed; the tensor keeps no
        host copy."""
        if dtype == "bf16":
            raise AlphaCudaError("uploadAsync: i32 or f32 only")
        if not array.flags["C_CONTIGUOUS"] or array.dtype != _NP[dtype]:
            raise AlphaCudaError("uploadAsync: contiguous array of the tensor's own type required")
        t = self._new(array.shape, dtype)
        check(self.lib.alpha_h2d(t.ptr, array.ctypes.data, array.nbytes))
        return t

    def eventCreate(self) -> "C.c_uint64":
        ev = C.c_uint64()
        check(self.lib.alpha_event_create(C.byref(ev)))
        return ev

    def eventRecord(self, ev) -> None:
        check(self.lib.alpha_event_record(ev.value))

    def eventSync(self, ev) -> None:
        check(self.lib.alpha_event_sync(ev.value))

    def eventDestroy(self, ev) -> None:
        check(self.lib.alpha_event_destroy(ev.value))

    def pinned_array(self, shape, np_dtype):
        """A numpy array over page-locked host memory (uploads from it are asynchronous) and
        the handle that keeps the allocation alive; free it with ``free_pinned``."""
        nbytes = int(np.prod(shape)) * np.dtype(np_dtype).itemsize
        p = C.c_void_p()
        check(self.lib.alpha_host_alloc(max(nbytes, 1), C.byref(p)))
        buf = (C.c_char * max(nbytes, 1)).from_address(p.value)
        arr = np.frombuffer(buf, dtype=np_dtype, count=int(np.prod(shape))).reshape(shape)
        arr[...] = 0
        return arr, p

    def free_pinned(self, handle) -> None:
        check(self.lib.alpha_host_free(handle))

    def _scalar_slot(self):
        free = self.__dict__.setdefault("_scalar_free", [])
        if free:
            return free.pop()
        arr, pin = self.pinned_array((1,), np.float32)
        ev = C.c_uint64()
        check(self.lib.alpha_event_create(C.byref(ev)))
        return (arr, pin, ev)

    def readScalarAsync(self, t: TensorData) -> "AsyncScalar":
        """Start copying a one-element tensor to pinned host memory; ``.get()`` on the returned
        handle waits only for that copy, not for work enqueued after this call — so the loss of
        step i can be read while step i+1 is already running."""
        return AsyncScalar(self, t)

    # ── elementwise (interfaces.ts:49-71) ────────────────────────────────────
    def _binary(self, op: int, a: TensorData, b: TensorData) -> TensorData:
        if a.dtype != b.dtype:
            raise AlphaCudaError(f"binary op: dtype mismatch {a.dtype} vs {b.dtype}")
        if a.shape == b.shape:
            out = self._new(a.shape, a.dtype)
            check(self.lib.alpha_binary(op, a.ptr, b.ptr, out.ptr, a.size, self._code(a.dtype)))
            return out
        shape = tuple(np.broadcast_shapes(a.shape, b.shape))     # packages/core/src/broadcast.ts
        nd = len(shape)

        def strides(s):
            s = (1,) * (nd - len(s)) + tuple(s)
            st, acc = [0] * nd, 1
            for d in range(nd - 1, -1, -1):
                st[d] = 0 if s[d] == 1 else acc
                acc *= s[d]
            return st
        if nd > 6:
            raise AlphaCudaError("broadcast: more than 6 dimensions")
        out = self._new(shape, a.dtype)
        A = (C.c_int64 * nd)
        check(self.lib.alpha_binary_bcast(op, a.ptr, b.ptr, out.ptr, nd, A(*shape), A(*strides(a.shape)),
                                          A(*strides(b.shape)), self._code(a.dtype)))
        return out

    def add(self, a, b): return self._binary(L.ADD, a, b)
    def sub(self, a, b): return self._binary(L.SUB, a, b)
    def mul(self, a, b): return self._binary(L.MUL, a, b)
    def div(self, a, b): return self._binary(L.DIV, a, b)

    def _unary(self, op: int, a: TensorData, p0: float = 0.0, p1: float = 0.0) -> TensorData:
        out = self._new(a.shape, a.dtype)
        check(self.lib.alpha_unary(op, a.ptr, out.ptr, a.size, float(p0), float(p1), self._code(a.dtype)))
        return out

    def neg(self, a): return self._unary(L.NEG, a)
    def exp(self, a): return self._unary(L.EXP, a)
    def log(self, a): return self._unary(L.LOG, a)
    def sqrt(self, a): return self._unary(L.SQRT, a)
    def pow(self, a, e): return self._unary(L.POW, a, e)
    def scale(self, a, s): return self._unary(L.SCALE, a, s)
    def clamp(self, a, lo, hi): return self._unary(L.CLAMP, a, lo, hi)
    def gelu(self, a): return self._unary(L.GELU, a)
    def relu(self, a): return self._unary(L.RELU, a)
    def silu(self, a): return self._unary(L.SILU, a)
    def softCap(self, a, cap): return self._unary(L.SOFTCAP, a, cap)

    def _unary_bwd(self, op, x, g, p0=0.0, p1=0.0) -> TensorData:
        self._same(x, g, "backward")
        out = self._new(x.shape, x.dtype)
        check(self.lib.alpha_unary_bwd(op, x.ptr, g.ptr, out.ptr, x.size, float(p0), float(p1), self._code(x.dtype)))
        return out

    def geluBackward(self, inp, grad): return self._unary_bwd(L.GELU, inp, grad)
    def reluBackward(self, inp, grad): return self._unary_bwd(L.RELU, inp, grad)
    def siluBackward(self, inp, grad): return self._unary_bwd(L.SILU, inp, grad)
    def clampBackward(self, inp, grad, lo, hi): return self._unary_bwd(L.CLAMP, inp, grad, lo, hi)
    def softCapBackward(self, grad, inp, cap): return self._unary_bwd(L.SOFTCAP, inp, grad, cap)

    def siluMul(self, a, b) -> TensorData:
        self._same(a, b, "siluMul")
        out = self._new(a.shape, a.dtype)
        check(self.lib.alpha_silu_mul_fwd(a.ptr, b.ptr, out.ptr, a.size, self._code(a.dtype)))
        return out

    def siluMulBackward(self, a, b, grad):
        da, db = self._new(a.shape, a.dtype), self._new(a.shape, a.dtype)
        check(self.lib.alpha_silu_mul_bwd(a.ptr, b.ptr, grad.ptr, da.ptr, db.ptr, a.size, self._code(a.dtype)))
        return [da, db]

    def addInplace(self, a: TensorData, b: TensorData) -> None:
        if a.size != b.size:
            raise AlphaCudaError(f"addInplace: size mismatch {a.shape} vs {b.shape}")
        check(self.lib.alpha_add_inplace(a.ptr, b.ptr, a.size, self._code(a.dtype), self._code(b.dtype)))
        a.invalidate_host()

    def scaleInplace(self, a: TensorData, s: float) -> None:
        check(self.lib.alpha_scale_inplace(a.ptr, float(s), a.size, self._code(a.dtype)))
        a.invalidate_host()

    def castDtype(self, a: TensorData, dtype: str) -> TensorData:
        if dtype == "f16":
            raise AlphaCudaError("castDtype: this backend stores half precision as bf16, not f16")
        out = self._new(a.shape, dtype)
        check(self.lib.alpha_cast(a.ptr, self._code(a.dtype), out.ptr, self._code(dtype), a.size))
        return out

    def castInto(self, src: TensorData, dst: TensorData) -> None:
        """dst[...] = src converted to dst's element type (same element count), in place."""
        if src.size != dst.size:
            raise AlphaCudaError(f"castInto: size mismatch {list(src.shape)} vs {list(dst.shape)}")
        check(self.lib.alpha_cast(src.ptr, self._code(src.dtype), dst.ptr, self._code(dst.dtype), src.size))
        dst.invalidate_host()

    def broadcast(self, a: TensorData, targetShape) -> TensorData:
        shape = tuple(int(d) for d in targetShape)
        nd = len(shape)
        s = (1,) * (nd - len(a.shape)) + a.shape
        st, acc = [0] * nd, 1
        for d in range(nd - 1, -1, -1):
            st[d] = 0 if (s[d] == 1 and shape[d] != 1) else acc
            acc *= s[d]
        out = self._new(shape, a.dtype)
        A = (C.c_int64 * nd)
        check(self.lib.alpha_broadcast(a.ptr, out.ptr, nd, A(*shape), A(*st), self._code(a.dtype)))
        return out

    def clone(self, a: TensorData) -> TensorData:
        out = self._new(a.shape, a.dtype)
        check(self.lib.alpha_d2d(out.ptr, a.ptr, a.nbytes))
        return out

    # ── matmul family (interfaces.ts:53,111-112) ─────────────────────────────
    def _gemm(self, layout, a, b, M, N, K, lda, ldb, out_dtype=None, epilogue=L.EPI_NONE, aux=None,
              out: TensorData | None = None, accumulate: bool = False, out_shape=None) -> TensorData:
        if a.dtype != b.dtype:
            raise AlphaCudaError(f"matmul: dtype mismatch {a.dtype} vs {b.dtype}")
        out_dtype = out_dtype or a.dtype
        if out is None:
            out = self._new(out_shape if out_shape is not None else (M, N), out_dtype)
        check(self.lib.alpha_gemm(layout, a.ptr, b.ptr, out.ptr, M, N, K, lda, ldb, N, self._code(a.dtype),
                                  self._code(out_dtype), epilogue, aux.ptr if aux is not None else 0, N,
                                  1 if accumulate else 0))
        out.invalidate_host()
        return out

    def matmul(self, a: TensorData, b: TensorData) -> TensorData:
        """cpu_ref.ts:166-258: [..., M, K] x [..., K, N] with broadcast batch dimensions."""
        if len(a.shape) < 2 or len(b.shape) < 2:
            raise AlphaCudaError(f"matmul requires at least 2D tensors, got {list(a.shape)} x {list(b.shape)}")
        M, K = a.shape[-2:]
        K2, N = b.shape[-2:]
        if K != K2:
            raise AlphaCudaError(f"matmul shape mismatch: {list(a.shape)} x {list(b.shape)}")
        ab, bb = a.shape[:-2], b.shape[:-2]
        if not ab and not bb:
            return self._gemm(L.GEMM_NN, a, b, M, N, K, K, N)
        if not bb:      # [..., M, K] x [K, N]: fold the batch into M
            rows = _size(ab) * M
            return self._gemm(L.GEMM_NN, a, b, rows, N, K, K, N, out_shape=ab + (M, N))
        batch_shape = tuple(np.broadcast_shapes(ab, bb))
        nb = _size(batch_shape)
        if a.dtype != "f32":
            raise AlphaCudaError("batched matmul is provided for f32 only (the unfused attention branch)")

        def bstride(s, per):
            if _size(s) == nb:
                return per
            if _size(s) == 1:
                return 0
            raise AlphaCudaError("matmul: partial batch broadcasting is not supported")
        out = self._new(batch_shape + (M, N), "f32")
        check(self.lib.alpha_gemm_batched_f32(L.GEMM_NN, a.ptr, b.ptr, out.ptr, M, N, K, K, N, N, nb,
                                              bstride(ab, M * K), bstride(bb, K * N), M * N))
        return out

    def matmulTransposed(self, a: TensorData, b: TensorData) -> TensorData:
        """C = A @ B^T with B stored [N, K] (ops.ts:191-196)."""
        K = a.shape[-1]
        N, K2 = b.shape[-2:]
        if K != K2 or len(b.shape) != 2:
            raise AlphaCudaError(f"matmulTransposed shape mismatch: {list(a.shape)} x {list(b.shape)}")
        rows = a.size // K
        return self._gemm(L.GEMM_NT, a, b, rows, N, K, K, K, out_shape=a.shape[:-1] + (N,))

    def matmulTransposedA(self, a: TensorData, b: TensorData, into: TensorData | None = None) -> TensorData:
        """C = A^T @ B with A stored [K, M], B [K, N] (ops.ts:176-177,224-225).  ``into``: an
        existing [M, N] gradient that the product is added to inside the GEMM (one pass instead
        of a product and a separate addInplace); it is returned."""
        K, M = a.size // a.shape[-1], a.shape[-1]
        K2, N = b.size // b.shape[-1], b.shape[-1]
        if K != K2:
            raise AlphaCudaError(f"matmulTransposedA shape mismatch: {list(a.shape)} x {list(b.shape)}")
        out_dtype = "f32" if a.dtype == "bf16" and self.param_grads_f32 else a.dtype
        if into is not None:
            if into.size != M * N or into.dtype != out_dtype:
                raise AlphaCudaError(f"matmulTransposedA: cannot accumulate into {list(into.shape)} {into.dtype}")
            return self._gemm(L.GEMM_TN, a, b, M, N, K, M, N, out_dtype=out_dtype, out=into, accumulate=True)
        return self._gemm(L.GEMM_TN, a, b, M, N, K, M, N, out_dtype=out_dtype)

    def pairSupported(self, first, second) -> bool:
        """Whether matmulTransposedAPair takes these two (a, b, into) triples: bf16 operands whose
        weight gradients are kept in f32."""
        return self.param_grads_f32 and all(a.dtype == "bf16" and b.dtype == "bf16" and (into is None or into.dtype == "f32")
                                            for a, b, into in (first, second))

    def matmulTransposedAPair(self, first, second) -> list:
        """Two weight gradients A_i^T @ B_i over the same K in one launch: each argument is
        (a [K, M], b [K, N], into or None) as for ``matmulTransposedA``; returns the two results.
        bf16 operands with f32 gradients only; two GEMMs that would each fill half of the device
        share the launch and need no split over K, any other pair runs as two GEMMs inside the
        library."""
        outs, args = [], []
        K = first[0].size // first[0].shape[-1]
        for a, b, into in (first, second):
            Ka, M = a.size // a.shape[-1], a.shape[-1]
            Kb, N = b.size // b.shape[-1], b.shape[-1]
            if Ka != K or Kb != K or a.dtype != "bf16" or b.dtype != "bf16" or not self.param_grads_f32:
                raise AlphaCudaError("matmulTransposedAPair: needs bf16 operands over one K and f32 gradients")
            if into is not None and (into.size != M * N or into.dtype != "f32"):
                raise AlphaCudaError(f"matmulTransposedAPair: cannot accumulate into {list(into.shape)} {into.dtype}")
            out = into if into is not None else self._new((M, N), "f32")
            outs.append(out)
            args += [a.ptr, b.ptr, out.ptr, M, N, M, N, N, 1 if into is not None else 0]
        check(self.lib.alpha_gemm_tn_pair(*args, K))
        for o in outs:
            o.invalidate_host()
        return outs

    def matmulInto(self, a: TensorData, b: TensorData, into: TensorData) -> TensorData:
        """into += A @ B for A [rows, K], B [K, N] with the add in the GEMM epilogue (the
        gradient of an activation that already has one from another consumer)."""
        K, N = b.shape
        rows = a.size // K
        if into.size != rows * N or into.dtype != a.dtype:
            raise AlphaCudaError(f"matmulInto: cannot accumulate into {list(into.shape)} {into.dtype}")
        return self._gemm(L.GEMM_NN, a, b, rows, N, K, K, N, epilogue=L.EPI_ADD, aux=into, out=into)

    #: weight gradients of bf16 GEMMs are produced in f32 (they feed f32 AdamW state)
    param_grads_f32 = True

    # fused forms (no reference counterpart as single dispatches; ops.ts:426-487 fuses only on the tape)
    def matmulTransposedGelu(self, a: TensorData, b: TensorData):
        """Returns (pre_activation, gelu(pre_activation)) from one GEMM launch."""
        K = a.shape[-1]
        N = b.shape[0]
        rows = a.size // K
        pre = self._new(a.shape[:-1] + (N,), a.dtype)
        act = self._gemm(L.GEMM_NT, a, b, rows, N, K, K, K, epilogue=L.EPI_GELU, aux=pre,
                         out_shape=a.shape[:-1] + (N,))
        return pre, act

    def matmulTransposedAdd(self, a: TensorData, b: TensorData, residual: TensorData) -> TensorData:
        """residual + A @ B^T in the GEMM epilogue."""
        K = a.shape[-1]
        N = b.shape[0]
        rows = a.size // K
        return self._gemm(L.GEMM_NT, a, b, rows, N, K, K, K, epilogue=L.EPI_ADD, aux=residual,
                          out_shape=residual.shape)

    def matmulGeluBackward(self, g: TensorData, w: TensorData, pre: TensorData) -> TensorData:
        """(G @ W) * gelu'(pre) in the GEMM epilogue; G [rows, N], W [N, K], pre [rows, K]."""
        N, K = w.shape
        rows = g.size // N
        return self._gemm(L.GEMM_NN, g, w, rows, K, N, N, K, epilogue=L.EPI_GELU_BWD, aux=pre, out_shape=pre.shape)

    # ── reductions (interfaces.ts:54-55,72-73,144-146) ───────────────────────
    def sum(self, a: TensorData, axis: int | None = None, keepdims: bool = False, _scale: float = 1.0) -> TensorData:
        if axis is None:
            shape = tuple(1 for _ in a.shape) if keepdims else ()
            out = self._new(shape, a.dtype)
            check(self.lib.alpha_sum_axis(a.ptr, out.ptr, 1, a.size, 1, _scale, self._code(a.dtype)))
            return out
        ax = axis + len(a.shape) if axis < 0 else axis
        if not 0 <= ax < len(a.shape):
            raise AlphaCudaError(f"axis {axis} out of range for shape {list(a.shape)}")
        outer, dim, inner = _size(a.shape[:ax]), a.shape[ax], _size(a.shape[ax + 1:])
        shape = a.shape[:ax] + ((1,) if keepdims else ()) + a.shape[ax + 1:]
        out = self._new(shape, a.dtype)
        check(self.lib.alpha_sum_axis(a.ptr, out.ptr, outer, dim, inner, _scale, self._code(a.dtype)))
        return out

    def mean(self, a, axis=None, keepdims=False) -> TensorData:
        n = a.size if axis is None else a.shape[axis]
        return self.sum(a, axis, keepdims, _scale=1.0 / n)

    def _softmax(self, a, axis, log_mode) -> TensorData:
        ax = len(a.shape) - 1 if axis is None else (axis + len(a.shape) if axis < 0 else axis)
        if ax != len(a.shape) - 1:
            raise AlphaCudaError("softmax: only the last axis is supported")
        cols = a.shape[-1]
        out = self._new(a.shape, a.dtype)
        check(self.lib.alpha_softmax(a.ptr, out.ptr, a.size // cols, cols, log_mode, self._code(a.dtype)))
        return out

    def softmax(self, a, axis=None): return self._softmax(a, axis, 0)
    def logSoftmax(self, a, axis=None): return self._softmax(a, axis, 1)

    def totalSumOfSquares(self, tensors: Sequence[TensorData]) -> TensorData:
        n = len(tensors)
        out = self._new((), "f32")
        ptrs = (C.c_uint64 * n)(*[t.ptr for t in tensors])
        counts = (C.c_int64 * n)(*[t.size for t in tensors])
        dts = (C.c_int32 * n)(*[self._code(t.dtype) for t in tensors])
        check(self.lib.alpha_sumsq_multi(ptrs, counts, dts, n, out.ptr))
        return out

    def sumOfSquares(self, t: TensorData) -> TensorData:
        return self.totalSumOfSquares([t])

    def checkFinite(self, t: TensorData) -> TensorData:
        out = self._new((), "f32")
        check(self.lib.alpha_check_finite(t.ptr, t.size, self._code(t.dtype), out.ptr))
        return out

    # ── nn (interfaces.ts:67-74, 103-105) ────────────────────────────────────
    def embedding(self, weight: TensorData, indices: TensorData) -> TensorData:
        vocab, dim = weight.shape
        out = self._new(tuple(indices.shape) + (dim,), weight.dtype)
        check(self.lib.alpha_embedding_fwd(weight.ptr, indices.ptr, out.ptr, indices.size, dim, vocab,
                                           self._code(weight.dtype)))
        return out

    def embeddingPos(self, wte: TensorData, wpe: TensorData, tokens: TensorData) -> TensorData:
        """wte[tokens] + wpe[position] in one pass (gpt.ts:362-379 as a single kernel)."""
        Bn, T = tokens.shape
        vocab, dim = wte.shape
        out = self._new((Bn, T, dim), wte.dtype)
        check(self.lib.alpha_embedding_pos_fwd(wte.ptr, wpe.ptr, tokens.ptr, out.ptr, Bn, T, dim, vocab,
                                               self._code(wte.dtype)))
        return out

    def embeddingBackward(self, indices: TensorData, gradOutput: TensorData, vocabSize: int,
                          out: TensorData | None = None) -> TensorData:
        dim = gradOutput.shape[-1]
        acc = out is not None
        if out is None:
            out = self._new((vocabSize, dim), "f32")
        check(self.lib.alpha_embedding_bwd(indices.ptr, gradOutput.ptr, out.ptr, indices.size, dim, vocabSize,
                                           self._code(gradOutput.dtype), 1 if acc else 0))
        out.invalidate_host()
        return out

    def layerNorm(self, x, weight, bias, eps) -> TensorData:
        dim = x.shape[-1]
        out = self._new(x.shape, x.dtype)
        check(self.lib.alpha_layernorm_fwd(x.ptr, weight.ptr, bias.ptr, out.ptr, x.size // dim, dim, float(eps),
                                           self._code(x.dtype)))
        return out

    def layerNormBackward(self, x, weight, gradOutput, eps, dxInto: TensorData | None = None) -> dict:
        """``dxInto``: an existing gradient of x; the kernel adds dx to it in place (one pass
        instead of a separate addInplace) and "dx" is that tensor."""
        dim = x.shape[-1]
        dx = dxInto if dxInto is not None else self._new(x.shape, x.dtype)
        dw, db = self._new(weight.shape, "f32"), self._new(weight.shape, "f32")
        check(self.lib.alpha_layernorm_bwd(x.ptr, weight.ptr, gradOutput.ptr, dx.ptr, dw.ptr, db.ptr,
                                           x.size // dim, dim, float(eps), self._code(x.dtype), 0,
                                           dxInto.ptr if dxInto is not None else 0))
        dx.invalidate_host()
        return {"dx": dx, "dw": dw, "db": db}

    def rmsNorm(self, x, weight, eps) -> TensorData:
        dim = x.shape[-1]
        out = self._new(x.shape, x.dtype)
        check(self.lib.alpha_rmsnorm_fwd(x.ptr, weight.ptr, out.ptr, x.size // dim, dim, float(eps),
                                         self._code(x.dtype)))
        return out

    def rmsNormBackward(self, x, weight, gradOutput, eps, dxInto: TensorData | None = None) -> dict:
        dim = x.shape[-1]
        dx = dxInto if dxInto is not None else self._new(x.shape, x.dtype)
        dw = self._new(weight.shape, "f32")
        check(self.lib.alpha_rmsnorm_bwd(x.ptr, weight.ptr, gradOutput.ptr, dx.ptr, dw.ptr, x.size // dim, dim,
                                         float(eps), self._code(x.dtype), 0, dxInto.ptr if dxInto is not None else 0))
        dx.invalidate_host()
        return {"dx": dx, "dw": dw}

    def rope(self, x: TensorData, batch: int, T: int, heads: int, D: int, ld: int, col_offset: int = 0,
             theta: float = 10000.0, inverse: bool = False) -> None:
        """In-place rotary embedding on the column block [col_offset, col_offset + heads*D) of x [batch*T, ld]."""
        p = x.ptr + col_offset * L.DTYPE_SIZE[x.dtype]
        check(self.lib.alpha_rope(p, p, batch, T, heads, D, ld, float(theta), 1 if inverse else 0,
                                  self._code(x.dtype)))
        x.invalidate_host()

    def ropeQkv(self, qkv: TensorData, batch: int, T: int, heads: int, theta: float = 10000.0,
                inverse: bool = False) -> TensorData:
        """Rotary embedding of the q and k column blocks of a fused activation [batch*T, 3E] into a
        new tensor (v copied alongside): one pass over the rows."""
        E3 = qkv.shape[-1]
        D = E3 // 3 // heads
        out = self._new(qkv.shape, qkv.dtype)
        check(self.lib.alpha_rope_qkv(qkv.ptr, out.ptr, batch, T, heads, D, float(theta), 1 if inverse else 0,
                                      self._code(qkv.dtype)))
        return out

    def crossEntropy(self, logits: TensorData, targets: TensorData) -> TensorData:
        N, V = logits.shape
        out = self._new((), "f32")
        check(self.lib.alpha_cross_entropy_fwd(logits.ptr, targets.ptr, out.ptr, N, V, V, self._code(logits.dtype)))
        return out

    def crossEntropyBackward(self, logits, targets, gradOutput) -> TensorData:
        N, V = logits.shape
        out = self._new(logits.shape, logits.dtype)
        check(self.lib.alpha_cross_entropy_bwd(logits.ptr, targets.ptr, gradOutput.ptr, out.ptr, N, V, V,
                                               self._code(logits.dtype)))
        return out

    def lmHeadLoss(self, x: TensorData, w: TensorData, targets: TensorData, gradScale: float = 1.0):
        """Fused head: logits = x @ w^T into a row-padded buffer, then softmax-CE forward and
        backward in one pass over it.  Returns (loss scalar f32, dlogits [N, ld], ld)."""
        V, E = w.shape
        N = x.size // E
        ld = (V + 63) // 64 * 64
        logits = TensorData((N, ld), x.dtype, _DeviceBuffer(N * ld * L.DTYPE_SIZE[x.dtype]))
        check(self.lib.alpha_gemm(L.GEMM_NT, x.ptr, w.ptr, logits.ptr, N, V, E, E, E, ld, self._code(x.dtype),
                                  self._code(x.dtype), L.EPI_NONE, 0, 0, 0))
        loss = self._new((), "f32")
        check(self.lib.alpha_softmax_ce_fwd_bwd(logits.ptr, targets.ptr, logits.ptr, loss.ptr, N, V, ld,
                                                float(gradScale), self._code(x.dtype)))
        return loss, logits, ld

    def lmHeadBackward(self, dlogits: TensorData, ld: int, x: TensorData, w: TensorData, dw_out: TensorData | None):
        """dx = dlogits @ w ; dw (+)= dlogits^T @ x, reading the padded dlogits in place."""
        V, E = w.shape
        N = x.size // E
        dx = self._new(x.shape, x.dtype)
        check(self.lib.alpha_gemm(L.GEMM_NN, dlogits.ptr, w.ptr, dx.ptr, N, E, V, ld, E, E, self._code(x.dtype),
                                  self._code(x.dtype), L.EPI_NONE, 0, 0, 0))
        acc = dw_out is not None
        dw_dtype = "f32" if (x.dtype == "f32" or self.param_grads_f32) else x.dtype
        dw = dw_out if acc else self._new((V, E), dw_dtype)
        check(self.lib.alpha_gemm(L.GEMM_TN, dlogits.ptr, x.ptr, dw.ptr, V, E, N, ld, E, E, self._code(x.dtype),
                                  self._code(dw.dtype), L.EPI_NONE, 0, 0, 1 if acc else 0))
        dw.invalidate_host()
        return dx, dw

    # ── views / layout (interfaces.ts:77-80,117-121) ─────────────────────────
    def reshape(self, a: TensorData, shape) -> TensorData:
        shape = tuple(int(d) for d in shape)
        if _size(shape) != a.size:
            raise AlphaCudaError(f"Cannot reshape {list(a.shape)} to {list(shape)}: size mismatch")
        a.ptr  # make sure the storage exists before it is shared
        return TensorData(shape, a.dtype, a._buf, None)

    def transpose(self, a: TensorData, dim0: int, dim1: int) -> TensorData:
        nd = len(a.shape)
        d0 = dim0 + nd if dim0 < 0 else dim0
        d1 = dim1 + nd if dim1 < 0 else dim1
        shape = list(a.shape)
        shape[d0], shape[d1] = shape[d1], shape[d0]
        out = self._new(shape, a.dtype)
        check(self.lib.alpha_transpose(a.ptr, out.ptr, nd, (C.c_int64 * nd)(*a.shape), d0, d1, self._code(a.dtype)))
        return out

    def slice(self, a: TensorData, starts, ends) -> TensorData:
        if len(a.shape) != 2 or starts[0] != 0 or ends[0] != a.shape[0]:
            raise AlphaCudaError("slice: only column ranges of 2-D tensors are on the train-step path")
        rows, cols = a.shape
        out = self._new((rows, ends[1] - starts[1]), a.dtype)
        check(self.lib.alpha_slice_cols(a.ptr, out.ptr, rows, cols, starts[1], ends[1], self._code(a.dtype)))
        return out

    def scatterSlice(self, grad: TensorData, origShape, starts, ends) -> TensorData:
        if len(origShape) != 2 or starts[0] != 0 or ends[0] != origShape[0]:
            raise AlphaCudaError("scatterSlice: only column ranges of 2-D tensors are on the train-step path")
        rows, cols = origShape
        out = self._new(origShape, grad.dtype)
        check(self.lib.alpha_scatter_cols(grad.ptr, out.ptr, rows, cols, starts[1], ends[1], self._code(grad.dtype)))
        return out

    def sliceQkv(self, a: TensorData):
        rows, c3 = a.shape
        d = c3 // 3
        q, k, v = (self._new((rows, d), a.dtype) for _ in range(3))
        check(self.lib.alpha_slice_qkv(a.ptr, q.ptr, k.ptr, v.ptr, rows, d, self._code(a.dtype)))
        return q, k, v

    def causalMask(self, size: int) -> TensorData:
        out = self._new((size, size), "f32")
        check(self.lib.alpha_causal_mask(out.ptr, size))
        return out

    def maskedFill(self, a: TensorData, mask: TensorData, value: float) -> TensorData:
        out = self._new(a.shape, a.dtype)
        check(self.lib.alpha_masked_fill(a.ptr, mask.ptr, out.ptr, a.size, mask.size, float(value),
                                         self._code(a.dtype)))
        return out

    def dropoutMask(self, shape, seed: int, counter: int, p: float, dtype: str = "f32") -> TensorData:
        out = self._new(shape, dtype)
        check(self.lib.alpha_dropout_mask(out.ptr, out.size, seed, counter, float(p), self._code(dtype)))
        return out

    def residualDropoutAdd(self, residual, projected, mask) -> TensorData:
        out = self._new(residual.shape, residual.dtype)
        check(self.lib.alpha_residual_dropout_add(residual.ptr, projected.ptr, mask.ptr, out.ptr, residual.size,
                                                  self._code(residual.dtype)))
        return out

    # ── fused attention (interfaces.ts:127-135) ──────────────────────────────
    def flashAttention(self, Q: TensorData, K: TensorData, V: TensorData, T: int, scale: float, softCap: float):
        """Q, K, V: [B*H, T, D] contiguous.  Returns {output [B*H,T,D], lse [B*H,T]}."""
        BH, T2, D = Q.shape
        if T2 != T:
            raise AlphaCudaError(f"flashAttention: T={T} does not match Q {list(Q.shape)}")
        p = L.AttnParams(batch=BH, heads=1, T=T, D=D, q_sb=T * D, q_sh=0, q_st=D, o_sb=T * D, o_sh=0, o_st=D,
                         scale=float(scale), soft_cap=float(softCap), dtype=self._code(Q.dtype))
        out, lse = self._new(Q.shape, Q.dtype), self._new((BH, T), "f32")
        check(self.lib.alpha_flash_attn_fwd(Q.ptr, K.ptr, V.ptr, out.ptr, lse.ptr, C.byref(p)))
        return {"output": out, "lse": lse}

    def flashAttentionBackward(self, Q, K, V, O, dO, lse, T: int, scale: float, softCap: float):
        BH, _, D = Q.shape
        p = L.AttnParams(batch=BH, heads=1, T=T, D=D, q_sb=T * D, q_sh=0, q_st=D, o_sb=T * D, o_sh=0, o_st=D,
                         scale=float(scale), soft_cap=float(softCap), dtype=self._code(Q.dtype))
        dq, dk, dv = (self._new(Q.shape, Q.dtype) for _ in range(3))
        check(self.lib.alpha_flash_attn_bwd(Q.ptr, K.ptr, V.ptr, O.ptr, dO.ptr, lse.ptr, dq.ptr, dk.ptr, dv.ptr,
                                            C.byref(p)))
        return {"dQ": dq, "dK": dk, "dV": dv}

    def _qkv_params(self, qkv: TensorData, Bn: int, T: int, H: int, scale: float, softCap: float):
        E3 = qkv.shape[-1]
        E = E3 // 3
        D = E // H
        return L.AttnParams(batch=Bn, heads=H, T=T, D=D, q_sb=T * E3, q_sh=D, q_st=E3, o_sb=T * E, o_sh=D, o_st=E,
                            scale=float(scale), soft_cap=float(softCap), dtype=self._code(qkv.dtype)), E, D

    def attentionQkv(self, qkv: TensorData, Bn: int, T: int, H: int, scale: float, softCap: float):
        """Causal multi-head attention reading q, k, v in place from the fused projection
        [B*T, 3E] (head h of q at columns h*D.., k at E + h*D.., v at 2E + h*D..) and writing
        the head-merged output [B*T, E].  Replaces sliceQkv + 3 reshapes/transposes +
        attention + the merge transpose of gpt.ts:234-254/256-279."""
        p, E, D = self._qkv_params(qkv, Bn, T, H, scale, softCap)
        es = L.DTYPE_SIZE[qkv.dtype]
        out, lse = self._new((Bn * T, E), qkv.dtype), self._new((Bn * H, T), "f32")
        base = qkv.ptr
        check(self.lib.alpha_flash_attn_fwd(base, base + E * es, base + 2 * E * es, out.ptr, lse.ptr, C.byref(p)))
        return out, lse

    def attentionQkvBackward(self, qkv, out, dout, lse, Bn: int, T: int, H: int, scale: float, softCap: float,
                             delta: TensorData | None = None):
        """Returns dqkv [B*T, 3E]: dq, dk, dv written straight into their column blocks.
        ``delta``: the row-dots dO.O [B, H, T] when the caller has them already (matmulRowdot);
        the forward output is then not read."""
        p, E, D = self._qkv_params(qkv, Bn, T, H, scale, softCap)
        es = L.DTYPE_SIZE[qkv.dtype]
        dqkv = self._new(qkv.shape, qkv.dtype)
        b, d = qkv.ptr, dqkv.ptr
        if delta is not None:
            check(self.lib.alpha_flash_attn_bwd_delta(b, b + E * es, b + 2 * E * es, dout.ptr, lse.ptr, delta.ptr,
                                                      d, d + E * es, d + 2 * E * es, C.byref(p)))
            return dqkv
        check(self.lib.alpha_flash_attn_bwd(b, b + E * es, b + 2 * E * es, out.ptr, dout.ptr, lse.ptr,
                                            d, d + E * es, d + 2 * E * es, C.byref(p)))
        return dqkv

    def rowdotSupported(self, g: TensorData, o: TensorData, H: int) -> bool:
        """Whether matmulRowdot / attentionQkvBackward(delta=) apply: bf16, head dim 64."""
        return g.dtype == "bf16" and o.dtype == "bf16" and o.shape[-1] == 64 * H

    def matmulRowdot(self, g: TensorData, w: TensorData, o: TensorData, T: int, H: int):
        """(G @ W, delta): the gradient of the attention output, dO = G @ W for G [rows, N], W [N, E],
        together with delta[b, h, t] = sum_d dO * O over each head's 64 columns, from one GEMM
        launch (the row-dot is taken in the epilogue, on dO as rounded to bf16)."""
        N, E = w.shape
        rows = g.size // N
        dO = self._new(o.shape, o.dtype)
        delta = self._new((rows // T, H, T), "f32")
        check(self.lib.alpha_gemm_nn_rowdot(g.ptr, w.ptr, dO.ptr, rows, E, N, N, E, E, o.ptr, E, delta.ptr, T, H))
        return dO, delta

    # ── optimizer (interfaces.ts:149-150) ────────────────────────────────────
    def adamwStep(self, params, grads, m, v, lr, beta1, beta2, eps, weightDecay, bc1, bc2, gradScale=1.0,
                  shadow: TensorData | None = None) -> None:
        check(self.lib.alpha_adamw(params.ptr, grads.ptr, m.ptr, v.ptr, params.size, lr, beta1, beta2, eps,
                                   weightDecay, bc1, bc2, gradScale, self._code(grads.dtype),
                                   shadow.ptr if shadow is not None else 0))
        for t in (params, m, v, shadow):
            if t is not None:
                t.invalidate_host()

    def adamwStepMulti(self, entries: Iterable[tuple], lr, beta1, beta2, eps, bc1, bc2, gradScale=1.0,
                       clipSumSq: TensorData | None = None, maxNorm: float = 0.0) -> None:
        """entries: (param, grad, m, v, weightDecay, shadow|None).  One launch for all tensors;
        with clipSumSq the clip coefficient is derived on the device (trainer.ts:1650-1656)."""
        entries = list(entries)
        arr = (L.AdamWTensor * len(entries))()
        for i, (p, g, m, v, wd, sh) in enumerate(entries):
            arr[i] = L.AdamWTensor(p.ptr, g.ptr, m.ptr, v.ptr, sh.ptr if sh is not None else 0, p.size, wd,
                                   self._code(g.dtype))
        check(self.lib.alpha_adamw_multi(arr, len(entries), lr, beta1, beta2, eps, bc1, bc2, gradScale,
                                         clipSumSq.ptr if clipSumSq is not None else 0, float(maxNorm)))
        for (p, g, m, v, wd, sh) in entries:
            for t in (p, m, v, sh):
                if t is not None:
                    t.invalidate_host()

    # ── comparison (interfaces.ts:87-88) — host reads, off the hot path ───────
    def equal(self, a: TensorData, b: TensorData) -> bool:
        return a.shape == b.shape and a.dtype == b.dtype and bool(np.all(a.data == b.data))

    def allClose(self, a: TensorData, b: TensorData, atol: float = 1e-5, rtol: float = 1e-8) -> bool:
        if a.shape != b.shape:
            return False
        x, y = a.data.astype(np.float64), b.data.astype(np.float64)
        return bool(np.all(np.abs(x - y) <= atol + rtol * np.abs(y)))

    # ── not on the train-step path (sampling / eval utilities of the interface) ─────────
    def _off_path(self, name):
        raise AlphaCudaError(f"{name} is not part of the train-step path this backend implements")

    def cat(self, tensors, axis): self._off_path("cat")
    def argmax(self, a, axis=None): self._off_path("argmax")
    def topk(self, a, k, axis=None): self._off_path("topk")
    def gather(self, a, axis, indices): self._off_path("gather")
