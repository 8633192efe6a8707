"""The failure paths of the device code, exercised without making a GPU fault, trap or hang.

Every spin-wait in the tensor-core kernels has a limit; when it runs out the kernel sets an
abort flag, all roles unwind, tensor memory is given back and an error word is set that
``alpha_check_async_error`` reports.  ``alpha_debug_wait_expiry`` runs a kernel with the same
skeleton whose producer waits, with a millisecond limit, on a barrier nothing signals: the wait
gives up and the kernel returns.  Checked: the status comes back with the expected message, the
error is reported once, and tensor-core work launched afterwards is correct (tensor memory was
freed, the context is intact).
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def B():
    from alpha2_b200.backend import CudaBackend
    b = CudaBackend(0)
    yield b
    b.checkAsyncError()


def _gemm_ok(B):
    r = np.random.default_rng(0)
    from tests.test_gpu_fullsize import bf16_round
    a, b = bf16_round(r.standard_normal((512, 256)) * 0.1), bf16_round(r.standard_normal((384, 256)) * 0.1)
    got = B.matmulTransposed(B.upload(a, "bf16"), B.upload(b, "bf16")).data
    want = a.astype(np.float64) @ b.astype(np.float64).T
    return float(np.max(np.abs(got - want))) < 2 ** -7 * float(np.max(np.abs(want))) + 1e-3


@pytest.mark.parametrize("blocks,limit_us", [(1, 1000), (148, 500), (296, 2000)])
def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable(B, blocks, limit_us):
    from alpha2_b200._lib import AlphaCudaError
    assert _gemm_ok(B)
    B.checkAsyncError()                                     # clean before the probe
    left = C.c_int(-1)
    assert B.lib.alpha_debug_wait_expiry(blocks, limit_us, C.byref(left)) == 0
    assert left.value == 6 * blocks                         # producer, MMA and four epilogue warps of every block
    with pytest.raises(AlphaCudaError, match="gave up a bounded wait"):
        B.checkAsyncError()
    B.checkAsyncError()                                     # reported once, then clear again
    assert _gemm_ok(B)                                      # tensor memory came back; tcgen05 work still runs
    # 512 columns per SM are needed by the paired GEMM: a leak in the probe would make this wait
    x = B.upload(np.ones((4096, 1024), np.float32), "bf16")
    y = B.matmulTransposed(x, x)
    assert float(y.data[0, 0]) == 1024.0
    B.checkAsyncError()


def test_probe_rejects_limits_outside_its_range(B):
    left = C.c_int(0)
    assert B.lib.alpha_debug_wait_expiry(1, 0, C.byref(left)) != 0
    assert B.lib.alpha_debug_wait_expiry(1, 10 ** 6, C.byref(left)) != 0
    assert B.lib.alpha_debug_wait_expiry(0, 100, C.byref(left)) != 0
    B.checkAsyncError()
