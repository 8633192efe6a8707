"""ctypes binding of libalpha_cuda.so (the C ABI declared in include/alpha_cuda.h).

This is the Python twin of the FFI stub a TypeScript host would write with bun:ffi.  The
library is built in-tree by ``python -m alpha2_b200.build``; loading fails loudly when it is
missing, and ``alpha_init`` fails loudly when no B200 is visible — there is no CPU path.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(HERE, "libalpha_cuda.so")

F32, BF16, I32 = 0, 1, 2
DTYPE_CODE = {"f32": F32, "bf16": BF16, "i32": I32}
DTYPE_SIZE = {"f32": 4, "bf16": 2, "i32": 4}

ADD, SUB, MUL, DIV = 0, 1, 2, 3
NEG, EXP, LOG, SQRT, RELU, SILU, GELU, SCALE, CLAMP, POW, SOFTCAP = range(11)
GEMM_NT, GEMM_NN, GEMM_TN = 0, 1, 2
EPI_NONE, EPI_GELU, EPI_ADD, EPI_GELU_BWD = 0, 1, 2, 3


class AlphaCudaError(RuntimeError):
    pass


class DeviceInfo(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("vendor_id", C.c_int32), ("sm_count", C.c_int32),
                ("cc_major", C.c_int32), ("cc_minor", C.c_int32), ("total_mem", C.c_uint64),
                ("l2_bytes", C.c_uint64)]


class MemStats(C.Structure):
    _fields_ = [("bytes_in_use", C.c_uint64), ("bytes_cached", C.c_uint64), ("peak_in_use", C.c_uint64),
                ("n_device_mallocs", C.c_uint64), ("n_allocs", C.c_uint64)]


class AttnParams(C.Structure):
    _fields_ = [("batch", C.c_int64), ("heads", C.c_int64), ("T", C.c_int64), ("D", C.c_int64),
                ("q_sb", C.c_int64), ("q_sh", C.c_int64), ("q_st", C.c_int64),
                ("o_sb", C.c_int64), ("o_sh", C.c_int64), ("o_st", C.c_int64),
                ("scale", C.c_float), ("soft_cap", C.c_float), ("dtype", C.c_int32)]


class AdamWTensor(C.Structure):
    _fields_ = [("p", C.c_uint64), ("g", C.c_uint64), ("m", C.c_uint64), ("v", C.c_uint64),
                ("p_shadow", C.c_uint64), ("n", C.c_int64), ("weight_decay", C.c_float),
                ("grad_dtype", C.c_int32)]


class ProfileEntry(C.Structure):
    _fields_ = [("ms", C.c_double), ("work", C.c_double), ("launches", C.c_int64)]


PROFILE_CATEGORIES = ["gemm_tc", "gemm_f32", "attn_fwd", "attn_bwd", "cross_entropy", "adamw", "norm", "embedding",
                      "elementwise"]


class HostRng(C.Structure):
    _fields_ = [("s0", C.c_uint32), ("s1", C.c_uint32), ("has_spare", C.c_int32), ("spare", C.c_double)]


_B, _I, _L, _F, _P = C.c_uint64, C.c_int, C.c_int64, C.c_float, C.c_void_p
_PL = C.POINTER(C.c_int64)

# name -> argtypes; every entry returns int status unless listed in _OTHER_RESTYPE.
SIGNATURES = {
    "alpha_init": [_I], "alpha_shutdown": [], "alpha_device_info": [C.POINTER(DeviceInfo)],
    "alpha_stream_sync": [], "alpha_launch_count": [C.POINTER(C.c_uint64)],
    "alpha_stream_handle": [C.POINTER(C.c_uint64)], "alpha_check_async_error": [],
    "alpha_debug_wait_expiry": [_I, _I, C.POINTER(C.c_int)],
    "alpha_range_push": [C.c_char_p], "alpha_range_pop": [],
    "alpha_profile_enable": [_I], "alpha_profile_read": [C.POINTER(ProfileEntry), _I],
    "alpha_event_create": [C.POINTER(C.c_uint64)], "alpha_event_record": [_B], "alpha_event_sync": [_B],
    "alpha_event_elapsed_ms": [_B, _B, C.POINTER(C.c_float)], "alpha_event_destroy": [_B],
    "alpha_alloc": [C.c_size_t, C.POINTER(C.c_uint64)], "alpha_free": [_B],
    "alpha_mem_stats": [C.POINTER(MemStats)], "alpha_purge_pools": [],
    "alpha_memset": [_B, _I, C.c_size_t], "alpha_h2d": [_B, _P, C.c_size_t], "alpha_d2h": [_P, _B, C.c_size_t],
    "alpha_d2h_async": [_P, _B, C.c_size_t],
    "alpha_d2d": [_B, _B, C.c_size_t], "alpha_host_alloc": [C.c_size_t, C.POINTER(C.c_void_p)],
    "alpha_host_free": [_P],
    "alpha_fill": [_B, _L, _F, _I], "alpha_binary": [_I, _B, _B, _B, _L, _I],
    "alpha_binary_bcast": [_I, _B, _B, _B, _I, _PL, _PL, _PL, _I],
    "alpha_unary": [_I, _B, _B, _L, _F, _F, _I], "alpha_unary_bwd": [_I, _B, _B, _B, _L, _F, _F, _I],
    "alpha_add_inplace": [_B, _B, _L, _I, _I], "alpha_scale_inplace": [_B, _F, _L, _I],
    "alpha_cast": [_B, _I, _B, _I, _L], "alpha_silu_mul_fwd": [_B, _B, _B, _L, _I],
    "alpha_silu_mul_bwd": [_B, _B, _B, _B, _B, _L, _I], "alpha_broadcast": [_B, _B, _I, _PL, _PL, _I],
    "alpha_sum_axis": [_B, _B, _L, _L, _L, _F, _I], "alpha_softmax": [_B, _B, _L, _L, _I, _I],
    "alpha_sumsq_multi": [C.POINTER(C.c_uint64), _PL, C.POINTER(C.c_int32), _I, _B],
    "alpha_check_finite": [_B, _L, _I, _B],
    "alpha_transpose": [_B, _B, _I, _PL, _I, _I, _I], "alpha_slice_cols": [_B, _B, _L, _L, _L, _L, _I],
    "alpha_scatter_cols": [_B, _B, _L, _L, _L, _L, _I], "alpha_slice_qkv": [_B, _B, _B, _B, _L, _L, _I],
    "alpha_causal_mask": [_B, _L], "alpha_masked_fill": [_B, _B, _B, _L, _L, _F, _I],
    "alpha_dropout_mask": [_B, _L, C.c_int32, C.c_int32, _F, _I],
    "alpha_residual_dropout_add": [_B, _B, _B, _B, _L, _I],
    "alpha_embedding_fwd": [_B, _B, _B, _L, _L, _L, _I],
    "alpha_embedding_pos_fwd": [_B, _B, _B, _B, _L, _L, _L, _L, _I],
    "alpha_embedding_bwd": [_B, _B, _B, _L, _L, _L, _I, _I],
    "alpha_layernorm_fwd": [_B, _B, _B, _B, _L, _L, _F, _I],
    "alpha_layernorm_bwd": [_B, _B, _B, _B, _B, _B, _L, _L, _F, _I, _I, _B],
    "alpha_rmsnorm_fwd": [_B, _B, _B, _L, _L, _F, _I],
    "alpha_rmsnorm_bwd": [_B, _B, _B, _B, _B, _L, _L, _F, _I, _I, _B],
    "alpha_gemm": [_I, _B, _B, _B, _L, _L, _L, _L, _L, _L, _I, _I, _I, _B, _L, _I],
    "alpha_gemm_nn_rowdot": [_B, _B, _B, _L, _L, _L, _L, _L, _L, _B, _L, _B, _L, _L],
    "alpha_gemm_tn_pair": [_B, _B, _B, _L, _L, _L, _L, _L, _I, _B, _B, _B, _L, _L, _L, _L, _L, _I, _L],
    "alpha_flash_attn_bwd_delta": [_B, _B, _B, _B, _B, _B, _B, _B, _B, C.POINTER(AttnParams)],
    "alpha_gemm_batched_f32": [_I, _B, _B, _B, _L, _L, _L, _L, _L, _L, _L, _L, _L, _L],
    "alpha_flash_attn_fwd": [_B, _B, _B, _B, _B, C.POINTER(AttnParams)],
    "alpha_flash_attn_bwd": [_B, _B, _B, _B, _B, _B, _B, _B, _B, C.POINTER(AttnParams)],
    "alpha_rope": [_B, _B, _L, _L, _L, _L, _L, _F, _I, _I],
    "alpha_set_launch_overlap": [_I],
    "alpha_rope_qkv": [_B, _B, _L, _L, _L, _L, _F, _I, _I],
    "alpha_cross_entropy_fwd": [_B, _B, _B, _L, _L, _L, _I],
    "alpha_cross_entropy_fwd_noalloc": [_B, _B, _B, _L, _L, _L, _I],
    "alpha_cross_entropy_bwd": [_B, _B, _B, _B, _L, _L, _L, _I],
    "alpha_softmax_ce_fwd_bwd": [_B, _B, _B, _B, _L, _L, _L, _F, _I],
    "alpha_adamw": [_B, _B, _B, _B, _L, _F, _F, _F, _F, _F, _F, _F, _F, _I, _B],
    "alpha_adamw_multi": [C.POINTER(AdamWTensor), _I, _F, _F, _F, _F, _F, _F, _F, _B, _F],
    "alpha_comm_unique_id": [_P], "alpha_comm_init_rank": [_I, _I, _P],
    "alpha_comm_allreduce_sum": [_B, _L, _I], "alpha_comm_wait": [], "alpha_comm_destroy": [],
    "alpha_comm_query": [C.POINTER(C.c_int), C.POINTER(C.c_int)], "alpha_comm_abort": [],
    "alpha_comm_allreduce_sum_bucket": [C.POINTER(C.c_uint64), _PL, _I, _I],
    "alpha_rng_seed": [C.POINTER(HostRng), C.c_uint32],
    "alpha_rng_fill_gauss": [C.POINTER(HostRng), _P, _L, C.c_double],
}
_OTHER_RESTYPE = {"alpha_last_error": ([], C.c_char_p), "alpha_rng_next": ([C.POINTER(HostRng)], C.c_double),
                  "alpha_rng_gauss": ([C.POINTER(HostRng)], C.c_double)}

_lib = None


def load():
    """Load libalpha_cuda.so and bind every entry point.  Raises if the library is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(SO_PATH):
        raise AlphaCudaError(
            f"{SO_PATH} is missing: build it with `python -m alpha2_b200.build` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback.")
    L = C.CDLL(SO_PATH, mode=C.RTLD_GLOBAL)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(L, name)
        fn.argtypes = argtypes
        fn.restype = C.c_int
    for name, (argtypes, restype) in _OTHER_RESTYPE.items():
        fn = getattr(L, name)
        fn.argtypes = argtypes
        fn.restype = restype
    _lib = L
    return L


def exported_names():
    return list(SIGNATURES) + list(_OTHER_RESTYPE)


def check(status: int) -> None:
    if status != 0:
        raise AlphaCudaError(load().alpha_last_error().decode("utf-8", "replace"))
