"""ctypes binding of ``libb200dq.so`` (the C ABI in ``include/b200dq.h``).

Mirrors how the reference's ctypes/Cython adapters drive a compiled kernel
library: ``lib.init()``, ``lib.call(...)``, ``lib.get_last_error()``
(tilelang/jit/adapter/cython/adapter.py:135-139, 338-345). There is no fallback:
a missing library or a failing call raises.
"""
from __future__ import annotations

import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200dq.so")

# enum values of include/b200dq.h
WF_U4_SZ, WF_U4_RAW, WF_S4_RAW, WF_FP4_E8M0, WF_I2_I8, WF_I4_I8, WF_U2_SZ, WF_LUT4_S = range(8)
ACT_F16, ACT_BF16, ACT_I8 = range(3)
OUT_F16, OUT_BF16, OUT_F32, OUT_I32 = range(4)
GF_TRANS_C, GF_HAS_BIAS, GF_ROW_SCALE, GF_FP4_SIMPLE = 1, 2, 4, 16

EXPORTED_SYMBOLS = (
    "b200dq_init",
    "b200dq_get_last_error",
    "b200dq_version",
    "b200dq_gemm",
    "b200dq_gemm_static_scratch",
    "b200dq_gemm_workspace_bytes",
    "b200dq_gemm_workspace_bytes_for",
    "b200dq_static_scratch_check",
    "b200dq_packed_weight_bytes",
    "b200dq_pack_weights",
    "b200dq_check_status",
    "b200dq_absmax_quant_int8",
    "b200dq_quant_mxfp4",
    "b200dq_gemm_mxfp4_native",
    "b200dq_tensor_peak",
    "b200dq_grouped_prefixes",
    "b200dq_silu_mul",
    "b200dq_unpack_int4_to_int8",
    "b200dq_moe_combine",
)


ABI_VERSION = 5      # b200dq_version(): layout of struct b200dq_gemm_args


class GemmArgs(ctypes.Structure):
    """``struct b200dq_gemm_args``."""

    _fields_ = [
        ("a", ctypes.c_void_p),
        ("wp", ctypes.c_void_p),
        ("bias", ctypes.c_void_p),
        ("row_scale", ctypes.c_void_p),
        ("c", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("M", ctypes.c_int32),
        ("N", ctypes.c_int32),
        ("K", ctypes.c_int32),
        ("group_size", ctypes.c_int32),
        ("weight_format", ctypes.c_int32),
        ("act_type", ctypes.c_int32),
        ("out_type", ctypes.c_int32),
        ("flags", ctypes.c_int32),
        ("tensor_scale", ctypes.c_float),
        ("code_bias", ctypes.c_uint32),
        ("fp4_exp_bias", ctypes.c_int32),
        ("token_tile", ctypes.c_int32),
        ("max_ctas", ctypes.c_int32),
        ("group_row_prefix", ctypes.c_void_p),
        ("group_tile_prefix", ctypes.c_void_p),
        ("group_weight_stride", ctypes.c_int64),
        ("num_groups", ctypes.c_int32),
        ("total_tiles", ctypes.c_int32),
        ("c_peers", ctypes.c_void_p * 7),
        ("num_peers", ctypes.c_int32),
        ("code_table", ctypes.c_float * 16),
    ]


class B200dqError(RuntimeError):
    pass


_lock = threading.Lock()
_lib = None


def _declare(lib):
    i32, vp, sz = ctypes.c_int32, ctypes.c_void_p, ctypes.c_size_t
    lib.b200dq_init.restype = ctypes.c_int
    lib.b200dq_init.argtypes = []
    lib.b200dq_get_last_error.restype = ctypes.c_char_p
    lib.b200dq_get_last_error.argtypes = []
    lib.b200dq_version.restype = ctypes.c_int
    lib.b200dq_version.argtypes = []
    lib.b200dq_gemm.restype = ctypes.c_int
    lib.b200dq_gemm.argtypes = [ctypes.POINTER(GemmArgs), vp]
    lib.b200dq_gemm_static_scratch.restype = ctypes.c_int
    lib.b200dq_gemm_static_scratch.argtypes = [ctypes.POINTER(GemmArgs), vp]
    lib.b200dq_gemm_workspace_bytes.restype = sz
    lib.b200dq_gemm_workspace_bytes.argtypes = [i32, i32, i32, i32, i32, i32, i32]
    lib.b200dq_gemm_workspace_bytes_for.restype = sz
    lib.b200dq_gemm_workspace_bytes_for.argtypes = [ctypes.POINTER(GemmArgs)]
    lib.b200dq_static_scratch_check.restype = ctypes.c_int
    lib.b200dq_static_scratch_check.argtypes = [ctypes.POINTER(GemmArgs), i32, ctypes.POINTER(sz), ctypes.POINTER(sz)]
    lib.b200dq_packed_weight_bytes.restype = sz
    lib.b200dq_packed_weight_bytes.argtypes = [i32, i32, i32, i32]
    lib.b200dq_pack_weights.restype = ctypes.c_int
    lib.b200dq_pack_weights.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]
    lib.b200dq_absmax_quant_int8.restype = ctypes.c_int
    lib.b200dq_absmax_quant_int8.argtypes = [vp, vp, vp, i32, i32, i32, vp]
    lib.b200dq_quant_mxfp4.restype = ctypes.c_int
    lib.b200dq_quant_mxfp4.argtypes = [vp, vp, vp, i32, i32, i32, i32, vp]
    lib.b200dq_grouped_prefixes.restype = ctypes.c_int
    lib.b200dq_grouped_prefixes.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp]
    lib.b200dq_tensor_peak.restype = ctypes.c_int
    lib.b200dq_tensor_peak.argtypes = [i32, i32, ctypes.POINTER(ctypes.c_double), vp]
    lib.b200dq_gemm_mxfp4_native.restype = ctypes.c_int
    lib.b200dq_gemm_mxfp4_native.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, vp]
    lib.b200dq_silu_mul.restype = ctypes.c_int
    lib.b200dq_silu_mul.argtypes = [vp, vp, ctypes.c_int64, i32, i32, vp]
    lib.b200dq_unpack_int4_to_int8.restype = ctypes.c_int
    lib.b200dq_unpack_int4_to_int8.argtypes = [vp, vp, ctypes.c_int64, vp]
    lib.b200dq_moe_combine.restype = ctypes.c_int
    lib.b200dq_moe_combine.argtypes = [vp, vp, vp, vp, ctypes.c_int64, i32, i32, i32, vp]
    lib.b200dq_check_status.restype = ctypes.c_int
    lib.b200dq_check_status.argtypes = [vp]


def load(path: str | None = None):
    """Load the shared library (once). Raises if it has not been built."""
    global _lib
    with _lock:
        if _lib is None:
            p = path or LIB_PATH
            if not os.path.exists(p):
                raise B200dqError(
                    f"{p} is missing: build it with `python -m tilelang_b200.build` "
                    "(there is no CPU or PyTorch fallback)"
                )
            lib = ctypes.CDLL(p)
            _declare(lib)
            if lib.b200dq_version() != ABI_VERSION:
                raise B200dqError(f"{p} has ABI version {lib.b200dq_version()}, this package expects {ABI_VERSION}: "
                                  "rebuild it with `python -m tilelang_b200.build`")
            _lib = lib
        return _lib


def last_error() -> str:
    return load().b200dq_get_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise B200dqError(f"{what}: {last_error()}")
