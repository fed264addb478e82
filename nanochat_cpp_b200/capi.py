"""ctypes binding of libmxb200.so, one function per entry point of include/mxb200.h.

The library is the product; this module only loads it and declares signatures. There is no fallback: if the
library is missing it is built with nvcc, and if that fails the import raises.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmxb200.so")

OK = 0
ERR_SHAPE, ERR_ALIGNMENT, ERR_NULL, ERR_ARGUMENT, ERR_WORKSPACE, ERR_DEVICE, ERR_DRIVER, ERR_LAUNCH, ERR_WATCHDOG = range(1, 10)
SCALE_REFERENCE, SCALE_OCP_FLOOR = 0, 1
PROLOGUE_NONE, PROLOGUE_RELU_SQUARE = 0, 1
OUT_BF16, OUT_F32 = 0, 1
STATIC_SCRATCH_BYTES = 32 << 20

# every symbol include/mxb200.h declares
SYMBOLS = (
    "mxb200_quantize_mx", "mxb200_quantize_mx_batch", "mxb200_quantize_mx_relu_square_bwd", "mxb200_gemm_bf16", "mxb200_gemm_f32",
    "mxb200_gemm_relu_square", "mxb200_gemm_relu_square_bwd", "mxb200_residual_norm_mx_fwd",
    "mxb200_softcap_ce_loss", "mxb200_softcap_ce_grad_mx",
    "mxb200_gemm_splits", "mxb200_gemm_workspace_bytes", "mxb200_gemm_splitk", "mxb200_gemm_splitk_static",
    "mxb200_strerror",
    "mxb200_device_status", "mxb200_selftest_bounded_wait", "mxb200_set_gemm_config", "mxb200_launch_count", "mxb200_version",
)


class MxOut(ctypes.Structure):
    """mxb200_mx_out / nanochat::kernels::MxOut."""
    _fields_ = [("data", ctypes.c_void_p), ("ld", ctypes.c_int64), ("scale", ctypes.c_void_p),
                ("scale_tiles", ctypes.c_int64)]


class QuantizeJob(ctypes.Structure):
    """mxb200_quantize_job."""
    _fields_ = [("x", ctypes.c_void_p), ("rows", ctypes.c_int64), ("cols", ctypes.c_int64), ("out", MxOut),
                ("out_t", MxOut)]


class ResidualNormMx(ctypes.Structure):
    """mxb200_residual_norm_mx."""
    _fields_ = [("x", ctypes.c_void_p), ("r", ctypes.c_void_p), ("x0", ctypes.c_void_p), ("lr", ctypes.c_void_p),
                ("l0", ctypes.c_void_p), ("s", ctypes.c_void_p), ("res", ctypes.c_void_p), ("n", ctypes.c_void_p),
                ("rstd", ctypes.c_void_p), ("rows", ctypes.c_int64), ("cols", ctypes.c_int32), ("eps", ctypes.c_float),
                ("out", MxOut), ("out_t", MxOut), ("n_cols", ctypes.c_int32)]


class Mxb200Error(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(f"{what}: {strerror(status)} (status {status})")


def _load() -> ctypes.CDLL:
    from .build import build, have_nvcc
    if not os.path.exists(LIB_PATH) or have_nvcc():
        build()  # returns at once unless a source is newer than the library: an edited kernel never runs stale
    lib = ctypes.CDLL(LIB_PATH)
    vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    lib.mxb200_quantize_mx.argtypes = [vp, i32, i64, i64, MxOut, MxOut, i32, i32, vp]
    lib.mxb200_quantize_mx_batch.argtypes = [ctypes.POINTER(QuantizeJob), i32, i32, i32, vp]
    lib.mxb200_quantize_mx_relu_square_bwd.argtypes = [vp, vp, i64, i64, MxOut, MxOut, i32, vp]
    lib.mxb200_gemm_bf16.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, vp]
    lib.mxb200_gemm_f32.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, vp, i32, vp]
    lib.mxb200_gemm_relu_square.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, vp]
    lib.mxb200_gemm_relu_square_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, vp]
    lib.mxb200_residual_norm_mx_fwd.argtypes = [ctypes.POINTER(ResidualNormMx), vp]
    f32 = ctypes.c_float
    lib.mxb200_softcap_ce_loss.argtypes = [vp, i64, i64, vp, i32, i32, f32, vp, vp, vp]
    lib.mxb200_softcap_ce_grad_mx.argtypes = [vp, i64, i64, vp, vp, i32, i32, f32, vp, i64, vp, MxOut, MxOut, i32, vp]
    lib.mxb200_gemm_splits.argtypes = [i64, i64, i64]
    lib.mxb200_gemm_workspace_bytes.argtypes = [i64, i64, i64, i32]
    lib.mxb200_gemm_workspace_bytes.restype = ctypes.c_size_t
    lib.mxb200_gemm_splitk.argtypes = [vp, vp, vp, vp, vp, i32, vp, i64, i64, i64, vp, i32, i32, vp, ctypes.c_size_t, vp]
    lib.mxb200_gemm_splitk_static.argtypes = [vp, vp, vp, vp, vp, i32, vp, i64, i64, i64, vp, i32, i32, vp]
    lib.mxb200_selftest_bounded_wait.argtypes = [ctypes.c_uint64, vp]
    lib.mxb200_strerror.argtypes = [i32]
    lib.mxb200_strerror.restype = ctypes.c_char_p
    lib.mxb200_device_status.argtypes = [ctypes.POINTER(ctypes.c_uint32)]
    lib.mxb200_set_gemm_config.argtypes = [i32, i32]
    lib.mxb200_launch_count.restype = ctypes.c_uint64
    for name in SYMBOLS:
        fn = getattr(lib, name)
        if fn.restype is ctypes.c_int and name not in ("mxb200_strerror",):
            fn.restype = ctypes.c_int
    return lib


lib = _load()


def strerror(status: int) -> str:
    return lib.mxb200_strerror(status).decode()


def check(status: int, what: str) -> None:
    if status != OK:
        raise Mxb200Error(status, what)


def launch_count() -> int:
    return int(lib.mxb200_launch_count())


def device_status() -> int:
    """Synchronises; returns the watchdog word (0 = no bounded wait ran out) and clears it."""
    w = ctypes.c_uint32(0)
    lib.mxb200_device_status(ctypes.byref(w))
    return int(w.value)
