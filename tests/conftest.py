import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu")


def _has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] == 10
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no sm_100 GPU here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle_c():
    """The plain-C oracle, built on demand."""
    import ctypes
    import subprocess
    path = os.path.join(ROOT, "oracle", "libmx_oracle.so")
    src = os.path.join(ROOT, "oracle", "mx_oracle.c")
    if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
        subprocess.check_call(["gcc", "-O2", "-fPIC", "-shared", "-ffp-contract=off", "-o", path, src, "-lm"])
    lib = ctypes.CDLL(path)
    lib.mxo_round_bf16.restype = ctypes.c_float
    lib.mxo_round_bf16.argtypes = [ctypes.c_float]
    lib.mxo_bf16_out.restype = ctypes.c_float
    lib.mxo_bf16_out.argtypes = [ctypes.c_float, ctypes.c_int, ctypes.c_float]
    lib.mxo_e4m3.restype = ctypes.c_uint8
    lib.mxo_e4m3.argtypes = [ctypes.c_float]
    lib.mxo_exponent.argtypes = [ctypes.c_float, ctypes.c_int]
    lib.mxo_scale_index.restype = ctypes.c_int64
    lib.mxo_scale_index.argtypes = [ctypes.c_int64] * 3
    vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    lib.mxo_quantize.argtypes = [vp, vp, i64, i64, i32, i32, i32, vp, i64, vp, i64]
    lib.mxo_dequantize.argtypes = [vp, vp, i64, i64, vp]
    lib.mxo_gemm_f32.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, ctypes.c_float, i32]
    lib.mxo_softcap_ce_loss.argtypes = [vp, i64, i64, vp, i32, i32, ctypes.c_float, vp, vp]
    lib.mxo_softcap_ce_grad.argtypes = [vp, i64, i64, vp, vp, i32, i32, ctypes.c_float, vp, i64, i64, vp]
    lib.mxo_residual_norm.argtypes = [vp, vp, vp, ctypes.c_float, ctypes.c_float, i64, i32, ctypes.c_float, vp, vp, vp, vp, vp]
    return lib
