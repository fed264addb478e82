"""Door to nanochat-cpp's own host engine built against libmxb200.so (oracle/_ref/nanochat_refhost.so, made by
oracle/refhost/Makefile from the unmodified reference sources plus the GEMM seam of oracle/refhost/b200_seam.cpp).
A checker for GPU tests; absent when the reference tree was not available at build time."""
from __future__ import annotations

import importlib.util
import os

_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "nanochat_refhost.so")
_mod = None


def available() -> bool:
    return os.path.exists(_PATH)


def module():
    global _mod
    if _mod is None:
        import torch  # noqa: F401  (libtorch must be loaded first)
        import nanochat_cpp_b200  # noqa: F401  (and libmxb200.so, which the module links)
        spec = importlib.util.spec_from_file_location("nanochat_refhost", _PATH)
        _mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(_mod)
    return _mod
