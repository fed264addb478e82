"""mxb200: the MXFP8 Linear path of nanochat-cpp (quantizer, block-scaled GEMM and their callers) on B200.

``capi`` binds the C-ABI library ``libmxb200.so`` (include/mxb200.h); ``engine`` mirrors the reference's host
interface (src/nanochat/model/fp8/fp8.h, mx_gemm.h) over it; ``dp_step`` is the data-parallel step."""
from .engine import *  # noqa: F401,F403
from . import capi, engine  # noqa: F401
