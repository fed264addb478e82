"""Seeded inputs shared by the parity tests: the distributions and edge cases nanochat-cpp's own tests use
(tests/test_fp8.cpp:156-163, 184-190, 328-335), drawn on the CPU."""
from __future__ import annotations

import numpy as np
import torch

from oracle import mx_oracle as mo


def quantizer_input(rows: int, cols: int, seed: int = 0) -> torch.Tensor:
    """Magnitudes from 1e-6 to 1e6 across columns, a zero block, a block whose maximum has a mantissa above
    1.75 (tests/test_fp8.cpp:159-163). fp32."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g) * torch.logspace(-6, 6, cols)
    x[0:1, 0:32] = 0
    x[1, 40] = 448 * 1.8
    return x


def gemm_operands(M: int, N: int, K: int, seed: int = 0):
    """a with magnitudes 1e-2..1e2 across K, b ~ N(0,1), both bf16 (tests/test_fp8.cpp:333-334)."""
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(M, K, generator=g) * torch.logspace(-2, 2, K)).to(torch.bfloat16)
    b = torch.randn(N, K, generator=g).to(torch.bfloat16)
    return a, b


def np_f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().to(torch.float32).cpu().numpy()


def np_u8(t: torch.Tensor) -> np.ndarray:
    return t.detach().view(torch.uint8).cpu().numpy()


def oracle_quantize(x: torch.Tensor, rows=True, cols=True, prologue=0, h=None, rule=0) -> dict:
    return mo.quantize_mx(np_f32(x), rows, cols, prologue, None if h is None else np_f32(h), rule)


def assert_quantized_equal(q, want: dict, what: str = ""):
    """q: engine Fp8Tensor on the GPU; want: oracle dict. Bit-exact."""
    pairs = [("data", q.data), ("scale", q.inv_scale), ("data_t", q.data_t), ("scale_t", q.inv_scale_t)]
    for key, got in pairs:
        if key not in want:
            assert got is None
            continue
        g = np_u8(got).reshape(-1)
        w = want[key].reshape(-1)
        bad = int((g != w).sum())
        assert bad == 0, f"{what} {key}: {bad} of {g.size} bytes differ (first at {int(np.argmax(g != w))})"
