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


def residual_norm_inputs(rows: int, cols: int, add: bool, blend: bool, seed: int = 0) -> dict:
    """Inputs of the fused residual step as nanochat-cpp's test draws them (tests/test_residual_norm.cpp:80-97):
    unit-normal bf16 x whose first row is scaled by 1e-4 (a tiny row, where eps matters), r at half that spread,
    five fp32 lambdas per kind, lr in [0.5, 1.5) and l0 in [0, 0.3), layer 3. CPU tensors."""
    g = torch.Generator().manual_seed(seed + 7 * rows + cols)
    x = torch.randn(rows, cols, generator=g).to(torch.bfloat16)
    x[0] = (x[0].float() * 1e-4).to(torch.bfloat16)
    r = (torch.randn(rows, cols, generator=g) * 0.5).to(torch.bfloat16) if add else None
    x0 = torch.randn(rows, cols, generator=g).to(torch.bfloat16) if blend else None
    lr = (torch.rand(5, generator=g) + 0.5) if blend else None
    l0 = (torch.rand(5, generator=g) * 0.3) if blend else None
    return {"x": x, "r": r, "x0": x0, "lr": lr, "l0": l0, "layer": 3}
