"""The reference's CPU-expressible formulation of the MXFP8 Linear path.

Test infrastructure and CPU baseline only; the product never imports this.

nanochat-cpp checks its CUDA kernels against a handful of torch-op helpers
(tests/test_fp8.cpp:25-49: ``mx_reference``, ``swizzle``, ``mx_dequantize``)
followed by ``torch::mm``. Those helpers run on any device, so on CPU they are
the reference's own CPU path: libtorch quantize -> dequantize -> fp32 matmul.
This file states the same op sequence through the Python front end of the
same libtorch kernels. It serves two purposes: it pins ``oracle/mx_oracle.py``
(the numpy restatement must agree bit for bit), and it is what the benchmark
times on the host cores as the reference arm.
"""
from __future__ import annotations

import torch


def mx_reference(x: torch.Tensor):
    """x (R, C) -> (e4m3 data (R, C), biased e8m0 exponents (R, C/32) uint8).
    tests/test_fp8.cpp:25-35."""
    R, C = x.shape
    b = x.to(torch.float32).view(R, C // 32, 32)
    amax_bits = b.abs().amax(-1).view(torch.int32)
    e = (torch.bitwise_right_shift(amax_bits, 23) - 8
         + (amax_bits.bitwise_and(0x7FFFFF) > 0x600000)).clamp(0, 253).to(torch.int32)
    mult = torch.bitwise_left_shift(254 - e, 23).to(torch.int32).view(torch.float32)
    return (b * mult.unsqueeze(-1)).to(torch.float8_e4m3fn).view(R, C), e.to(torch.uint8)


def swizzle(s: torch.Tensor) -> torch.Tensor:
    """tests/test_fp8.cpp:37-41."""
    R, B = s.shape
    return s.view(R // 128, 4, 32, B // 4, 4).permute(0, 3, 2, 1, 4).reshape(-1)


def mx_dequantize(data: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """tests/test_fp8.cpp:43-49."""
    R, C = data.shape
    e = scale.view(torch.uint8).view(R // 128, C // 128, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(R, C // 32)
    mult = torch.pow(2.0, e.to(torch.float32) - 127)
    return (data.to(torch.float32).view(R, C // 32, 32) * mult.unsqueeze(-1)).view(R, C)


def quantize_mx(x: torch.Tensor, rows: bool = True, cols: bool = True, relu_square: bool = False) -> dict:
    """Both layouts, as tests/test_fp8.cpp:170-172 builds the expectation."""
    src = torch.relu(x).square() if relu_square else x
    out = {}
    if rows:
        d, e = mx_reference(src)
        out["data"], out["scale"] = d, swizzle(e)
    if cols:
        d, e = mx_reference(src.t().contiguous())
        out["data_t"], out["scale_t"] = d, swizzle(e)
    return out


def linear_forward(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor | None = None) -> torch.Tensor:
    """quantize -> dequantize -> fp32 mm -> bf16 (tests/test_fp8.cpp:202-206);
    the optional residual add rounds twice, as
    src/nanochat/model/ops/residual_norm_kernel.cu:96-104."""
    xq, wq = quantize_mx(x, True, False), quantize_mx(w, True, False)
    y = torch.mm(mx_dequantize(xq["data"], xq["scale"]), mx_dequantize(wq["data"], wq["scale"]).t()).to(torch.bfloat16)
    if resid is not None:
        y = (y.float() + resid.float()).to(torch.bfloat16)
    return y


def linear_backward(x: torch.Tensor, w: torch.Tensor, dy: torch.Tensor):
    """dX = deq(dY) . deq(W_t)^T and dW = deq(dY_t) . deq(X_t)^T
    (tests/test_fp8.cpp:207-208)."""
    xq, wq, gq = quantize_mx(x, False, True), quantize_mx(w, False, True), quantize_mx(dy, True, True)
    dx = torch.mm(mx_dequantize(gq["data"], gq["scale"]), mx_dequantize(wq["data_t"], wq["scale_t"]).t())
    dw = torch.mm(mx_dequantize(gq["data_t"], gq["scale_t"]), mx_dequantize(xq["data_t"], xq["scale_t"]).t())
    return dx.to(torch.bfloat16), dw
