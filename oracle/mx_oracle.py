"""CPU oracle for the MXFP8 Linear path: test infrastructure, never the product.

A numpy restatement of nanochat-cpp's MX quantizer and block-scaled GEMM
semantics. Only tests, the smoke check and the CPU-baseline leg of the
benchmark may import this module; the product path is the CUDA library and
fails loudly when that is missing.

Each function cites the reference lines it restates (paths are relative to
the nanochat-cpp repository root).

Parity pin: the reference holds no stored vectors for MX. This oracle is
pinned (a) against the reference's own torch-op test oracle restated in
``oracle/torch_reference.py`` (tests/test_fp8.cpp:25-49), run on CPU, and
(b) against ``tests/golden/*.npz``: bytes written by the reference's own CUDA
quantizer kernel (src/nanochat/model/fp8/fp8_kernel.cu, compiled unmodified
for sm_100 from the reference tree) on a B200.
"""
from __future__ import annotations

import numpy as np

BLOCK = 32          # values per E8M0 scale (src/nanochat/model/fp8/fp8_kernel.h:26)
SCALE_RULE_REFERENCE = 0   # 2^ceil(log2(amax/448)), the reference's rule
SCALE_RULE_OCP_FLOOR = 1   # 2^(floor(log2(amax)) - 8), saturating

PROLOGUE_NONE = 0
PROLOGUE_RELU_SQUARE = 1
PROLOGUE_RELU_SQUARE_BWD = 2


# --------------------------------------------------------------------------- bf16 helpers

def round_bf16(x: np.ndarray) -> np.ndarray:
    """fp32 -> nearest-even bf16, returned as fp32 (what __float2bfloat16 then
    __bfloat162float give; src/nanochat/model/fp8/fp8_kernel.cu:44-50)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    nan = np.isnan(x)
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    rounded = np.where(nan, 0x7FFF0000, rounded).astype(np.uint32)
    return rounded.view(np.float32).reshape(x.shape)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    return (round_bf16(x).view(np.uint32) >> 16).astype(np.uint16)


# --------------------------------------------------------------------------- scale arithmetic

def mx_exponent(amax: np.ndarray, rule: int = SCALE_RULE_REFERENCE) -> np.ndarray:
    """Biased E8M0 byte for a block maximum.

    Reference rule (src/nanochat/model/fp8/mx_kernel.cuh:29-34,
    tests/test_fp8.cpp:29-32): e = (bits >> 23) - 8 + (mantissa > 0x600000),
    clamped to [0, 253]; integer arithmetic on the float's bits.
    ``SCALE_RULE_OCP_FLOOR`` drops the mantissa bump."""
    bits = np.ascontiguousarray(amax, dtype=np.float32).view(np.uint32).astype(np.int64)
    e = (bits >> 23) - 8
    if rule == SCALE_RULE_REFERENCE:
        e = e + ((bits & 0x7FFFFF) > 0x600000)
    return np.clip(e, 0, 253).astype(np.int32).reshape(np.shape(amax))


def mx_multiplier(e: np.ndarray) -> np.ndarray:
    """2^(127 - e) exactly, built from bits (src/nanochat/model/fp8/mx_kernel.cuh:37-39)."""
    return ((254 - np.asarray(e, dtype=np.int64)).astype(np.uint32) << 23).view(np.float32)


def e4m3_from_f32(x: np.ndarray) -> np.ndarray:
    """fp32 -> E4M3 byte, round-to-nearest-even, saturating to +-448, NaN -> 0x7f.

    What ``__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3)`` gives
    (src/nanochat/model/fp8/mx_kernel.cuh:61)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    sign = (x.view(np.uint32) >> 31).astype(np.uint8) << 7
    a = np.abs(x).astype(np.float64)
    nan = np.isnan(a)
    a = np.where(nan, 0.0, np.minimum(a, 448.0))
    # quantum: 2^-9 below the smallest normal 2^-6, else 2^(floor(log2 a) - 3)
    _, ex = np.frexp(a)                       # a = m * 2^ex, m in [0.5, 1)
    fl = ex - 1                               # floor(log2 a) for a > 0
    q = np.where(a < 2.0 ** -6, 2.0 ** -9, np.exp2((fl - 3).astype(np.float64)))
    r = np.rint(a / q) * q                    # ties to even
    r = np.minimum(r, 448.0)
    _, ex2 = np.frexp(r)
    fl2 = ex2 - 1
    normal = r >= 2.0 ** -6
    exp_field = np.where(normal, fl2 + 7, 0).astype(np.int64)
    mant = np.where(normal, np.rint((r / np.exp2(np.where(normal, fl2, 0).astype(np.float64)) - 1.0) * 8.0),
                    np.rint(r / 2.0 ** -9)).astype(np.int64)
    out = ((exp_field << 3) | mant).astype(np.uint8)
    out = np.where(r == 0.0, 0, out).astype(np.uint8) | sign
    # the hardware conversion yields the positive canonical NaN
    out = np.where(nan, 0x7F, out).astype(np.uint8)
    return out.reshape(x.shape)


_E4M3_TABLE = None


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    global _E4M3_TABLE
    if _E4M3_TABLE is None:
        t = np.zeros(256, dtype=np.float32)
        for v in range(256):
            s = -1.0 if v & 0x80 else 1.0
            ef, m = (v >> 3) & 0xF, v & 7
            if ef == 0xF and m == 7:
                t[v] = np.nan
            elif ef == 0:
                t[v] = s * m * 2.0 ** -9
            else:
                t[v] = s * (1 + m / 8.0) * 2.0 ** (ef - 7)
        _E4M3_TABLE = t
    return _E4M3_TABLE[np.asarray(b, dtype=np.uint8)]


# --------------------------------------------------------------------------- scale layout

def swizzle(e: np.ndarray) -> np.ndarray:
    """(R, B) scale bytes -> cuBLAS's swizzled layout: 128 x 4 tiles of 512 B,
    byte (r & 31) * 16 + ((r >> 5) & 3) * 4 + (b & 3)
    (src/nanochat/model/fp8/mx_kernel.cuh:41-44, tests/test_fp8.cpp:37-41)."""
    R, B = e.shape
    assert R % 128 == 0 and B % 4 == 0
    return np.ascontiguousarray(
        e.reshape(R // 128, 4, 32, B // 4, 4).transpose(0, 3, 2, 1, 4)).reshape(-1)


def unswizzle(s: np.ndarray, R: int, B: int) -> np.ndarray:
    """Inverse of :func:`swizzle` (tests/test_fp8.cpp:45)."""
    return np.ascontiguousarray(
        np.asarray(s).reshape(R // 128, B // 4, 32, 4, 4).transpose(0, 3, 2, 1, 4)).reshape(R, B)


def mx_scale_index(row: int, block: int, tiles: int) -> int:
    """Byte offset of (row, block) in a swizzled buffer with `tiles` tiles per
    128 rows (src/nanochat/model/fp8/mx_kernel.cuh:42-44)."""
    return ((row >> 7) * tiles + (block >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (block & 3)


# --------------------------------------------------------------------------- quantizer

def apply_prologue(x: np.ndarray, prologue: int = PROLOGUE_NONE, h: np.ndarray | None = None) -> np.ndarray:
    """The value each element takes before quantization.

    relu^2: float(bf16(max(v, 0)^2)) (src/nanochat/model/fp8/fp8_kernel.cu:44-50);
    relu^2 backward: float(bf16(h > 0 ? g * (2 h) : 0)) from g = x and h
    (src/nanochat/model/fp8/fp8_kernel.cu:154-168)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if prologue == PROLOGUE_NONE:
        return x
    with np.errstate(over="ignore", invalid="ignore"):
        if prologue == PROLOGUE_RELU_SQUARE:
            r = np.where(x <= 0, np.float32(0), x)
            return round_bf16(r * r)
        if prologue == PROLOGUE_RELU_SQUARE_BWD:
            h = np.ascontiguousarray(h, dtype=np.float32)
            return round_bf16(np.where(h <= 0, np.float32(0), x * (np.float32(2) * h)))
    raise ValueError(prologue)


def mx_reference(x: np.ndarray, rule: int = SCALE_RULE_REFERENCE):
    """x (R, C) fp32 -> (E4M3 bytes (R, C), unswizzled E8M0 bytes (R, C/32)).

    amax over 32 consecutive values with NaNs skipped (fmaxf,
    src/nanochat/model/fp8/mx_kernel.cuh:82-90), exponent, exact power-of-two
    multiplier, saturating RNE cast (mx_kernel.cuh:53-65; tests/test_fp8.cpp:25-35)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    R, C = x.shape
    assert C % BLOCK == 0
    b = x.reshape(R, C // BLOCK, BLOCK)
    with np.errstate(invalid="ignore"):
        amax = np.fmax.reduce(np.abs(b), axis=-1, initial=np.float32(0))
    e = mx_exponent(amax, rule)
    mult = mx_multiplier(e)
    with np.errstate(over="ignore", invalid="ignore"):
        scaled = b * mult[..., None]
    return e4m3_from_f32(scaled).reshape(R, C), e.astype(np.uint8)


def quantize_mx(x: np.ndarray, rows: bool = True, cols: bool = True, prologue: int = PROLOGUE_NONE,
                h: np.ndarray | None = None, rule: int = SCALE_RULE_REFERENCE) -> dict:
    """Both layouts of a tensor, as the reference's quantize_mx
    (src/nanochat/model/fp8/fp8.h:82-84, fp8_kernel.h:35-39): ``data`` (R, C) +
    swizzled ``scale`` with blocks along C, and ``data_t`` (C, R) + ``scale_t``
    with blocks along R. data_t is x re-quantized along columns, not a byte
    transpose (tests/test_fp8.cpp:172)."""
    v = apply_prologue(x, prologue, h)
    out = {}
    if rows:
        d, e = mx_reference(v, rule)
        out["data"], out["scale"] = d, swizzle(e)
    if cols:
        d, e = mx_reference(np.ascontiguousarray(v.T), rule)
        out["data_t"], out["scale_t"] = d, swizzle(e)
    return out


def mx_dequantize(data: np.ndarray, scale: np.ndarray, dtype=np.float32) -> np.ndarray:
    """(R, C) bytes + swizzled scales -> values (tests/test_fp8.cpp:43-49)."""
    R, C = data.shape
    e = unswizzle(scale, R, C // BLOCK).astype(np.float64)
    mult = np.exp2(e - 127.0)
    v = e4m3_to_f32(data).astype(np.float64).reshape(R, C // BLOCK, BLOCK) * mult[..., None]
    return v.reshape(R, C).astype(dtype)


# --------------------------------------------------------------------------- GEMM

def mx_gemm_ref(a, a_scale, b, b_scale, acc_dtype=np.float32) -> np.ndarray:
    """alpha = 1 product of dequantized operands: D[M, N] = deq(A)[M, K] . deq(B)[N, K]^T
    (src/nanochat/model/fp8/mx_gemm.h:18-22; tests/test_fp8.cpp:206)."""
    return mx_dequantize(a, a_scale, acc_dtype) @ mx_dequantize(b, b_scale, acc_dtype).T


def gemm_bf16_out(acc: np.ndarray, resid: np.ndarray | None = None) -> np.ndarray:
    """bf16 output rounding, returned as fp32 values. With a residual the sum
    is rounded a second time: bf16(float(bf16(acc)) + float(resid))
    (src/nanochat/model/ops/residual_norm_kernel.cu:96-104)."""
    out = round_bf16(acc.astype(np.float32))
    if resid is not None:
        out = round_bf16(out + np.asarray(resid, dtype=np.float32))
    return out


def gemm_f32_out(acc, alpha: float = 1.0, d_old=None) -> np.ndarray:
    """fp32 output: d = alpha * acc (+ d_old when accumulating)
    (src/nanochat/model/fp8/mx_gemm.h:44-50)."""
    out = np.float32(alpha) * acc.astype(np.float32)
    if d_old is not None:
        out = out + np.asarray(d_old, dtype=np.float32)
    return out


def residual_norm(x, r=None, x0=None, lr: float = 1.0, l0: float = 0.0, eps: float = 1e-6, rstd=None):
    """Fused residual add + lambda blend + RMS norm over rows of bf16 values held as fp32
    (src/nanochat/model/ops/residual_norm_kernel.cu:80-128):
      s = r ? bf16(x + r) : x;  res = x0 ? bf16(bf16(lr_b * s) + bf16(l0_b * x0)) : s;  n = bf16(res * rstd)
    The sum of squares is taken in the kernel's order (lane l of 32 owns columns (it * 32 + l) * 8 .. + 7, fp32
    accumulation in column order, then the xor 16..1 butterfly); a bf16 square is exact in fp32, so the kernel's
    fused multiply-add and a plain add agree. rstd given: used as is (the device's rsqrt is approximate).
    Returns (s, res, rstd, n); s is None without r."""
    x = np.asarray(x, dtype=np.float32)
    rows, cols = x.shape
    s = None
    v = x
    if r is not None:
        v = round_bf16(x + np.asarray(r, dtype=np.float32))
        s = v
    if x0 is not None:
        lr_b, l0_b = round_bf16(np.float32(lr)), round_bf16(np.float32(l0))
        v = round_bf16(round_bf16(lr_b * v) + round_bf16(l0_b * np.asarray(x0, dtype=np.float32)))
    res = v
    iters = (cols + 255) // 256
    padded = np.zeros((rows, iters * 256), dtype=np.float32)
    padded[:, :cols] = res
    sq = (padded * padded).reshape(rows, iters, 32, 8)      # [row, it, lane, k]: exact products
    lanes = np.zeros((rows, 32), dtype=np.float32)
    for it in range(iters):
        for k in range(8):
            lanes = (lanes + sq[:, it, :, k]).astype(np.float32)
    idx = np.arange(32)
    for o in (16, 8, 4, 2, 1):
        lanes = (lanes + lanes[:, idx ^ o]).astype(np.float32)
    mean = (lanes[:, 0] / np.float32(cols) + np.float32(eps)).astype(np.float32)
    if rstd is None:
        rstd = (1.0 / np.sqrt(mean.astype(np.float64))).astype(np.float32)
    rstd = np.asarray(rstd, dtype=np.float32)
    n = round_bf16(res * rstd[:, None])
    return s, res, rstd, n


def softcap_ce_loss(logits, targets, vocab: int, softcap: float):
    """Per row of bf16 logits held as fp32 (rows, padded): lse = log sum exp(capped) over the first `vocab` columns with
    capped = softcap * tanh(z / softcap), loss = lse - capped[target]; target < 0: loss 0, lse nan (unset in the
    kernel) (src/nanochat/model/ops/softcap_ce_kernel.cu:62-103). Computed in float64 and rounded: the kernel's fp32
    tanhf / expf / logf and its summation order agree with this to a few ulp, not bit for bit."""
    z = np.asarray(logits, dtype=np.float64)[:, :vocab]
    t = np.asarray(targets, dtype=np.int64)
    capped = softcap * np.tanh(z / softcap)
    lse = np.log(np.exp(capped - softcap).sum(axis=1)) + softcap
    rows = np.arange(z.shape[0])
    loss = lse - capped[rows, np.clip(t, 0, vocab - 1)]
    valid = t >= 0
    return np.where(valid, loss, 0.0).astype(np.float32), np.where(valid, lse, np.nan).astype(np.float32)


def softcap_ce_grad(logits, targets, lse, vocab: int, softcap: float, scale=1.0):
    """The loss's gradient with respect to the logits as the bf16 the reference's grad kernel writes
    (src/nanochat/model/ops/softcap_ce_kernel.cu:49-54, 105-114): bf16((p - onehot) * (1 - th^2) * scale) with
    th = tanh(z / softcap), p = exp(softcap * th - lse); 0 for rows with target < 0 and for columns >= vocab. scale: a
    number or one per row. In float64 then rounded: values that sit on a bf16 rounding boundary may differ from the
    kernel's fp32 arithmetic by one bf16 ulp."""
    z = np.asarray(logits, dtype=np.float64)
    rows, padded = z.shape
    t = np.asarray(targets, dtype=np.int64)
    th = np.tanh(z / softcap)
    lse64 = np.where(t >= 0, np.asarray(lse, dtype=np.float64), 0.0)
    p = np.exp(softcap * th - lse64[:, None])
    onehot = np.zeros_like(z)
    valid = t >= 0
    onehot[np.arange(rows)[valid], t[valid]] = 1.0
    g = (p - onehot) * (1.0 - th * th) * (np.asarray(scale, dtype=np.float64).reshape(-1, 1) if np.ndim(scale) else scale)
    g[:, vocab:] = 0.0
    g[~valid] = 0.0
    return round_bf16(g.astype(np.float32))


def rel_norm_diff(a, b) -> float:
    """||a - b|| / ||b|| in fp64 (tests/test_fp8.cpp:20-23)."""
    a64, b64 = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a64 - b64) / (np.linalg.norm(b64) + 1e-30))
