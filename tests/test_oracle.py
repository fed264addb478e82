"""CPU: the numpy oracle against the reference's torch-op formulation, the plain-C oracle, and the golden
bytes written by the reference's own CUDA kernel (tests/golden)."""
import ctypes
import glob
import os

import numpy as np
import pytest
import torch

from helpers import quantizer_input, gemm_operands, np_f32, np_u8, residual_norm_inputs
from oracle import mx_oracle as mo
from oracle import torch_reference as tr

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SHAPES = [(128, 128), (256, 384), (384, 1024)]  # tests/test_fp8.cpp:158


@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("relu_square", [False, True])
def test_numpy_oracle_matches_reference_torch_ops(rows, cols, dtype, relu_square):
    """Mirrors Fp8.MxQuantizeMatchesTorchOps (tests/test_fp8.cpp:156-181) with the oracle in the kernel's seat."""
    if relu_square and dtype != torch.bfloat16:
        pytest.skip("relu^2 reads bf16 only")
    x = quantizer_input(rows, cols).to(dtype)
    want = tr.quantize_mx(x, True, True, relu_square)
    got = mo.quantize_mx(np_f32(x), True, True, mo.PROLOGUE_RELU_SQUARE if relu_square else mo.PROLOGUE_NONE)
    for key in ("data", "scale", "data_t", "scale_t"):
        assert np.array_equal(np_u8(want[key]).reshape(-1), got[key].reshape(-1)), key


def test_e4m3_cast_matches_torch_over_the_whole_range():
    v = torch.linspace(-448, 448, 400001)
    assert np.array_equal(np_u8(v.to(torch.float8_e4m3fn)), mo.e4m3_from_f32(v.numpy()))
    g = torch.Generator().manual_seed(1)
    v = (torch.randn(200000, generator=g) * torch.logspace(-12, 2, 200000)).clamp(-448, 448)
    assert np.array_equal(np_u8(v.to(torch.float8_e4m3fn)), mo.e4m3_from_f32(v.numpy()))
    # every byte round-trips
    b = np.arange(256, dtype=np.uint8)
    vals = mo.e4m3_to_f32(b)
    ok = ~np.isnan(vals)
    back = mo.e4m3_from_f32(vals[ok])
    assert np.array_equal(back & 0x7F, b[ok] & 0x7F)


def test_saturation_nan_inf():
    x = np.array([500.0, -1e9, np.inf, -np.inf, np.nan, 464.0, 463.9, 448.0], dtype=np.float32)
    assert mo.e4m3_from_f32(x).tolist() == [0x7E, 0xFE, 0x7E, 0xFE, 0x7F, 0x7E, 0x7E, 0x7E]


def test_scale_rules_differ_only_above_mantissa_1_75():
    amax = np.array([1.8 * 512, 448.0, 1.0, 1.76, 1.75, 0.0, 1.5 * 2.0 ** 127, 1e-45], dtype=np.float32)
    ref, flo = mo.mx_exponent(amax, 0), mo.mx_exponent(amax, 1)
    assert (ref - flo).tolist() == [1, 0, 0, 1, 0, 0, 0, 0]
    assert ref[5] == 0 and ref[6] <= 253
    # reference rule never needs saturation: amax * 2^(127 - e) <= 448
    big = np.abs(np.random.default_rng(0).standard_normal(10000).astype(np.float32)) * 1e3 + 1e-3
    assert np.all(big * mo.mx_multiplier(mo.mx_exponent(big, 0)) <= 448.0)
    assert np.any(big * mo.mx_multiplier(mo.mx_exponent(big, 1)) > 448.0)


def test_swizzle_is_the_index_function():
    R, B = 256, 12
    e = np.arange(R * B, dtype=np.uint32).reshape(R, B)
    s = mo.swizzle((e % 251).astype(np.uint8))
    for r, b in [(0, 0), (1, 0), (31, 3), (32, 0), (127, 11), (128, 4), (255, 11)]:
        assert s[mo.mx_scale_index(r, b, B // 4)] == e[r, b] % 251
    assert np.array_equal(mo.unswizzle(s, R, B), (e % 251).astype(np.uint8))


@pytest.mark.parametrize("rule", [0, 1])
@pytest.mark.parametrize("prologue", [0, 1, 2])
def test_c_oracle_matches_numpy_oracle(oracle_c, rule, prologue):
    R, C = 256, 384
    x = np_f32(quantizer_input(R, C, seed=3).to(torch.bfloat16))
    x[5, 7], x[6, 70], x[7, 100] = np.nan, np.inf, -np.inf
    h = np_f32(torch.randn(R, C, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16))
    want = mo.quantize_mx(x, True, True, prologue, h, rule)
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    for transposed in (0, 1):
        Rr, Cc = (C, R) if transposed else (R, C)
        data = np.zeros((Rr, Cc), np.uint8)
        scale = np.zeros(Rr * Cc // 32, np.uint8)
        oracle_c.mxo_quantize(x.ctypes.data_as(vp), h.ctypes.data_as(vp), i64(R), i64(C), transposed, prologue, rule,
                              data.ctypes.data_as(vp), i64(Cc), scale.ctypes.data_as(vp), i64(Cc // 128))
        assert np.array_equal(data, want["data_t" if transposed else "data"])
        assert np.array_equal(scale, want["scale_t" if transposed else "scale"])


def test_gemm_oracles_agree(oracle_c):
    """numpy dequantize -> fp32 matmul vs the C oracle's double-precision triple loop, and both vs the
    reference's torch-op dequantize (tests/test_fp8.cpp:43-49, 206)."""
    M, N, K = 128, 256, 384
    a, b = gemm_operands(M, N, K)
    qa, qb = mo.quantize_mx(np_f32(a), True, False), mo.quantize_mx(np_f32(b), True, False)
    ref = mo.mx_gemm_ref(qa["data"], qa["scale"], qb["data"], qb["scale"])
    d = np.zeros((M, N), np.float32)
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    oracle_c.mxo_gemm_f32(qa["data"].ctypes.data_as(vp), qa["scale"].ctypes.data_as(vp), qb["data"].ctypes.data_as(vp),
                          qb["scale"].ctypes.data_as(vp), d.ctypes.data_as(vp), i64(M), i64(N), i64(K),
                          ctypes.c_float(1.0), 0)
    assert mo.rel_norm_diff(ref, d) < 1e-6
    ta = tr.mx_dequantize(torch.from_numpy(qa["data"]).view(torch.float8_e4m3fn), torch.from_numpy(qa["scale"]))
    tb = tr.mx_dequantize(torch.from_numpy(qb["data"]).view(torch.float8_e4m3fn), torch.from_numpy(qb["scale"]))
    assert mo.rel_norm_diff(ref, torch.mm(ta, tb.t()).numpy()) < 1e-6


def test_residual_rounding_is_two_roundings(oracle_c):
    acc = np.array([1.00390625, 3.0000001, -2.5], dtype=np.float32)
    r = np.array([1.0, 1e-3, 2.5], dtype=np.float32)
    out = mo.gemm_bf16_out(acc, r)
    want = mo.round_bf16(mo.round_bf16(acc) + r)
    assert np.array_equal(out, want)
    for i in range(3):
        assert oracle_c.mxo_bf16_out(float(acc[i]), 1, float(r[i])) == out[i]


def _golden_files():
    return sorted(glob.glob(os.path.join(GOLDEN, "quantize_*.npz")))


@pytest.mark.parametrize("path", _golden_files() or [None])
def test_oracle_matches_reference_kernel_golden(path):
    """Bytes the reference's own nanochat_mx_quantize_* kernels wrote on a B200 (tests/golden/make_golden.py)."""
    if path is None:
        pytest.skip("no golden files yet")
    g = np.load(path)
    x = mo.bf16_bits_to_f32(g["x_bf16_bits"]) if "x_bf16_bits" in g else g["x_f32"]
    pro = int(g["prologue"])
    h = mo.bf16_bits_to_f32(g["h_bf16_bits"]) if "h_bf16_bits" in g else None
    want = mo.quantize_mx(x, True, True, pro, h)
    for key in ("data", "scale", "data_t", "scale_t"):
        assert np.array_equal(want[key].reshape(-1), g[key].reshape(-1)), (os.path.basename(path), key)


def _gemm_golden_files():
    return sorted(glob.glob(os.path.join(GOLDEN, "gemm_*.npz")))


@pytest.mark.parametrize("path", _gemm_golden_files() or [None])
def test_gemm_oracle_matches_cublaslt_golden(path):
    """fp32 outputs of cuBLASLt's MXFP8 GEMM (the reference's --gemm=cublas arithmetic, mx_gemm.cpp:158) on a
    B200 for the same quantized operands. Tolerance 1e-5, the reference's own backend-vs-backend bar for fp32
    (tests/test_fp8.cpp:343)."""
    if path is None:
        pytest.skip("no golden files yet")
    g = np.load(path)
    ref = mo.mx_gemm_ref(g["a"], g["a_scale"], g["b"], g["b_scale"])
    assert mo.rel_norm_diff(ref, g["d_f32"]) < 1e-5


# ---------------------------------------------------------------- fused residual step

RN_CASES = [(128, 768, True, True), (128, 256, False, False), (64, 1536, True, False), (32, 2048, False, True),
            (5, 136, True, True), (3, 24, True, True)]  # the last two: partial warp passes (tests/test_residual_norm.cpp:98)


def _rn_args(rows, cols, add, blend):
    inp = residual_norm_inputs(rows, cols, add, blend)
    f = lambda t: None if t is None else np.ascontiguousarray(np_f32(t))
    lr, l0 = (float(inp["lr"][inp["layer"]]), float(inp["l0"][inp["layer"]])) if blend else (1.0, 0.0)
    return inp, f(inp["x"]), f(inp["r"]), f(inp["x0"]), lr, l0, float(np.finfo(np.float32).eps)


@pytest.mark.parametrize("rows,cols,add,blend", RN_CASES)
def test_residual_norm_numpy_matches_c(oracle_c, rows, cols, add, blend):
    _, x, r, x0, lr, l0, eps = _rn_args(rows, cols, add, blend)
    s, res, rstd, n = mo.residual_norm(x, r, x0, lr, l0, eps)
    cs, cres, cn, crstd = np.zeros_like(x), np.zeros_like(x), np.zeros_like(x), np.zeros(rows, np.float32)
    p = lambda a: None if a is None else a.ctypes.data
    oracle_c.mxo_residual_norm(p(x), p(r), p(x0), lr, l0, rows, cols, eps, None, p(cs) if add else None, p(cres),
                               p(crstd), p(cn))
    assert np.array_equal(res, cres) and np.array_equal(rstd, crstd) and np.array_equal(n, cn)
    assert s is None or np.array_equal(s, cs)


@pytest.mark.parametrize("rows,cols,add,blend", RN_CASES)
def test_residual_norm_matches_torch_ops(rows, cols, add, blend):
    """The op-by-op bf16 path the fused kernel is checked against (tests/test_residual_norm.cpp:41-51), with the
    lambdas rounded to bf16 as type promotion does on the device: res bit for bit, n within one bf16 rounding of
    F.rms_norm."""
    inp, x, r, x0, lr, l0, eps = _rn_args(rows, cols, add, blend)
    s, res, rstd, n = mo.residual_norm(x, r, x0, lr, l0, eps)
    ts = inp["x"] + inp["r"] if add else inp["x"]
    tres = ts
    if blend:
        k = inp["layer"]
        tres = inp["lr"][k].to(torch.bfloat16) * ts + inp["l0"][k].to(torch.bfloat16) * inp["x0"]
    assert np.array_equal(np_f32(tres), res)
    want = torch.nn.functional.rms_norm(tres.float(), (cols,), eps=eps).numpy()
    assert np.all(np.abs(n - want) <= np.maximum(np.abs(want) * 2.0 ** -8, 1e-30))
    ref_rstd = 1.0 / np.sqrt((res.astype(np.float64) ** 2).mean(axis=1) + eps)
    assert np.allclose(rstd, ref_rstd, rtol=5e-7)


def _rn_golden_files():
    return sorted(glob.glob(os.path.join(GOLDEN, "residual_norm_*.npz")))


@pytest.mark.parametrize("path", _rn_golden_files() or [None])
def test_residual_norm_oracle_matches_reference_kernel_golden(path):
    """What the reference's own nanochat_residual_norm_mx_fwd_c* kernel wrote on a B200 (tests/golden/make_golden.py):
    s, res and the MX bytes bit for bit, n bit for bit given the kernel's rstd, rstd itself within the device
    rsqrt's 2 ulp."""
    if path is None:
        pytest.skip("no golden files yet")
    g = np.load(path)
    f = lambda k: mo.bf16_bits_to_f32(g[k]) if k in g else None
    x, r, x0 = f("x_bf16_bits"), f("r_bf16_bits"), f("x0_bf16_bits")
    lr, l0, eps = float(g["lr"]), float(g["l0"]), float(g["eps"])
    s, res, rstd, _ = mo.residual_norm(x, r, x0, lr, l0, eps)
    assert np.array_equal(res, f("res_bf16_bits"))
    if "s_bf16_bits" in g:
        assert np.array_equal(s, f("s_bf16_bits"))
    assert np.allclose(rstd, g["rstd"], rtol=3e-7, atol=0)
    _, _, _, n = mo.residual_norm(x, r, x0, lr, l0, eps, rstd=g["rstd"])
    assert np.array_equal(n, f("n_bf16_bits"))
    want = mo.quantize_mx(n)
    for key in ("data", "scale", "data_t", "scale_t"):
        assert np.array_equal(want[key].reshape(-1), g[key].reshape(-1)), (os.path.basename(path), key)


# ---------------------------------------------------------------- chunked lm_head loss

def _ce_case(rows=128, padded=256, vocab=250, seed=0):
    g = torch.Generator().manual_seed(seed)
    logits = (torch.randn(rows, padded, generator=g) * 8).to(torch.bfloat16)
    targets = torch.randint(vocab, (rows,), generator=g, dtype=torch.int64)
    targets[:5] = -1
    scale = torch.rand(rows, generator=g) + 0.5
    return np.ascontiguousarray(np_f32(logits)), targets.numpy(), scale.numpy(), vocab


def test_softcap_ce_oracles_agree_and_match_torch(oracle_c):
    """numpy (float64) and C (fp32 in the kernel's summation order) restatements against each other and against
    torch's cross_entropy of the capped logits (tests/test_softcap_ce.cpp:27-35)."""
    z, t, scale, vocab = _ce_case()
    rows, padded = z.shape
    loss, lse = mo.softcap_ce_loss(z, t, vocab, 15.0)
    closs, clse = np.zeros(rows, np.float32), np.zeros(rows, np.float32)
    oracle_c.mxo_softcap_ce_loss(z.ctypes.data, rows, padded, t.ctypes.data, vocab, padded, 15.0, closs.ctypes.data,
                                 clse.ctypes.data)
    valid = t >= 0
    assert np.allclose(loss, closs, rtol=2e-6, atol=2e-6) and np.allclose(lse[valid], clse[valid], rtol=1e-6)
    capped = 15 * torch.tanh(torch.from_numpy(z[:, :vocab]) / 15)
    want = torch.nn.functional.cross_entropy(capped, torch.from_numpy(t), ignore_index=-1, reduction="none").numpy()
    assert np.allclose(loss, want, rtol=1e-5, atol=1e-5)
    # gradient: autograd of the same graph, scaled per row
    zt = torch.from_numpy(z).double().requires_grad_()
    l = torch.nn.functional.cross_entropy(15 * torch.tanh(zt[:, :vocab] / 15), torch.from_numpy(t), ignore_index=-1,
                                          reduction="none")
    (l * torch.from_numpy(scale).double()).sum().backward()
    g = mo.softcap_ce_grad(z, t, lse, vocab, 15.0, scale)
    assert np.abs(g - zt.grad.numpy()).max() <= 2.0 ** -8 * np.abs(zt.grad.numpy()).max()
    cg = np.zeros_like(z)
    oracle_c.mxo_softcap_ce_grad(z.ctypes.data, rows, padded, t.ctypes.data, clse.ctypes.data, vocab, padded, 15.0,
                                 np.ascontiguousarray(scale).ctypes.data, 1, 0, cg.ctypes.data)
    assert (cg != g).mean() < 2e-3 and np.abs(cg - g).max() <= 2.0 ** -7 * np.abs(g).max()


def _ce_golden_files():
    return sorted(glob.glob(os.path.join(GOLDEN, "softcap_ce_*.npz")))


@pytest.mark.parametrize("path", _ce_golden_files() or [None])
def test_softcap_ce_oracle_matches_reference_kernel_golden(path):
    """What the reference's own softcap cross-entropy kernels gave on a B200 (tests/golden/make_golden.py): loss and
    lse to fp32 rounding (host and device tanh / exp / log differ in the last bits), the bf16 gradient and its MX
    bytes up to the rare value that sits on a rounding boundary; quantize_mx of the kernel's own bf16 gradient bit for
    bit."""
    if path is None:
        pytest.skip("no golden files yet")
    g = np.load(path)
    z = mo.bf16_bits_to_f32(g["logits_bf16_bits"])
    t, vocab, softcap = g["targets"], int(g["vocab"]), float(g["softcap"])
    valid = t >= 0
    loss, lse = mo.softcap_ce_loss(z, t, vocab, softcap)
    assert np.allclose(loss, g["loss"], rtol=2e-6, atol=2e-6)
    assert np.allclose(lse[valid], g["lse"][valid], rtol=1e-6)
    scale = g["grad_scale"] if "grad_scale" in g else 1.0
    if int(g["num_valid"]) > 0:
        scale = scale / np.float32(int(g["num_valid"]))
    grad = mo.softcap_ce_grad(z, t, g["lse"], vocab, softcap, scale)
    want_grad = mo.bf16_bits_to_f32(g["grad_bf16_bits"])
    assert (grad != want_grad).mean() < 2e-3
    assert np.abs(grad - want_grad).max() <= 2.0 ** -7 * np.abs(want_grad).max()
    q = mo.quantize_mx(want_grad)
    for key in ("data", "scale", "data_t", "scale_t"):
        assert np.array_equal(q[key].reshape(-1), g[key].reshape(-1)), (os.path.basename(path), key)
