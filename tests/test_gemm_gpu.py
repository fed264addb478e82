"""GPU parity of the block-scaled GEMM, through the C ABI, against the CPU oracle (dequantize -> fp32 matmul)
and against cuBLASLt (the reference's --gemm=cublas arithmetic, reached through torch._scaled_mm)."""
import numpy as np
import pytest
import torch

import nanochat_cpp_b200 as nc
from helpers import gemm_operands, np_f32, np_u8
from oracle import mx_oracle as mo

pytestmark = pytest.mark.gpu

# tests/test_fp8.cpp:331-332, 187 (512x384x256 as M,N,K), BASELINE config 1 (2048x3072x768)
SHAPES = [(128, 128, 128), (256, 384, 512), (640, 256, 1536), (512, 384, 256), (2048, 3072, 768)]
TOL_BF16 = 2e-3   # north_star: relative Frobenius error vs dequantize-then-fp32-matmul
TOL_F32 = 1e-5    # tests/test_fp8.cpp:343


def rel(a: torch.Tensor, b: torch.Tensor) -> float:
    a64, b64 = a.double(), b.double()
    return ((a64 - b64).norm() / (b64.norm() + 1e-30)).item()


def quantized(M, N, K, seed=0):
    a, b = gemm_operands(M, N, K, seed)
    qa, qb = nc.quantize_mx(a.cuda(), True, False), nc.quantize_mx(b.cuda(), True, False)
    return qa, qb


def oracle_product(qa, qb) -> torch.Tensor:
    ref = mo.mx_gemm_ref(np_u8(qa.data), np_u8(qa.inv_scale), np_u8(qb.data), np_u8(qb.inv_scale))
    return torch.from_numpy(ref)


def scaled_mm(qa, qb, dtype):
    return torch._scaled_mm(qa.data, qb.data.t(), qa.inv_scale, qb.inv_scale, None, None, dtype, False)


@pytest.fixture(autouse=True)
def _default_config():
    nc.capi.lib.mxb200_set_gemm_config(0, 0)
    yield
    nc.capi.lib.mxb200_set_gemm_config(0, 0)
    assert nc.capi.device_status() == 0, "a bounded wait ran out inside the GEMM"


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("tile_n", [128, 256, 384, 512])
def test_bf16_and_f32_match_oracle(M, N, K, tile_n):
    nc.capi.lib.mxb200_set_gemm_config(tile_n, 0)
    qa, qb = quantized(M, N, K)
    want = oracle_product(qa, qb)
    got_bf16 = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.bfloat16)
    got_f32 = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.float32)
    assert rel(got_f32.cpu(), want) < TOL_F32
    assert rel(got_bf16.float().cpu(), want) < TOL_BF16
    # the bf16 output is the fp32 one rounded once (bit-exact: same accumulator, same rounding)
    assert torch.equal(got_bf16, got_f32.to(torch.bfloat16))


@pytest.mark.parametrize("M,N,K", SHAPES[:4])
def test_matches_cublaslt(M, N, K):
    """Fp8.CutlassGemmMatchesCublas (tests/test_fp8.cpp:328-360) with this library in CUTLASS's seat."""
    qa, qb = quantized(M, N, K)
    for dtype, tol in ((torch.bfloat16, TOL_BF16), (torch.float32, TOL_F32)):
        want = scaled_mm(qa, qb, dtype)
        got = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, dtype)
        assert rel(got.float(), want.float()) < tol, (M, N, K, dtype)


@pytest.mark.parametrize("M,N,K", [(256, 384, 512), (640, 256, 1536)])
def test_f32_accumulate_with_device_alpha(M, N, K):
    """d += alpha * a.b^T with alpha on the device (tests/test_fp8.cpp:346-358)."""
    qa, qb = quantized(M, N, K)
    alpha = torch.full((1,), 0.5, device="cuda")
    g = torch.Generator().manual_seed(9)
    d0 = torch.randn(M, N, generator=g)
    got = d0.cuda().clone()
    nc.mx_gemm_f32(qa.data, qa.inv_scale, qb.data, qb.inv_scale, got, True, alpha)
    want = mo.gemm_f32_out(oracle_product(qa, qb).numpy(), 0.5, d0.numpy())
    assert rel(got.cpu(), torch.from_numpy(want)) < TOL_F32
    # = then += gives twice the product (tests/test_fp8.cpp:268-273)
    acc = torch.empty(M, N, device="cuda")
    nc.mx_gemm_f32(qa.data, qa.inv_scale, qb.data, qb.inv_scale, acc, False)
    once = acc.clone()
    nc.mx_gemm_f32(qa.data, qa.inv_scale, qb.data, qb.inv_scale, acc, True)
    assert rel(acc, 2 * once) < 1e-6


@pytest.mark.parametrize("tile_n", [128, 256, 384, 512])
def test_fused_residual_is_bit_exact_with_separate_add(tile_n):
    """bf16(float(bf16(acc)) + resid): the reference's separate x + r (residual_norm_kernel.cu:96-104)."""
    nc.capi.lib.mxb200_set_gemm_config(tile_n, 0)
    M, N, K = 512, 768, 256
    qa, qb = quantized(M, N, K, seed=4)
    g = torch.Generator().manual_seed(5)
    r = torch.randn(M, N, generator=g).to(torch.bfloat16).cuda()
    plain = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.bfloat16)
    fused = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.bfloat16, resid=r)
    assert torch.equal(fused, (plain.float() + r.float()).to(torch.bfloat16))
    # in place: the residual stream is also the output
    out = r.clone()
    nc.mx_gemm_out(out, qa.data, qa.inv_scale, qb.data, qb.inv_scale, resid=out)
    assert torch.equal(out, fused)
    want = mo.gemm_bf16_out(oracle_product(qa, qb).numpy(), np_f32(r))
    assert rel(fused.float().cpu(), torch.from_numpy(want)) < TOL_BF16


@pytest.mark.parametrize("M,N", [(256, 384), (256, 640), (384, 384), (640, 896), (128, 1024)])
@pytest.mark.parametrize("tile_n", [256, 384, 512])
def test_partial_last_tiles(M, N, tile_n):
    """N % 256 == 128 (and, for the CTA-pair kernel, M % 256 == 128): the last tile is half empty."""
    nc.capi.lib.mxb200_set_gemm_config(tile_n, 0)
    qa, qb = quantized(M, N, 512, seed=6)
    want = oracle_product(qa, qb)
    canary = torch.full((M * N + 4096,), float("nan"), device="cuda")
    out = canary[: M * N].view(M, N)
    nc.mx_gemm_out(out, qa.data, qa.inv_scale, qb.data, qb.inv_scale)
    assert rel(out.cpu(), want) < TOL_F32
    assert torch.isnan(canary[M * N:]).all(), "wrote past the output"
    out16 = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    nc.mx_gemm_out(out16, qa.data, qa.inv_scale, qb.data, qb.inv_scale)
    assert torch.equal(out16, out.to(torch.bfloat16))


@pytest.mark.parametrize("splits", [2, 3, 4])
@pytest.mark.parametrize("tile_n", [128, 256, 384, 512])
def test_split_k_matches_single_pass_and_is_deterministic(splits, tile_n):
    """The weight-gradient shape class: long K, few tiles. Slices are summed in fixed order."""
    nc.capi.lib.mxb200_set_gemm_config(tile_n, 0)
    M, N, K = 256, 384, 4096
    g = torch.Generator().manual_seed(8)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    b = torch.randn(N, K, generator=g).to(torch.bfloat16)
    qa, qb = nc.quantize_mx(a.cuda(), True, False), nc.quantize_mx(b.cuda(), True, False)
    want = oracle_product(qa, qb)
    one = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.float32, splits=1)
    runs = [nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.float32, splits=splits) for _ in range(3)]
    assert rel(runs[0].cpu(), want) < TOL_F32
    assert rel(runs[0], one) < 1e-6
    assert torch.equal(runs[0], runs[1]) and torch.equal(runs[1], runs[2])
    # += with alpha through the split path, and a bf16 output with residual
    alpha = torch.full((1,), 2.0, device="cuda")
    acc = torch.ones(M, N, device="cuda")
    nc.mx_gemm_f32(qa.data, qa.inv_scale, qb.data, qb.inv_scale, acc, True, alpha, splits=splits)
    assert rel(acc, 1 + 2 * runs[0]) < 1e-6
    r = torch.randn(M, N, generator=g).to(torch.bfloat16).cuda()
    fused = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.bfloat16, resid=r, splits=splits)
    assert torch.equal(fused, (runs[0].to(torch.bfloat16).float() + r.float()).to(torch.bfloat16))


def test_scales_vary_per_block_and_row():
    """Operands whose scales differ for every (row, K block): catches any slip in the scale plumbing
    (which byte of which TMEM column feeds which MMA step)."""
    M, N, K = 256, 256, 1024
    g = torch.Generator().manual_seed(10)
    rowmag = torch.logspace(-3, 3, M).unsqueeze(1)
    blkmag = torch.logspace(-2, 2, K // 32).repeat_interleave(32).unsqueeze(0)
    a = (torch.randn(M, K, generator=g) * rowmag * blkmag).to(torch.bfloat16)
    b = (torch.randn(N, K, generator=g) * torch.logspace(2, -2, N).unsqueeze(1) * blkmag.flip(1)).to(torch.bfloat16)
    qa, qb = nc.quantize_mx(a.cuda(), True, False), nc.quantize_mx(b.cuda(), True, False)
    assert len(torch.unique(qa.inv_scale.view(torch.uint8))) > 20
    want = oracle_product(qa, qb)
    got = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.float32)
    # row-wise, so that small-magnitude rows count too
    err = ((got.cpu().double() - want.double()).norm(dim=1) / want.double().norm(dim=1)).max().item()
    assert err < TOL_F32


def test_linear_forward_backward_matches_dequantized():
    """Fp8.MxMatmulMatchesDequantized (tests/test_fp8.cpp:184-212): y, dx, dw of one Linear."""
    Ntok, cin, cout = 512, 256, 384
    g = torch.Generator().manual_seed(0)
    x0 = (torch.randn(Ntok, cin, generator=g) * torch.logspace(-2, 2, cin)).to(torch.bfloat16)
    w0 = torch.randn(cout, cin, generator=g) * 0.05
    g0 = (torch.randn(Ntok, cout, generator=g) * torch.logspace(-3, 1, cout)).to(torch.bfloat16)
    x = x0.cuda().requires_grad_()
    w = w0.cuda().requires_grad_()
    y = nc.fp8_matmul(x, w)
    y.backward(g0.cuda())
    assert w.grad.dtype == torch.float32
    xq, wq, gq = (mo.quantize_mx(np_f32(t)) for t in (x0, w0, g0))
    y_ref = mo.mx_gemm_ref(xq["data"], xq["scale"], wq["data"], wq["scale"])
    dx_ref = mo.mx_gemm_ref(gq["data"], gq["scale"], wq["data_t"], wq["scale_t"])
    dw_ref = mo.mx_gemm_ref(gq["data_t"], gq["scale_t"], xq["data_t"], xq["scale_t"])
    assert rel(y.detach().float().cpu(), torch.from_numpy(y_ref)) < TOL_BF16
    assert rel(x.grad.float().cpu(), torch.from_numpy(dx_ref)) < TOL_BF16
    assert rel(w.grad.cpu(), torch.from_numpy(dw_ref)) < TOL_F32
    # a second micro-step accumulates in fp32 (tests/test_fp8.cpp:289-290)
    nc.fp8_matmul(x, w).backward(g0.cuda())
    assert rel(w.grad.cpu(), torch.from_numpy(2 * dw_ref)) < TOL_F32


def test_merged_qkv_grads_share_one_buffer():
    """tests/test_fp8.cpp:297-309: three weights, one wgrad GEMM, .grads are row blocks of one buffer."""
    Ntok, cin = 512, 384
    g = torch.Generator().manual_seed(2)
    x = torch.randn(Ntok, cin, generator=g).to(torch.bfloat16).cuda()
    ws = [(torch.randn(r, cin, generator=g) * 0.05).cuda().requires_grad_() for r in (128, 256, 128)]
    gs = torch.randn(Ntok, 512, generator=g).to(torch.bfloat16).cuda()
    xq, gq = nc.quantize_mx(x), nc.quantize_mx(gs)
    for _ in range(2):
        nc.mx_grad_weights(gq.data_t, gq.inv_scale_t, xq.data_t, xq.inv_scale_t, ws)
    ref = 2 * mo.mx_gemm_ref(np_u8(gq.data_t), np_u8(gq.inv_scale_t), np_u8(xq.data_t), np_u8(xq.inv_scale_t))
    row = 0
    for w in ws:
        assert w.grad.data_ptr() == ws[0].grad.data_ptr() + row * cin * 4
        assert rel(w.grad.cpu(), torch.from_numpy(ref[row:row + w.size(0)])) < TOL_F32
        row += w.size(0)


def test_full_size_against_cublaslt_and_linearity():
    """BASELINE config 2's QKV projection (M=16384, N=4608, K=1536), too large for the CPU oracle in seconds:
    checked against cuBLASLt on the same operands, plus linearity in alpha and exactness of += 0."""
    M, N, K = 16384, 4608, 1536
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    b = (torch.randn(N, K, generator=g, device="cuda") / K ** 0.5).to(torch.bfloat16)
    qa, qb = nc.quantize_mx(a, True, False), nc.quantize_mx(b, True, False)
    got = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.bfloat16)
    want = scaled_mm(qa, qb, torch.bfloat16)
    assert rel(got.float(), want.float()) < TOL_BF16
    f1 = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.float32)
    assert rel(f1, scaled_mm(qa, qb, torch.float32)) < TOL_F32
    f2 = torch.zeros_like(f1)
    nc.mx_gemm_f32(qa.data, qa.inv_scale, qb.data, qb.inv_scale, f2, True, torch.full((1,), 2.0, device="cuda"))
    assert torch.equal(f2, 2 * f1)  # power-of-two alpha and += 0 are exact
    # sampled rows against the CPU oracle
    rows = torch.tensor([0, 127, 128, 4095, 8191, 16383])
    sub = mo.mx_dequantize(np_u8(qa.data), np_u8(qa.inv_scale))[rows.numpy()] @ mo.mx_dequantize(np_u8(qb.data), np_u8(qb.inv_scale)).T
    assert rel(f1[rows.cuda()].cpu(), torch.from_numpy(sub)) < TOL_F32


def test_argument_errors():
    qa, qb = quantized(128, 128, 128)
    out = torch.empty(128, 128, dtype=torch.bfloat16, device="cuda")
    lib = nc.capi.lib
    s = torch.cuda.current_stream().cuda_stream
    assert lib.mxb200_gemm_bf16(qa.data.data_ptr(), qa.inv_scale.data_ptr(), qb.data.data_ptr(), qb.inv_scale.data_ptr(),
                                out.data_ptr(), None, 128, 100, 128, s) == nc.capi.ERR_SHAPE
    assert lib.mxb200_gemm_bf16(None, qa.inv_scale.data_ptr(), qb.data.data_ptr(), qb.inv_scale.data_ptr(),
                                out.data_ptr(), None, 128, 128, 128, s) == nc.capi.ERR_NULL
    assert lib.mxb200_gemm_bf16(qa.data.data_ptr() + 8, qa.inv_scale.data_ptr(), qb.data.data_ptr(), qb.inv_scale.data_ptr(),
                                out.data_ptr(), None, 128, 128, 128, s) == nc.capi.ERR_ALIGNMENT
    assert lib.mxb200_gemm_splitk(qa.data.data_ptr(), qa.inv_scale.data_ptr(), qb.data.data_ptr(), qb.inv_scale.data_ptr(),
                                  out.data_ptr(), 0, None, 128, 128, 128, None, 0, 1, None, 0, s) == nc.capi.OK
    K = 1024
    qa, qb = quantized(128, 128, K)
    assert lib.mxb200_gemm_splitk(qa.data.data_ptr(), qa.inv_scale.data_ptr(), qb.data.data_ptr(), qb.inv_scale.data_ptr(),
                                  out.data_ptr(), 0, None, 128, 128, K, None, 0, 2, None, 0, s) == nc.capi.ERR_WORKSPACE
    with pytest.raises(RuntimeError):
        nc.mx_gemm(qa.data, qa.inv_scale, qb.data[:, :512], qb.inv_scale, torch.bfloat16)


# tests/test_fp8.cpp:368-369, plus a tile-crossing shape with M % 256 == 128 and one of BASELINE's MLP size class
FUSED_SHAPES = [(128, 128, 128), (256, 384, 512), (640, 512, 1536), (2048, 6144, 1536)]


@pytest.mark.parametrize("M,N,K", FUSED_SHAPES)
@pytest.mark.parametrize("tile_n", [0, 384, 512])
def test_relu_square_gemm_matches_unfused(M, N, K, tile_n):
    """Fp8.CutlassReluSquareGemmMatchesUnfused (tests/test_fp8.cpp:363-390): the fc GEMM with relu^2's MX quantize
    in the epilogue vs the GEMM then quantize_mx, bit for bit."""
    nc.capi.lib.mxb200_set_gemm_config(tile_n, 0)
    qa, qb = quantized(M, N, K, seed=12)
    want_h = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.bfloat16)
    want = nc.quantize_mx(want_h, True, True, True)
    h = torch.full_like(want_h, float("nan"))
    got = nc.empty_mx(M, N, h.device)
    for t in (got.data, got.data_t, got.inv_scale, got.inv_scale_t):
        t.view(torch.uint8).zero_()
    assert nc.mx_gemm_relu_square(h, got.data, got.inv_scale, got.data_t, got.inv_scale_t, qa.data, qa.inv_scale,
                                  qb.data, qb.inv_scale)
    assert torch.equal(h, want_h)
    for name in ("data", "inv_scale", "data_t", "inv_scale_t"):
        g, w = getattr(got, name).view(torch.uint8), getattr(want, name).view(torch.uint8)
        assert torch.equal(g, w), f"{name}: {(g != w).sum().item()} bytes differ"
    # and against the CPU oracle end to end on the small shapes
    if M * N <= 640 * 512:
        ref = mo.quantize_mx(np_f32(want_h), True, True, mo.PROLOGUE_RELU_SQUARE)
        assert np.array_equal(np_u8(got.data), ref["data"]) and np.array_equal(np_u8(got.inv_scale_t), ref["scale_t"])


@pytest.mark.parametrize("M,N,K", FUSED_SHAPES)
@pytest.mark.parametrize("tile_n", [0, 384, 512])
def test_relu_square_bwd_gemm_matches_unfused(M, N, K, tile_n):
    """Fp8.CutlassReluSquareBwdGemmMatchesUnfused (tests/test_fp8.cpp:394-426): the proj dgrad GEMM with relu^2's
    backward quantize in the epilogue vs the GEMM then quantize_mx_relu_square_bwd, bit for bit."""
    nc.capi.lib.mxb200_set_gemm_config(tile_n, 0)
    qa, qb = quantized(M, N, K, seed=13)
    g = torch.Generator().manual_seed(14)
    h = torch.randn(M, N, generator=g).to(torch.bfloat16).cuda()
    ga = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.bfloat16)
    want = nc.quantize_mx_relu_square_bwd(ga, h)
    got = nc.empty_mx(M, N, h.device)
    for t in (got.data, got.data_t, got.inv_scale, got.inv_scale_t):
        t.view(torch.uint8).zero_()
    assert nc.mx_gemm_relu_square_bwd(qa.data, qa.inv_scale, qb.data, qb.inv_scale, h, got.data, got.inv_scale,
                                      got.data_t, got.inv_scale_t)
    for name in ("data", "inv_scale", "data_t", "inv_scale_t"):
        gt, w = getattr(got, name).view(torch.uint8), getattr(want, name).view(torch.uint8)
        assert torch.equal(gt, w), f"{name}: {(gt != w).sum().item()} bytes differ"


@pytest.mark.parametrize("max_ctas", [2, 6, 50])
def test_tile_scheduler_with_few_pairs(max_ctas):
    """The CTA-pair kernel's pairs draw their tiles from a global counter: with the launch capped to a few CTAs each
    pair walks many tiles, and the result is the same bits as with the whole machine."""
    M, N, K = 1024, 1280, 512
    qa, qb = quantized(M, N, K, seed=21)
    full = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.bfloat16)
    nc.capi.lib.mxb200_set_gemm_config(0, max_ctas)
    few = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.bfloat16)
    assert torch.equal(few, full)
    assert rel(few.float().cpu(), oracle_product(qa, qb)) < TOL_BF16
    f32 = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.float32, splits=2)
    assert rel(f32.cpu(), oracle_product(qa, qb)) < TOL_F32


def test_overlapping_launches_on_two_streams():
    """Launches that overlap on the device take different scheduler counters: two streams of GEMMs of different
    shapes, 30 launches each, give what the same launches give one after another."""
    qa1, qb1 = quantized(2048, 1024, 512, seed=22)
    qa2, qb2 = quantized(1024, 1536, 1024, seed=23)
    want1 = nc.mx_gemm(qa1.data, qa1.inv_scale, qb1.data, qb1.inv_scale, torch.bfloat16)
    want2 = nc.mx_gemm(qa2.data, qa2.inv_scale, qb2.data, qb2.inv_scale, torch.bfloat16)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    outs1 = [torch.empty_like(want1) for _ in range(30)]
    outs2 = [torch.empty_like(want2) for _ in range(30)]
    for i in range(30):
        with torch.cuda.stream(s1):
            nc.mx_gemm_out(outs1[i], qa1.data, qa1.inv_scale, qb1.data, qb1.inv_scale)
        with torch.cuda.stream(s2):
            nc.mx_gemm_out(outs2[i], qa2.data, qa2.inv_scale, qb2.data, qb2.inv_scale)
    torch.cuda.synchronize()
    assert all(torch.equal(o, want1) for o in outs1)
    assert all(torch.equal(o, want2) for o in outs2)


def test_bounded_wait_reports_and_clears():
    """Every device-side wait gives up after a limit, records where, and the kernel returns: a warp that waits 1 ms on a
    barrier nothing arrives on comes back, the status call reports it once, and the device goes on working."""
    lib = nc.capi.lib
    assert nc.capi.device_status() == 0
    assert lib.mxb200_selftest_bounded_wait(1_000_000, torch.cuda.current_stream().cuda_stream) == nc.capi.OK
    import ctypes
    word = ctypes.c_uint32(0)
    assert lib.mxb200_device_status(ctypes.byref(word)) == nc.capi.ERR_WATCHDOG
    assert word.value == 0x8000007F
    assert lib.mxb200_device_status(ctypes.byref(word)) == nc.capi.OK and word.value == 0
    assert lib.mxb200_selftest_bounded_wait(0, None) == nc.capi.ERR_ARGUMENT
    assert lib.mxb200_selftest_bounded_wait(20_000_000, None) == nc.capi.ERR_ARGUMENT
    qa, qb = quantized(256, 256, 256, seed=31)
    got = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.float32)
    assert rel(got.cpu(), oracle_product(qa, qb)) < TOL_F32


def test_gemm_after_an_unreported_give_up():
    """A bounded wait that ran out and was never read back with mxb200_device_status must not disturb the launches
    that follow: the scheduler counters of a launch are left at zero by its last pair whether or not a wait gave up,
    so GEMMs of several shapes right after a give-up still match the oracle. The status word is read (and cleared)
    only at the end."""
    lib = nc.capi.lib
    assert nc.capi.device_status() == 0
    assert lib.mxb200_selftest_bounded_wait(500_000, torch.cuda.current_stream().cuda_stream) == nc.capi.OK
    for M, N, K, seed in ((512, 768, 256, 41), (1024, 1280, 512, 42), (256, 256, 1024, 43)):
        qa, qb = quantized(M, N, K, seed=seed)
        for _ in range(3):
            got = nc.mx_gemm(qa.data, qa.inv_scale, qb.data, qb.inv_scale, torch.float32)
        assert rel(got.cpu(), oracle_product(qa, qb)) < TOL_F32
    assert nc.capi.device_status() == 0x8000007F  # the give-up is still reported, once
    assert nc.capi.device_status() == 0
