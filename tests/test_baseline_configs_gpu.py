"""GPU parity on the benchmark's own configurations: the d12 single Linear with its seed, distribution and scale rule
(bit-exact quantization, GEMM within 2e-3 of dequantize-then-fp32-matmul, the whole product on the CPU oracle), and
the d24 forward / backward / lm_head sets at full size through properties that do not need a full CPU product:
bit-exact quantization of every operand, sampled rows of the product against the oracle, linearity, and the fused
residual against the separate add."""
import numpy as np
import pytest
import torch

import nanochat_cpp_b200 as nc
from helpers import assert_quantized_equal, np_f32, np_u8
from oracle import mx_oracle as mo

pytestmark = pytest.mark.gpu
TOL_BF16, TOL_F32 = 2e-3, 1e-5


def rel(a, b):
    a64, b64 = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a64 - b64) / (np.linalg.norm(b64) + 1e-30))


@pytest.mark.parametrize("rule", [nc.SCALE_REFERENCE, nc.SCALE_OCP_FLOOR])
def test_config1_d12_mlp_fc_forward(rule):
    """A bf16 [2048, 768] ~ N(0,1), W bf16 [3072, 768] ~ N(0, 1/sqrt(768)), seed 0, A drawn before W, both quantized
    along K; with the reference's scale rule and with the 2^(floor(log2 amax) - 8) rule the configuration names."""
    g = torch.Generator().manual_seed(0)
    a = torch.randn(2048, 768, generator=g).to(torch.bfloat16)
    w = (torch.randn(3072, 768, generator=g) / 768 ** 0.5).to(torch.bfloat16)
    qa = nc.quantize_mx(a.cuda(), True, False, scale_rule=rule)
    qw = nc.quantize_mx(w.cuda(), True, False, scale_rule=rule)
    oa = mo.quantize_mx(np_f32(a), True, False, rule=rule)
    ow = mo.quantize_mx(np_f32(w), True, False, rule=rule)
    assert_quantized_equal(qa, oa, "A")
    assert_quantized_equal(qw, ow, "W")
    want = mo.mx_gemm_ref(oa["data"], oa["scale"], ow["data"], ow["scale"])
    y = nc.mx_gemm(qa.data, qa.inv_scale, qw.data, qw.inv_scale, torch.bfloat16)
    assert rel(np_f32(y), want) < TOL_BF16
    y32 = nc.mx_gemm(qa.data, qa.inv_scale, qw.data, qw.inv_scale, torch.float32)
    assert rel(np_f32(y32), want) < TOL_F32
    # and the quantized product is close to the bf16 Linear it replaces (e4m3 resolution, ~4% per element, averaged)
    assert rel(want, np_f32(a) @ np_f32(w).T) < 0.05


def sampled_product(qa, qb, rows):
    """Rows `rows` of deq(a) . deq(b)^T on the CPU oracle."""
    da = mo.mx_dequantize(np_u8(qa.data), np_u8(qa.inv_scale))[rows]
    db = mo.mx_dequantize(np_u8(qb.data), np_u8(qb.inv_scale))
    return da @ db.T


ROWS = np.array([0, 31, 128, 4097, 8191, 12345, 16383])


@pytest.mark.parametrize("name,N,K,resid", [("qkv", 4608, 1536, False), ("attn_out", 1536, 1536, True),
                                            ("mlp_fc", 6144, 1536, False), ("mlp_proj", 1536, 6144, True)])
def test_config2_d24_forward_set(name, N, K, resid):
    """M = 16384 tokens, activations ~ N(0,1), weights ~ N(0, 1/sqrt(K)), bf16 out, fused residual on attn-out / proj."""
    M = 16384
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).to(torch.bfloat16)
    r = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16) if resid else None
    qx, qw = nc.quantize_mx(x, True, False), nc.quantize_mx(w, True, False)
    # quantization bit-exact on a slab of rows (the full tensors are compared with the reference kernel elsewhere)
    slab = slice(4096, 4096 + 256)
    ox = mo.quantize_mx(np_f32(x[slab]), True, False)
    assert np.array_equal(np_u8(qx.data[slab]), ox["data"])
    y = nc.mx_gemm(qx.data, qx.inv_scale, qw.data, qw.inv_scale, torch.bfloat16, resid=r)
    want = sampled_product(qx, qw, ROWS)
    if resid:
        plain = nc.mx_gemm(qx.data, qx.inv_scale, qw.data, qw.inv_scale, torch.bfloat16)
        assert torch.equal(y, plain + r)  # the fused add rounds as the separate one, everywhere
        want = mo.gemm_bf16_out(want, np_f32(r)[ROWS])
    assert rel(np_f32(y)[ROWS], want) < TOL_BF16


@pytest.mark.parametrize("name,N,K", [("qkv", 4608, 1536), ("attn_out", 1536, 1536), ("mlp_fc", 6144, 1536),
                                      ("mlp_proj", 1536, 6144)])
def test_config3_d24_backward_set(name, N, K):
    """dY bf16 [16384, N] ~ N(0, 1e-3): dgrad dX = dYq . (W_t)^T and wgrad dW = (dY_t)q . (X_t)q^T with the scales along
    the 16384 tokens; bf16 into the bucket and fp32 accumulation."""
    M = 16384
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).to(torch.bfloat16)
    dy = (torch.randn(M, N, device="cuda", generator=g) * 1e-3).to(torch.bfloat16)
    qx, qw, qg = nc.quantize_mx(x), nc.quantize_mx(w), nc.quantize_mx(dy)
    # column-wise (transposed) quantization along the tokens: a slab of columns against the oracle
    cols = slice(256, 384)
    og = mo.quantize_mx(np_f32(dy[:, cols]), False, True)
    assert np.array_equal(np_u8(qg.data_t[cols]), og["data_t"])
    # dgrad: [M, K] = dYq [M, N] . W_t [K, N]^T
    dx = nc.mx_gemm(qg.data, qg.inv_scale, qw.data_t, qw.inv_scale_t, torch.bfloat16)
    da = mo.mx_dequantize(np_u8(qg.data), np_u8(qg.inv_scale))[ROWS]
    dw_t = mo.mx_dequantize(np_u8(qw.data_t), np_u8(qw.inv_scale_t))
    assert rel(np_f32(dx)[ROWS], da @ dw_t.T) < TOL_BF16
    # wgrad: [N, K] = dY_t [N, M] . X_t [K, M]^T, fp32 then accumulated, and bf16 for the bucket
    dw = torch.zeros(N, K, dtype=torch.float32, device="cuda")
    nc.mx_gemm_f32(qg.data_t, qg.inv_scale_t, qx.data_t, qx.inv_scale_t, dw, False)
    rows = np.array([0, 127, 128, N // 2 + 5, N - 1])
    dg_t = mo.mx_dequantize(np_u8(qg.data_t), np_u8(qg.inv_scale_t))[rows]
    dx_t = mo.mx_dequantize(np_u8(qx.data_t), np_u8(qx.inv_scale_t))
    want = dg_t.astype(np.float64) @ dx_t.astype(np.float64).T
    assert rel(np_f32(dw)[rows], want) < TOL_F32 * 3  # K = 16384 terms: fp32 accumulation order
    first = dw.clone()
    nc.mx_gemm_f32(qg.data_t, qg.inv_scale_t, qx.data_t, qx.inv_scale_t, dw, True)
    assert torch.equal(dw, 2 * first)  # += of the same product is exact doubling
    dw16 = nc.mx_gemm(qg.data_t, qg.inv_scale_t, qx.data_t, qx.inv_scale_t, torch.bfloat16)
    assert torch.equal(dw16, first.to(torch.bfloat16))


def test_config4_lm_head_chunks_student_t():
    """X = 0.5 StudentT(nu = 3) drawn as N(0,1) / sqrt(chi2_3 / 3), W_lm [32768, 1536] ~ N(0, 1/sqrt(1536)), row chunks
    of 2048 tokens: the heavy tails spread the E8M0 scales over many values and every chunk equals the same rows of
    the unchunked product."""
    M, C, V, chunk = 16384, 1536, 32768, 2048
    g = torch.Generator(device="cuda").manual_seed(4)
    z = torch.randn(M, C, device="cuda", generator=g)
    chi2 = torch.randn(M, C, 3, device="cuda", generator=g).square().sum(-1)
    x = (0.5 * z / (chi2 / 3).sqrt()).to(torch.bfloat16)
    w = (torch.randn(V, C, device="cuda", generator=g) / C ** 0.5).to(torch.bfloat16)
    qx, qw = nc.quantize_mx(x), nc.quantize_mx(w, True, False)
    scales = np_u8(qx.inv_scale)
    normal = np_u8(nc.quantize_mx(z.to(torch.bfloat16), True, False).inv_scale)
    # 32-value block maxima of a normal draw span three or four binades; the heavy tails more than double that
    assert len(np.unique(scales)) >= 8 and len(np.unique(scales)) >= 2 * len(np.unique(normal))
    slab = slice(2048, 2048 + 128)
    ox = mo.quantize_mx(np_f32(x[slab]))
    assert np.array_equal(np_u8(qx.data[slab]), ox["data"])
    assert np.array_equal(np_u8(qx.data_t[:, slab]), ox["data_t"])
    blocks = C // 32
    rows = np.array([0, 100, 2047])
    for c in (0, 3, 7):
        begin = c * chunk
        logits = nc.mx_gemm(qx.data[begin:begin + chunk], qx.inv_scale[begin * blocks:(begin + chunk) * blocks],
                            qw.data, qw.inv_scale, torch.bfloat16)
        da = mo.mx_dequantize(np_u8(qx.data), np_u8(qx.inv_scale))[begin + rows]
        db = mo.mx_dequantize(np_u8(qw.data), np_u8(qw.inv_scale))
        assert rel(np_f32(logits)[rows], da @ db.T) < TOL_BF16, c


def student_t_activations(g, M, C):
    z = torch.randn(M, C, device="cuda", generator=g)
    chi2 = torch.randn(M, C, 3, device="cuda", generator=g).square().sum(-1)
    return (0.5 * z / (chi2 / 3).sqrt()).to(torch.bfloat16)


def test_config4_lm_head_backward_chunks():
    """The other two GEMMs of the chunked lm_head (src/nanochat/model/ops/softcap_ce.cpp:88, 109): per chunk of 2048
    tokens dX = gq . (W_t)^T with K = the 32768-entry vocabulary, and once over all chunks dW = (g_t)q . (X_t)q^T with
    K = 16384 tokens, the gradient's transposed layout written chunk by chunk into one (vocab, tokens) buffer.
    dlogits ~ N(0, 1e-3) bf16; sampled rows against the oracle's dequantized products."""
    M, C, V, chunk = 16384, 1536, 32768, 2048
    g = torch.Generator(device="cuda").manual_seed(5)
    x = student_t_activations(g, M, C)
    w = (torch.randn(V, C, device="cuda", generator=g) / C ** 0.5).to(torch.bfloat16)
    qx, qw = nc.quantize_mx(x, False, True), nc.quantize_mx(w, False, True)
    g_all = nc.empty_mx(M, V, x.device, rows=False)  # only the (vocab, tokens) layout is kept across chunks
    dw_t = mo.mx_dequantize(np_u8(qw.data_t), np_u8(qw.inv_scale_t))  # [C, V]
    rows = np.array([0, 777, 2047])
    for c in range(M // chunk):
        begin = c * chunk
        dl = (torch.randn(chunk, V, device="cuda", generator=g) * 1e-3).to(torch.bfloat16)
        gq = nc.empty_mx(chunk, V, x.device, cols=False)
        nc.quantize_mx_into(dl, False, nc.mx_out(gq.data, gq.inv_scale),
                            nc.mx_out(g_all.data_t, g_all.inv_scale_t, 0, begin))
        if c in (0, 5):
            og = mo.quantize_mx(np_f32(dl[:, 4096:4224]), False, True)
            assert np.array_equal(np_u8(g_all.data_t[4096:4224, begin:begin + chunk]), og["data_t"])
            dx = nc.mx_gemm(gq.data, gq.inv_scale, qw.data_t, qw.inv_scale_t, torch.bfloat16)  # [2048, 1536], K = 32768
            da = mo.mx_dequantize(np_u8(gq.data), np_u8(gq.inv_scale))[rows]
            assert rel(np_f32(dx)[rows], da @ dw_t.T) < TOL_BF16, c
        del dl, gq
    # the one weight-gradient GEMM over all tokens: [V, C] = g_t [V, M] . X_t [C, M]^T
    dw = torch.zeros(V, C, dtype=torch.float32, device="cuda")
    nc.mx_gemm_f32(g_all.data_t, g_all.inv_scale_t, qx.data_t, qx.inv_scale_t, dw, False)
    dx_t = mo.mx_dequantize(np_u8(qx.data_t), np_u8(qx.inv_scale_t)).astype(np.float64)
    per_row_tile = (M // 128) * 512  # scale bytes of one 128-row tile of the (vocab, tokens) layout
    for rt, inside in ((0, [0, 127]), (157, [1, 64]), (V // 128 - 1, [126, 127])):
        slab = slice(rt * 128, rt * 128 + 128)
        dg_t = mo.mx_dequantize(np_u8(g_all.data_t[slab]),
                                np_u8(g_all.inv_scale_t[rt * per_row_tile:(rt + 1) * per_row_tile]))[inside]
        want = dg_t.astype(np.float64) @ dx_t.T
        got = np_f32(dw[slab])[inside]
        assert rel(got, want) < TOL_F32 * 3, rt  # 16384 terms: fp32 accumulation order
    dw16 = nc.mx_gemm(g_all.data_t, g_all.inv_scale_t, qx.data_t, qx.inv_scale_t, torch.bfloat16)
    assert torch.equal(dw16, dw.to(torch.bfloat16))
    alpha = torch.tensor([0.125], device="cuda")
    first = dw.clone()
    nc.mx_gemm_f32(g_all.data_t, g_all.inv_scale_t, qx.data_t, qx.inv_scale_t, dw, True, alpha=alpha)
    assert torch.equal(dw, first * 1.125)  # += alpha . product, alpha a power of two: exact


def test_fused_quantize_epilogues_at_d24_size():
    """The two GEMMs of the relu^2 MLP that quantize in their epilogue (src/nanochat/model/fp8/fp8.cpp:279-284,
    318-323), at the d24 step's own size 16384 x 6144 x 1536: h and MX(relu(h)^2), and MX(dh) from ga and h, equal
    the GEMM followed by the stand-alone quantizer bit for bit (tests/test_fp8.cpp:363-426 at small sizes)."""
    M, N, K = 16384, 6144, 1536
    g = torch.Generator(device="cuda").manual_seed(6)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).to(torch.bfloat16)
    qx, qw = nc.quantize_mx(x, True, False), nc.quantize_mx(w, True, False)
    want_h = nc.mx_gemm(qx.data, qx.inv_scale, qw.data, qw.inv_scale, torch.bfloat16)
    want = nc.quantize_mx(want_h, True, True, True)
    h = torch.full_like(want_h, float("nan"))
    got = nc.empty_mx(M, N, x.device)
    for t in (got.data, got.data_t, got.inv_scale, got.inv_scale_t):
        t.view(torch.uint8).zero_()
    assert nc.mx_gemm_relu_square(h, got.data, got.inv_scale, got.data_t, got.inv_scale_t, qx.data, qx.inv_scale,
                                  qw.data, qw.inv_scale)
    assert torch.equal(h, want_h)
    for name in ("data", "inv_scale", "data_t", "inv_scale_t"):
        a, b = getattr(got, name).view(torch.uint8), getattr(want, name).view(torch.uint8)
        assert torch.equal(a, b), f"relu^2 {name}: {(a != b).sum().item()} bytes differ"
    # a slab of the fused output against the CPU oracle's relu^2 prologue
    slab = slice(8192, 8192 + 128)
    ref = mo.quantize_mx(np_f32(want_h[slab, :256]), True, False, mo.PROLOGUE_RELU_SQUARE)
    assert np.array_equal(np_u8(got.data[slab, :256]), ref["data"])
    # backward form: ga = dYq . (W_proj_t)^T with the same operand shapes, h the forward's output
    want_bwd = nc.quantize_mx_relu_square_bwd(want_h, h)  # ga := want_h as a stand-in gradient of the same shape
    for t in (got.data, got.data_t, got.inv_scale, got.inv_scale_t):
        t.view(torch.uint8).zero_()
    assert nc.mx_gemm_relu_square_bwd(qx.data, qx.inv_scale, qw.data, qw.inv_scale, h, got.data, got.inv_scale,
                                      got.data_t, got.inv_scale_t)
    for name in ("data", "inv_scale", "data_t", "inv_scale_t"):
        a, b = getattr(got, name).view(torch.uint8), getattr(want_bwd, name).view(torch.uint8)
        assert torch.equal(a, b), f"relu^2 bwd {name}: {(a != b).sum().item()} bytes differ"


@pytest.mark.parametrize("depth", [12, 26])
def test_d12_and_d26_linear_shapes(depth):
    """The tile scheduler is sized for d12 to d26 (n_embd = 64 x depth, src/nanochat/model/gpt.cpp:25-39): every Linear
    shape of the two end points (C = 768 and C = 1664, whose K = 13 x 128 and N = 4992 / 6656 are not multiples of either
    tile width) forward, dgrad and wgrad at M = 4096 tokens: sampled rows against the oracle's dequantized product,
    the whole output against cuBLASLt's MXFP8 GEMM on the same operands, and determinism."""
    C, M = 64 * depth, 4096
    g = torch.Generator(device="cuda").manual_seed(100 + depth)
    rows = np.array([0, 127, 128, 2049, M - 1])
    for name, N, K in (("qkv", 3 * C, C), ("attn_out", C, C), ("mlp_fc", 4 * C, C), ("mlp_proj", C, 4 * C)):
        x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
        w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).to(torch.bfloat16)
        dy = (torch.randn(M, N, device="cuda", generator=g) * 1e-3).to(torch.bfloat16)
        qx, qw, qg = nc.quantize_mx(x), nc.quantize_mx(w), nc.quantize_mx(dy)
        cases = (("fwd", qx.data, qx.inv_scale, qw.data, qw.inv_scale, torch.bfloat16),
                 ("dgrad", qg.data, qg.inv_scale, qw.data_t, qw.inv_scale_t, torch.bfloat16),
                 ("wgrad", qg.data_t, qg.inv_scale_t, qx.data_t, qx.inv_scale_t, torch.float32))
        for what, a, a_s, b, b_s, dt in cases:
            y = nc.mx_gemm(a, a_s, b, b_s, dt)
            assert torch.equal(y, nc.mx_gemm(a, a_s, b, b_s, dt)), (name, what)
            lt = torch._scaled_mm(a, b.t(), a_s, b_s, None, None, dt, False)
            assert rel(np_f32(y), np_f32(lt)) < (TOL_BF16 if dt == torch.bfloat16 else TOL_F32), (name, what)
            r = rows[rows < a.size(0)]
            da = mo.mx_dequantize(np_u8(a), np_u8(a_s))[r].astype(np.float64)
            db = mo.mx_dequantize(np_u8(b), np_u8(b_s)).astype(np.float64)
            tol = TOL_BF16 if dt == torch.bfloat16 else TOL_F32 * 3
            assert rel(np_f32(y)[r], da @ db.T) < tol, (name, what)
