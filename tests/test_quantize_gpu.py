"""GPU parity of the MX quantizer, through the C ABI: bit-exact against the CPU oracle and against the
reference's own CUDA kernel compiled from its source."""
import numpy as np
import pytest
import torch

import nanochat_cpp_b200 as nc
import refkernel
from helpers import assert_quantized_equal, np_u8, oracle_quantize, quantizer_input
from oracle import mx_oracle as mo

pytestmark = pytest.mark.gpu
SHAPES = [(128, 128), (256, 384), (384, 1024)]  # tests/test_fp8.cpp:158


@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("relu_square", [False, True])
def test_matches_oracle(rows, cols, dtype, relu_square):
    """Fp8.MxQuantizeMatchesTorchOps (tests/test_fp8.cpp:156-181): bytes and swizzled scales, both layouts."""
    if relu_square and dtype != torch.bfloat16:
        pytest.skip("relu^2 reads bf16 only")
    x = quantizer_input(rows, cols).to(dtype)
    q = nc.quantize_mx(x.cuda(), True, True, relu_square)
    want = oracle_quantize(x, True, True, mo.PROLOGUE_RELU_SQUARE if relu_square else 0)
    assert_quantized_equal(q, want, f"{rows}x{cols} {dtype} relu2={relu_square}")


@pytest.mark.parametrize("rule", [nc.SCALE_REFERENCE, nc.SCALE_OCP_FLOOR])
def test_scale_rules(rule):
    x = quantizer_input(256, 384, seed=5).to(torch.bfloat16)
    q = nc.quantize_mx(x.cuda(), scale_rule=rule)
    assert_quantized_equal(q, oracle_quantize(x, rule=rule), f"rule {rule}")


def test_rows_only_and_cols_only():
    x = quantizer_input(256, 256, seed=2).to(torch.bfloat16)
    want = oracle_quantize(x)
    q = nc.quantize_mx(x.cuda(), True, False)
    assert q.data_t is None
    assert_quantized_equal(q, {k: want[k] for k in ("data", "scale")}, "rows only")
    q = nc.quantize_mx(x.cuda(), False, True)
    assert q.data is None
    assert_quantized_equal(q, {k: want[k] for k in ("data_t", "scale_t")}, "cols only")


def test_nan_inf_zero_and_extremes():
    """amax skips NaN, elements saturate, the exponent clamps (mx_kernel.cuh:29-34, 61, 82-90)."""
    x = quantizer_input(128, 256, seed=7)
    x[3, 5] = float("nan")
    x[4, 64:96] = float("nan")  # a block of only NaN
    x[5, 100] = float("inf")
    x[6, 130] = float("-inf")
    x[7, :] = 0
    x[8, 0:32] = 3e38
    x[9, 32:64] = 1e-45
    x[10, 64:96] = -0.0
    for dtype in (torch.float32, torch.bfloat16):
        xd = x.to(dtype)
        q = nc.quantize_mx(xd.cuda())
        assert_quantized_equal(q, oracle_quantize(xd), f"edge cases {dtype}")


def test_relu_square_bwd():
    g = torch.Generator().manual_seed(11)
    gr = (torch.randn(256, 384, generator=g) * torch.logspace(-3, 1, 384)).to(torch.bfloat16)
    h = torch.randn(256, 384, generator=g).to(torch.bfloat16)
    q = nc.quantize_mx_relu_square_bwd(gr.cuda(), h.cuda())
    assert_quantized_equal(q, oracle_quantize(gr, prologue=mo.PROLOGUE_RELU_SQUARE_BWD, h=h), "relu^2 bwd")


def test_subview_merged_qkv():
    """Three weights quantized into row ranges of one buffer and column ranges of its transpose
    (fp8.cpp:155-171); equals quantizing the concatenation."""
    g = torch.Generator().manual_seed(13)
    ws = [torch.randn(r, 256, generator=g) * 0.05 for r in (128, 256, 128)]
    out = nc.mx_qkv_weights(*[w.cuda() for w in ws])
    want = oracle_quantize(torch.cat(ws, 0))
    got = nc.Fp8Tensor(out[0], out[1], out[2], out[3])
    assert_quantized_equal(got, want, "merged qkv")


def test_shape_and_alignment_errors():
    x = torch.zeros(128, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        nc.quantize_mx(x)
    x = torch.zeros(128, 128, dtype=torch.float32, device="cuda")
    with pytest.raises(RuntimeError):
        nc.quantize_mx(x, relu_square=True)
    # 16-byte but not 32-byte aligned buffers take the narrow load/store path
    base = torch.zeros(256 * 256 + 8, dtype=torch.float32, device="cuda")
    xin = quantizer_input(256, 256, seed=17)
    view = base[4:4 + 256 * 256].view(256, 256)
    assert view.data_ptr() % 32 == 16
    view.copy_(xin)
    assert_quantized_equal(nc.quantize_mx(view), oracle_quantize(xin), "16-byte aligned fp32 input")


@pytest.mark.skipif(not refkernel.available(), reason="reference kernel library not built")
@pytest.mark.parametrize("rows,cols,dtype", [(256, 384, torch.bfloat16), (384, 1024, torch.float32),
                                             (16384, 1536, torch.bfloat16), (2048, 6144, torch.bfloat16)])
def test_matches_reference_cuda_kernel(rows, cols, dtype):
    """Same input through nanochat_mx_quantize_* (the reference's kernel, unmodified) and through this library:
    identical bytes, at BASELINE sizes too."""
    g = torch.Generator(device="cuda").manual_seed(0)
    x = (torch.randn(rows, cols, generator=g, device="cuda") * torch.logspace(-4, 4, cols, device="cuda")).to(dtype)
    for relu_square in (False, True):
        if relu_square and dtype != torch.bfloat16:
            continue
        ref = refkernel.quantize_mx(x, relu_square)
        q = nc.quantize_mx(x, True, True, relu_square)
        for got, want, name in zip((q.data, q.inv_scale, q.data_t, q.inv_scale_t), ref, ("data", "scale", "data_t", "scale_t")):
            assert torch.equal(got.view(torch.uint8).reshape(-1), want.reshape(-1)), f"{name} relu2={relu_square}"


@pytest.mark.skipif(not refkernel.available(), reason="reference kernel library not built")
def test_oracle_matches_reference_cuda_kernel():
    """Pins the oracle itself against the reference's kernel run here."""
    x = quantizer_input(256, 384, seed=21).to(torch.bfloat16)
    ref = refkernel.quantize_mx(x.cuda())
    want = oracle_quantize(x)
    for t, key in zip(ref, ("data", "scale", "data_t", "scale_t")):
        assert np.array_equal(t.cpu().numpy().reshape(-1), want[key].reshape(-1)), key


def test_full_size_roundtrip_property():
    """Config 2's activation shape: dequantized values lie within half an E4M3 ulp of the input and every
    scale is the smallest admissible power of two (size-independent properties, checked on the GPU)."""
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(16384, 1536, generator=g, device="cuda").to(torch.bfloat16)
    q = nc.quantize_mx(x)
    e = q.inv_scale.view(torch.uint8).view(128, 12, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(16384, 48).float()
    scale = torch.exp2(e - 127)
    deq = q.data.float().view(16384, 48, 32) * scale.unsqueeze(-1)
    xb = x.float().view(16384, 48, 32)
    amax = xb.abs().amax(-1)
    assert torch.all(amax / scale <= 448)
    assert torch.all(amax / scale > 224)          # one exponent lower would overflow
    # relative error of normal values: at most 2^-4 (3 mantissa bits, round to nearest)
    big = xb.abs() >= (scale * 2.0 ** -6).unsqueeze(-1)
    rel = ((deq - xb).abs() / xb.abs().clamp_min(1e-30))[big]
    assert rel.max().item() <= 2.0 ** -4 + 1e-6
    # the transposed layout holds the same tensor: dequantize and compare loosely
    et = q.inv_scale_t.view(torch.uint8).view(12, 128, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(1536, 512).float()
    deqt = (q.data_t.float().view(1536, 512, 32) * torch.exp2(et - 127).unsqueeze(-1)).view(1536, 16384)
    assert (deqt.t() - x.float()).norm() / x.float().norm() < 0.04


# ---- the streaming form: plain bf16 tensors of more than 4 tiles per SM (592 on a B200) go through persistent CTAs

STREAM_SHAPE = (2048, 5120)  # 640 tiles


def _stream_input(seed=11):
    x = quantizer_input(*STREAM_SHAPE, seed=seed)
    x[3, 5] = float("nan")
    x[130, 64:96] = float("nan")  # a block of only NaN
    x[5, 100] = float("inf")
    x[700, 130] = float("-inf")
    x[7, :] = 0
    x[8, 0:32] = 3e38
    x[9, 32:64] = 1e-45
    x[10, 64:96] = -0.0
    return x.to(torch.bfloat16)


@pytest.mark.parametrize("rule", [nc.SCALE_REFERENCE, nc.SCALE_OCP_FLOOR])
def test_streaming_form_matches_oracle(rule):
    """Same bytes as the oracle on a tensor large enough for the persistent kernel, edge values included."""
    x = _stream_input()
    q = nc.quantize_mx(x.cuda(), scale_rule=rule)
    assert_quantized_equal(q, oracle_quantize(x, rule=rule), f"streaming form, rule {rule}")
    assert nc.capi.device_status() == 0


def test_streaming_form_rows_only_and_cols_only():
    x = _stream_input(seed=12)
    want = oracle_quantize(x)
    q = nc.quantize_mx(x.cuda(), True, False)
    assert_quantized_equal(q, {k: want[k] for k in ("data", "scale")}, "streaming form, rows only")
    q = nc.quantize_mx(x.cuda(), False, True)
    assert_quantized_equal(q, {k: want[k] for k in ("data_t", "scale_t")}, "streaming form, cols only")


def test_streaming_form_equals_one_shot_kernel_at_full_size():
    """Config 2's activation (1536 tiles, persistent kernel) against the same tensor quantized in slices of 512 rows
    (48 tiles each, one CTA per tile): same bytes and scales in both layouts."""
    g = torch.Generator(device="cuda").manual_seed(4)
    R, C, S = 16384, 1536, 512
    x = (torch.randn(R, C, generator=g, device="cuda") * torch.logspace(-3, 3, C, device="cuda")).to(torch.bfloat16)
    q = nc.quantize_mx(x)
    sc = q.inv_scale.view(torch.uint8).view(R // 128, C // 128, 512)
    sct = q.inv_scale_t.view(torch.uint8).view(C // 128, R // 128, 512)
    for i in range(R // S):
        part = nc.quantize_mx(x[i * S:(i + 1) * S])
        assert torch.equal(part.data.view(torch.uint8), q.data[i * S:(i + 1) * S].view(torch.uint8))
        assert torch.equal(part.data_t.view(torch.uint8), q.data_t[:, i * S:(i + 1) * S].view(torch.uint8))
        assert torch.equal(part.inv_scale.view(torch.uint8).view(S // 128, C // 128, 512), sc[i * S // 128:(i + 1) * S // 128])
        assert torch.equal(part.inv_scale_t.view(torch.uint8).view(C // 128, S // 128, 512),
                           sct[:, i * S // 128:(i + 1) * S // 128])


def test_streaming_form_overlapping_launches_and_slot_reuse():
    """Launches of the persistent kernel that overlap on two streams each draw tiles from their own counter, and a
    counter is handed back zeroed: 600 launches (the library keeps 256 counters) all give the first launch's bytes."""
    x = _stream_input(seed=13).cuda()
    want = nc.quantize_mx(x)
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = [[nc.empty_mx(*STREAM_SHAPE, x.device) for _ in range(2)] for _ in streams]
    for k in range(300):
        for s, mine in zip(streams, outs):
            with torch.cuda.stream(s):
                out, out_t = nc.mx_outs(mine[k & 1])
                nc.quantize_mx_into(x, False, out, out_t)
    torch.cuda.synchronize()
    for mine in outs:
        for q in mine:
            for a, b in ((q.data, want.data), (q.inv_scale, want.inv_scale), (q.data_t, want.data_t),
                         (q.inv_scale_t, want.inv_scale_t)):
                assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    assert nc.capi.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batch_equals_separate_calls(dtype):
    """mxb200_quantize_mx_batch: 40 tensors of mixed shapes (more than one launch holds), some into sub-views of a
    larger buffer as the merged q/k/v weight is built (src/nanochat/model/fp8/fp8.cpp:155-171), one rows-only, one
    cols-only: the same bytes as a call per tensor."""
    g = torch.Generator().manual_seed(12)
    shapes = [(128, 128), (256, 384), (384, 128), (128, 512)] * 10
    xs = [(torch.randn(r, c, generator=g) * (1 + i)).to(dtype).cuda() for i, (r, c) in enumerate(shapes)]
    xs[3][5, 7] = float("nan")
    want = [nc.quantize_mx(x) for x in xs]
    got = [nc.empty_mx(x.size(0), x.size(1), x.device) for x in xs]
    jobs = [(x, *nc.mx_outs(q)) for x, q in zip(xs, got)]
    none = nc.capi.MxOut(None, 0, None, 0)
    jobs[1] = (xs[1], jobs[1][1], none)   # rows only
    jobs[2] = (xs[2], none, jobs[2][2])   # columns only
    nc.quantize_mx_batch_into(jobs)
    for i, (q, w) in enumerate(zip(got, want)):
        if i != 2:
            assert torch.equal(q.data.view(torch.uint8), w.data.view(torch.uint8)), i
            assert torch.equal(q.inv_scale.view(torch.uint8), w.inv_scale.view(torch.uint8)), i
        if i != 1:
            assert torch.equal(q.data_t.view(torch.uint8), w.data_t.view(torch.uint8)), i
            assert torch.equal(q.inv_scale_t.view(torch.uint8), w.inv_scale_t.view(torch.uint8)), i
    # merged q/k/v: three parts into row ranges of one buffer == the concatenation quantized at once
    parts = [torch.randn(r, 256, generator=g).to(dtype).cuda() for r in (256, 128, 128)]
    merged = nc.mx_qkv_weights(*parts)
    whole = nc.quantize_mx(torch.cat(parts, 0))
    for a, b in zip(merged, (whole.data, whole.data_t, whole.inv_scale, whole.inv_scale_t)):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))


def test_batch_rejects_bad_jobs():
    x = torch.zeros(128, 128, dtype=torch.bfloat16, device="cuda")
    q = nc.empty_mx(128, 128, x.device)
    out, out_t = nc.mx_outs(q)
    with pytest.raises(RuntimeError):
        nc.quantize_mx_batch_into([(x, out, out_t), (x.float(), out, out_t)])  # mixed dtypes
    with pytest.raises(RuntimeError):
        nc.quantize_mx_batch_into([(x[:, :64], out, out_t)])
    nc.quantize_mx_batch_into([])  # nothing to do
