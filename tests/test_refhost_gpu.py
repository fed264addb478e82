"""GPU: nanochat-cpp's own host engine as a caller of this library.

oracle/_ref/nanochat_refhost.so is the reference's fp8.cpp, mx_gemm.cpp, ops/softcap_ce.cpp and ops/residual_norm.cpp
compiled unmodified, with the one seam file of its CUTLASS backend (mx_gemm_kernel.h:13-32) answered by libmxb200.so.
With MxGemmBackend::Cutlass the reference's autograd functions (Float8Matmul fp8.cpp:240-260, MxQkv :424-462,
Fp8ReluSquareMlp :265-338, the chunked lm_head loss ops/softcap_ce.cpp:27-110, mx_grad_weights fp8.cpp:470-514)
therefore run on the B200 kernels: their outputs and .grads must equal what this package's own mirror of those
functions (nanochat_cpp_b200/engine.py) gives, bit for bit, which proves both the drop-in and the mirror. With
MxGemmBackend::Cublas the same build is the reference as it runs on a B200 (cuBLASLt): the two backends agree
within the reference's own bars, 2e-3 for bf16 outputs and 1e-5 for fp32 (tests/test_fp8.cpp:328-360)."""
import pytest
import torch

import nanochat_cpp_b200 as nc
import refhost

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not refhost.available(), reason="the reference host engine was not built")]


def rel(a, b):
    a64, b64 = a.double(), b.double()
    return ((a64 - b64).norm() / (b64.norm() + 1e-30)).item()


@pytest.fixture(autouse=True)
def _cutlass_backend():
    refhost.module().set_backend("cutlass")
    yield
    refhost.module().set_backend("cublas")


def _inputs(N, C, outs, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(N, C, device="cuda", generator=g).to(torch.bfloat16)
    ws = [torch.randn(n, C, device="cuda", generator=g) * 0.05 * (1 + i) for i, n in enumerate(outs)]
    ups = [torch.randn(N, n, device="cuda", generator=g).to(torch.bfloat16) for n in outs]
    return x, ws, ups


def test_quantize_and_gemm_through_the_reference_host():
    """quantize_mx (the reference's kernel, called by its host code) and mx_gemm / mx_gemm_f32 (this library behind
    the seam) against the package's own calls."""
    ref = refhost.module()
    x, (w,), _ = _inputs(384, 512, [256], 1)
    qr = ref.quantize_mx(x, True, True, False)
    q = nc.quantize_mx(x)
    for got, want in zip(qr, (q.data, q.inv_scale, q.data_t, q.inv_scale_t)):
        assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
    qw = nc.quantize_mx(w.to(torch.bfloat16), True, False)
    y_ref = ref.mx_gemm(q.data, q.inv_scale, qw.data, qw.inv_scale, False)
    assert torch.equal(y_ref, nc.mx_gemm(q.data, q.inv_scale, qw.data, qw.inv_scale, torch.bfloat16))
    out = torch.randn(384, 256, device="cuda")
    want = out.clone()
    alpha = torch.full((1,), 0.5, device="cuda")
    ref.mx_gemm_f32(q.data, q.inv_scale, qw.data, qw.inv_scale, out, True, alpha)
    nc.mx_gemm_f32(q.data, q.inv_scale, qw.data, qw.inv_scale, want, True, alpha=alpha)
    assert torch.equal(out, want)
    ref.set_backend("cublas")
    y_lt = ref.mx_gemm(q.data, q.inv_scale, qw.data, qw.inv_scale, False)
    assert rel(y_ref, y_lt) < 2e-3  # Fp8.CutlassGemmMatchesCublas
    f_lt = ref.mx_gemm(q.data, q.inv_scale, qw.data, qw.inv_scale, True)
    assert rel(nc.mx_gemm(q.data, q.inv_scale, qw.data, qw.inv_scale, torch.float32), f_lt) < 1e-5


@pytest.mark.parametrize("N,C,out", [(256, 384, 512), (640, 256, 1536)])
def test_fp8_matmul_forward_backward(N, C, out):
    """Float8Matmul: y, dx and the fp32 weight gradient written straight into .grad, then accumulated by a second
    backward (Fp8.MxGradAccumulatesIntoGrad, tests/test_fp8.cpp)."""
    ref = refhost.module()
    x0, (w0,), (up,) = _inputs(N, C, [out], 2)
    res = {}
    for name, fn in (("ref", ref.fp8_matmul), ("ours", nc.fp8_matmul)):
        x, w = x0.clone().requires_grad_(), w0.clone().requires_grad_()
        y = fn(x, w)
        (y.float() * up).sum().backward()
        g1 = w.grad.clone()
        (fn(x, w).float() * up).sum().backward()  # a second micro-step: += into the same .grad
        res[name] = (y.detach(), x.grad.clone(), g1, w.grad.clone())
    for a, b, what in zip(res["ref"], res["ours"], ("y", "dx over two steps", "dw", "dw accumulated")):
        assert a.dtype == b.dtype and torch.equal(a, b), what
    assert res["ref"][2].dtype == torch.float32
    # the reference on cuBLASLt agrees with the reference on this library
    ref.set_backend("cublas")
    x, w = x0.clone().requires_grad_(), w0.clone().requires_grad_()
    y = ref.fp8_matmul(x, w)
    (y.float() * up).sum().backward()
    assert rel(res["ref"][0], y) < 2e-3
    assert rel(res["ref"][2], w.grad) < 1e-5


def test_fp8_qkv_merged():
    """MxQkv: one forward, one dgrad, one wgrad GEMM over the concatenated weights; q/k/v .grads are row blocks of
    one buffer (tests/test_qkv.cpp:29-84, tests/test_fp8.cpp:305-308)."""
    ref = refhost.module()
    N, C, gate = 640, 256, 12
    x0, ws0, ups = _inputs(N, C, [256, 128, 128], 3)
    up_gate = torch.randn(N, gate, device="cuda").to(torch.bfloat16)
    res = {}
    for name, fn in (("ref", ref.fp8_qkv), ("ours", nc.fp8_qkv)):
        x = x0.clone().requires_grad_()
        ws = [w.clone().requires_grad_() for w in ws0]
        outs = fn(x, ws[0], ws[1], ws[2], gate)
        loss = (outs[3].float() * up_gate).sum()
        for o, u in zip(outs[:3], ups):
            loss = loss + (o.float() * u).sum()
        loss.backward()
        assert ws[1].grad.data_ptr() == ws[0].grad.data_ptr() + 256 * C * 4, name
        res[name] = [o.detach() for o in outs] + [x.grad] + [w.grad for w in ws]
    assert len(res["ref"]) == len(res["ours"])
    for i, (a, b) in enumerate(zip(res["ref"], res["ours"])):
        assert torch.equal(a, b), i


@pytest.mark.parametrize("N,C,H", [(256, 256, 1024), (640, 384, 1536)])
def test_fp8_relu_square_mlp(N, C, H):
    """Fp8ReluSquareMlp, MX branch: with the Cutlass backend the reference calls the two fused-quantize GEMMs
    (mx_gemm_relu_square, mx_gemm_relu_square_bwd: fp8.cpp:279-284, 318-323), here this library's."""
    ref = refhost.module()
    g = torch.Generator(device="cuda").manual_seed(4)
    x0 = torch.randn(N, C, device="cuda", generator=g).to(torch.bfloat16)
    wf0 = torch.randn(H, C, device="cuda", generator=g) / C ** 0.5
    wp0 = torch.randn(C, H, device="cuda", generator=g) / H ** 0.5
    up = torch.randn(N, C, device="cuda", generator=g).to(torch.bfloat16)
    res = {}
    for name, fn in (("ref", ref.fp8_relu_square_mlp), ("ours", nc.fp8_relu_square_mlp)):
        x, wf, wp = x0.clone().requires_grad_(), wf0.clone().requires_grad_(), wp0.clone().requires_grad_()
        y = fn(x, wf, wp)
        (y.float() * up).sum().backward()
        res[name] = (y.detach(), x.grad, wf.grad, wp.grad)
    for a, b, what in zip(res["ref"], res["ours"], ("y", "dx", "dw_fc", "dw_proj")):
        assert torch.equal(a, b), what
    # against the reference's cuBLASLt backend, which quantizes relu^2 and its backward in separate kernels
    ref.set_backend("cublas")
    x, wf, wp = x0.clone().requires_grad_(), wf0.clone().requires_grad_(), wp0.clone().requires_grad_()
    y = ref.fp8_relu_square_mlp(x, wf, wp)
    (y.float() * up).sum().backward()
    assert rel(res["ref"][0], y) < 2e-3
    assert rel(res["ref"][1], x.grad) < 4e-3   # two quantized GEMMs deep
    assert rel(res["ref"][2], wf.grad) < 4e-3
    assert rel(res["ref"][3], wp.grad) < 1e-5 * 100  # fp32 product of re-quantized operands whose bf16 inputs differ in rare ulps


@pytest.mark.parametrize("reduction", ["mean", "sum"])
def test_softcap_cross_entropy_chunked(reduction):
    """The chunked lm_head loss (ops/softcap_ce.cpp:27-110): per chunk a logits GEMM, the loss pass, the gradient
    quantized to MX, dX; one weight-gradient GEMM over all chunks with the loss gradient as device alpha."""
    ref = refhost.module()
    N, C, V, vocab, chunk = 512, 256, 640, 600, 128
    g = torch.Generator(device="cuda").manual_seed(5)
    x0 = torch.randn(N, C, device="cuda", generator=g).to(torch.bfloat16)
    w0 = torch.randn(V, C, device="cuda", generator=g) / C ** 0.5
    t = torch.randint(0, vocab, (N,), device="cuda", generator=g)
    t[::7] = -1
    res = {}
    for name in ("ref", "ours"):
        x, w = x0.clone().requires_grad_(), w0.clone().requires_grad_()
        if name == "ref":
            loss = ref.softcap_cross_entropy(x, w, t, vocab, 15.0, chunk, reduction)
        else:
            loss = nc.softcap_cross_entropy(x, w, t, vocab, 15.0, chunk, reduction)
        (loss * 1.5).backward()
        res[name] = (loss.detach(), x.grad, w.grad)
    for a, b, what in zip(res["ref"], res["ours"], ("loss", "dx", "dw")):
        assert torch.equal(a, b), what
