"""GPU: the chunked lm_head loss path under MX, through the C ABI. The loss pass and the gradient-quantizing prologue
are bit-exact against the reference's own kernels compiled from their source (same fp32 expressions, same summation
order, same device math functions); against the CPU oracle, whose tanh / exp come from the host, the bar is a
tolerance. The chunk driver is checked as the reference checks its own (tests/test_softcap_ce.cpp:100-158)."""
import numpy as np
import pytest
import torch

import nanochat_cpp_b200 as nc
import refkernel
from helpers import assert_quantized_equal, np_f32, np_u8
from oracle import mx_oracle as mo

pytestmark = pytest.mark.gpu


def ce_inputs(rows, padded, vocab, seed=0, ignored=7):
    """tests/test_softcap_ce.cpp:124-131: logits ~ 8 N(0,1) in bf16, uniform targets, the first rows ignored, per-row
    upstream scales in [0.5, 1.5)."""
    g = torch.Generator().manual_seed(seed)
    logits = (torch.randn(rows, padded, generator=g) * 8).to(torch.bfloat16)
    targets = torch.randint(vocab, (rows,), generator=g, dtype=torch.int64)
    targets[:ignored] = -1
    grad_scale = torch.rand(rows, generator=g) + 0.5
    return logits, targets, grad_scale


@pytest.mark.parametrize("rows,padded,vocab", [(256, 512, 500), (128, 4096, 4000), (128, 128, 128)])
def test_loss_pass_matches_reference_kernel(rows, padded, vocab):
    if not refkernel.available():
        pytest.skip("reference kernel library not built")
    logits, targets, _ = ce_inputs(rows, padded, vocab)
    z, t = logits.cuda(), targets.cuda()
    loss, lse = nc.softcap_ce_loss(z, t, vocab, 15.0)
    ref_loss, ref_lse, _ = refkernel.softcap_ce(z, t, vocab, 15.0)
    valid = (t >= 0)
    assert torch.equal(loss, ref_loss)
    assert torch.equal(lse[valid], ref_lse[valid])
    o_loss, o_lse = mo.softcap_ce_loss(np_f32(logits), targets.numpy(), vocab, 15.0)
    assert np.allclose(np_f32(loss), o_loss, rtol=2e-6, atol=2e-6)
    assert np.allclose(np_f32(lse)[valid.cpu().numpy()], o_lse[valid.cpu().numpy()], rtol=1e-6)


@pytest.mark.parametrize("per_row", [False, True])
@pytest.mark.parametrize("rows,padded,vocab", [(256, 512, 500), (128, 1024, 1024)])
def test_grad_mx_matches_reference_kernel(rows, padded, vocab, per_row):
    """SoftcapCE.MxGradMatchesQuantizedGrad (tests/test_softcap_ce.cpp:121-158): the MX of the gradient from the
    logits and lse == quantize_mx of the gradient the bf16 kernel writes, both from the reference's kernels."""
    if not refkernel.available():
        pytest.skip("reference kernel library not built")
    logits, targets, grad_scale = ce_inputs(rows, padded, vocab, seed=1)
    z, t = logits.cuda(), targets.cuda()
    scale = grad_scale.cuda() if per_row else None
    valid = None if per_row else (t >= 0).sum()
    loss, lse = nc.softcap_ce_loss(z, t, vocab, 15.0)
    q = nc.empty_mx(rows, padded, z.device)
    out, out_t = nc.mx_outs(q)
    nc.softcap_ce_grad_mx(z, t, lse, vocab, 15.0, out, out_t, scale, valid)
    # the reference's MX gradient kernel on the same logits and lse
    want = dict(zip(("data", "scale", "data_t", "scale_t"),
                    (np_u8(x) for x in refkernel.softcap_ce_grad_mx(z, t, lse, vocab, 15.0, scale, valid))))
    assert_quantized_equal(q, want, f"per_row={per_row}")
    # ... and the reference's bf16 gradient kernel followed by the quantizer
    _, _, grad = refkernel.softcap_ce(z, t, vocab, 15.0, True, scale, valid)
    assert_quantized_equal(q, {k: np_u8(v) for k, v in zip(("data", "scale", "data_t", "scale_t"),
                                                              refkernel.quantize_mx(grad))}, "bf16 grad then quantize")
    assert_quantized_equal(nc.quantize_mx(grad), want, "own quantizer on the reference's bf16 gradient")


def test_grad_matches_oracle_within_rounding():
    rows, padded, vocab = 128, 256, 250
    logits, targets, grad_scale = ce_inputs(rows, padded, vocab, seed=2)
    z, t = logits.cuda(), targets.cuda()
    loss, lse = nc.softcap_ce_loss(z, t, vocab, 15.0)
    q = nc.empty_mx(rows, padded, z.device)
    out, out_t = nc.mx_outs(q)
    nc.softcap_ce_grad_mx(z, t, lse, vocab, 15.0, out, out_t, grad_scale.cuda(), None)
    g = mo.softcap_ce_grad(np_f32(logits), targets.numpy(), np_f32(lse), vocab, 15.0, grad_scale.numpy())
    want = mo.quantize_mx(g)
    got = np_u8(q.data)
    # host tanh / exp differ from the device's in the last bits: a value on a rounding boundary may land one step away
    assert (got != want["data"]).mean() < 2e-3
    assert (np_u8(q.inv_scale).reshape(-1) != want["scale"].reshape(-1)).mean() < 2e-3
    deq = mo.mx_dequantize(got, np_u8(q.inv_scale))
    assert mo.rel_norm_diff(deq, g) < 0.04  # e4m3 resolution
    assert np.all(deq[:7] == 0) and np.all(deq[:, vocab:] == 0)


def reference_loss(x, w, targets, vocab, reduction):
    """What the model does without chunking, with the matmul under MX (tests/test_softcap_ce.cpp:101-105)."""
    logits = nc.fp8_matmul(x, w)[:, :vocab].float()
    logits = 15 * torch.tanh(logits / 15)
    return torch.nn.functional.cross_entropy(logits, targets, ignore_index=-1, reduction=reduction)


@pytest.mark.parametrize("chunk", [1024, 256])
def test_chunked_loss_matches_unchunked(chunk):
    """SoftcapCE fp8 part, recipe Mx (tests/test_softcap_ce.cpp:100-119)."""
    N, C, vocab, padded = 1024, 128, 1000, 1024
    g = torch.Generator(device="cuda").manual_seed(0)
    x0 = torch.randn(N, C, device="cuda", generator=g).to(torch.bfloat16)
    w0 = torch.randn(padded, C, device="cuda", generator=g) * 0.5
    targets = torch.randint(0, vocab, (N,), device="cuda", generator=g)
    targets[:50] = -1
    x2, w2 = x0.clone().requires_grad_(), w0.clone().requires_grad_()
    want = reference_loss(x2, w2, targets, vocab, "mean")
    want.backward()
    x1, w1 = x0.clone().requires_grad_(), w0.clone().requires_grad_()
    got = nc.softcap_cross_entropy(x1, w1, targets, vocab, 15, chunk)
    got.backward()

    def rel_norm(a, b):
        return ((a.double() - b.double()).norm() / (b.double().norm() + 1e-30)).item()
    assert abs(got.item() - want.item()) / abs(want.item()) < 1e-5
    assert rel_norm(x1.grad, x2.grad) < 1e-3
    assert rel_norm(w1.grad, w2.grad) < 5e-3  # the Linear rounds grad_w's operand to bf16; the chunks keep fp32
    assert w1.grad[vocab:].abs().max().item() == 0.0
    assert w1.grad.dtype == torch.float32


@pytest.mark.parametrize("reduction", ["sum", "none"])
def test_reductions_and_upstream_gradient(reduction):
    N, C, vocab, padded = 512, 128, 500, 512
    g = torch.Generator(device="cuda").manual_seed(4)
    x0 = torch.randn(N, C, device="cuda", generator=g).to(torch.bfloat16)
    w0 = torch.randn(padded, C, device="cuda", generator=g) * 0.5
    targets = torch.randint(0, vocab, (N,), device="cuda", generator=g)
    targets[5:9] = -1
    x1, w1 = x0.clone().requires_grad_(), w0.clone().requires_grad_()
    x2, w2 = x0.clone().requires_grad_(), w0.clone().requires_grad_()
    got = nc.softcap_cross_entropy(x1, w1, targets, vocab, 15, 128, reduction)
    want = reference_loss(x2, w2, targets, vocab, reduction)
    assert ((got.double() - want.double()).abs().max() / want.double().abs().max()).item() < 1e-5
    # none: the per-row upstream gradient enters the kernel before the gradient is quantized, as it does in the unchunked
    # graph. sum: the forward has already quantized the gradient at scale 1 and the backward multiplies afterwards
    # (softcap_ce.cpp:177-183), so only a power of two reproduces the unchunked graph's e4m3 roundings
    up = torch.rand(want.shape, device="cuda", generator=g) if reduction == "none" else torch.tensor(0.5, device="cuda")
    (got * up).sum().backward()
    (want * up).sum().backward()
    rel = lambda a, b: ((a.double() - b.double()).norm() / (b.double().norm() + 1e-30)).item()
    assert rel(x1.grad, x2.grad) < 2e-3
    assert rel(w1.grad, w2.grad) < 6e-3


def test_weight_grad_accumulates_and_ignores_chunk_size():
    """SoftcapCE.WeightGradAccumulates, MX (tests/test_softcap_ce.cpp:160-200): micro-steps add into .grad; every
    chunk's transposed gradient feeds one GEMM, so the chunk size does not change the weight gradient's bits."""
    N, C, vocab, padded = 512, 128, 1000, 1024
    g = torch.Generator(device="cuda").manual_seed(0)
    w0 = torch.randn(padded, C, device="cuda", generator=g) * 0.5
    xs = [torch.randn(N, C, device="cuda", generator=g).to(torch.bfloat16) for _ in range(2)]
    targets = torch.randint(0, vocab, (N,), device="cuda", generator=g)
    grads = []
    for chunk in (512, 128):
        w = w0.clone().requires_grad_()
        for i, s in enumerate((0.5, 0.25)):
            (nc.softcap_cross_entropy(xs[i], w, targets, vocab, 15, chunk) * s).backward()
        grads.append(w.grad.clone())
    assert torch.equal(grads[0], grads[1])
    single = []
    for i, s in enumerate((0.5, 0.25)):
        w = w0.clone().requires_grad_()
        (nc.softcap_cross_entropy(xs[i], w, targets, vocab, 15, 512) * s).backward()
        single.append(w.grad)
    assert torch.allclose(grads[0], single[0] + single[1], rtol=1e-5, atol=1e-8)


def test_argument_errors():
    x = torch.zeros(128, 128, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(256, 128, device="cuda")
    t = torch.zeros(128, dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError):
        nc.softcap_cross_entropy(x, w, t, 200, 15, 100)      # chunk_rows % 128
    with pytest.raises(ValueError):
        nc.softcap_cross_entropy(x.float(), w, t, 200, 15, 128)
    with pytest.raises(ValueError):
        nc.softcap_cross_entropy(x, w, t[:64], 200, 15, 128)
    z = torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(nc.capi.Mxb200Error):
        nc.softcap_ce_loss(z, t, 300, 15.0)                   # vocab > padded
