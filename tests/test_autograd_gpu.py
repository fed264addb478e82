"""GPU: the autograd mirrors of nanochat-cpp's MX Linears above the C ABI: merged q/k/v (MxQkv) against three separate
Linears, and the relu^2 MLP (Fp8ReluSquareMlp, fused GEMM epilogues) against its op-by-op composition, bit for bit
where the reference's own tests ask for it (tests/test_qkv.cpp:29-84, src/nanochat/model/fp8/fp8.h:46-54)."""
import pytest
import torch

import nanochat_cpp_b200 as nc

pytestmark = pytest.mark.gpu


def rel(a, b):
    a64, b64 = a.double(), b.double()
    return ((a64 - b64).norm() / (b64.norm() + 1e-30)).item()


def mismatch(a, b):
    return (a != b).double().mean().item()


@pytest.mark.parametrize("nq,nkv", [(256, 256), (256, 128)])  # MHA, GQA (tests/test_qkv.cpp:33)
def test_qkv_matches_separate_matmuls(nq, nkv):
    """Qkv.Fp8MatchesSeparateMatmuls, MX recipe (tests/test_qkv.cpp:29-84)."""
    N, C, gate_cols = 640, 256, 12
    g = torch.Generator(device="cuda").manual_seed(0)
    x_in = torch.randn(N, C, device="cuda", generator=g).to(torch.bfloat16)
    w_in, up = [], []
    for i, n in enumerate((nq, nkv, nkv)):
        w_in.append(torch.randn(n, C, device="cuda", generator=g) * 0.05 * (1 + i))  # distinct scales
        up.append(torch.randn(N, n, device="cuda", generator=g).to(torch.bfloat16) * (1 + i))
    up_gate = torch.randn(N, gate_cols, device="cuda", generator=g).to(torch.bfloat16)

    x = x_in.clone().requires_grad_()
    w = [t.clone().requires_grad_() for t in w_in]
    out = nc.fp8_qkv(x, w[0], w[1], w[2], gate_cols)
    assert len(out) == 4
    assert torch.equal(out[3], x_in[:, :gate_cols])
    loss = (out[3].float() * up_gate).sum()
    for i in range(3):
        loss = loss + (out[i].float() * up[i]).sum()
    loss.backward()

    dx_ref = torch.zeros(N, C, dtype=torch.float64, device="cuda")
    dx_ref[:, :gate_cols] += up_gate.double()
    for i in range(3):
        xi = x_in.clone().requires_grad_()
        wi = w_in[i].clone().requires_grad_()
        o = nc.fp8_matmul(xi, wi)
        (o.float() * up[i]).sum().backward()
        assert torch.equal(out[i], o), i
        # the merged GEMM may accumulate in another order: rare 1-ulp differences
        assert mismatch(w[i].grad, wi.grad) < 1e-4, i
        assert rel(w[i].grad, wi.grad) < 4e-3, i
        dx_ref += xi.grad.double()
    assert rel(x.grad, dx_ref) < 4e-3  # one GEMM rounded once against three bf16 roundings
    assert all(t.grad.data_ptr() == w[0].grad.data_ptr() + off * C * 4
               for t, off in zip(w, (0, nq, nq + nkv)))  # row blocks of one buffer (tests/test_fp8.cpp:305-308)


def test_qkv_accumulates_over_micro_steps():
    """Fp8.MxGradAccumulatesIntoGrad, merged part (tests/test_fp8.cpp:296-309)."""
    N, cin = 512, 384
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(N, cin, device="cuda", generator=g).to(torch.bfloat16)
    ws = [(torch.randn(r, cin, device="cuda", generator=g) * 0.05).requires_grad_() for r in (128, 256, 128)]
    gs = torch.randn(N, 512, device="cuda", generator=g).to(torch.bfloat16)
    for _ in range(2):
        q, k, v = nc.fp8_qkv(x, ws[0], ws[1], ws[2])
        torch.cat([q, k, v], 1).backward(gs)
    gq, xq = nc.quantize_mx(gs), nc.quantize_mx(x)
    want = 2 * nc.mx_gemm(gq.data_t, gq.inv_scale_t, xq.data_t, xq.inv_scale_t, torch.float32)
    row = 0
    for w in ws:
        assert w.grad.data_ptr() == ws[0].grad.data_ptr() + row * cin * 4
        assert rel(w.grad, want[row:row + w.size(0)]) < 1e-6
        row += w.size(0)


@pytest.mark.parametrize("N,cin,hidden,cout", [(256, 256, 1024, 256), (512, 384, 1536, 384)])
def test_relu_square_mlp_matches_composition(N, cin, hidden, cout):
    """fp8_relu_square_mlp == fp8_matmul(relu(fp8_matmul(x, w_fc))^2, w_proj), outputs and every gradient bit for bit
    (src/nanochat/model/fp8/fp8.h:46-48; the fused epilogues are pinned by tests/test_fp8.cpp:363-426)."""
    g = torch.Generator(device="cuda").manual_seed(5)
    x_in = torch.randn(N, cin, device="cuda", generator=g).to(torch.bfloat16)
    fc_in = torch.randn(hidden, cin, device="cuda", generator=g) * cin ** -0.5
    proj_in = torch.randn(cout, hidden, device="cuda", generator=g) * hidden ** -0.5
    go = torch.randn(N, cout, device="cuda", generator=g).to(torch.bfloat16)

    x, fc, proj = x_in.clone().requires_grad_(), fc_in.clone().requires_grad_(), proj_in.clone().requires_grad_()
    y = nc.fp8_relu_square_mlp(x, fc, proj)
    y.backward(go)

    x2, fc2, proj2 = x_in.clone().requires_grad_(), fc_in.clone().requires_grad_(), proj_in.clone().requires_grad_()
    h = nc.fp8_matmul(x2, fc2)
    y2 = nc.fp8_matmul(torch.relu(h).square(), proj2)
    y2.backward(go)

    assert torch.equal(y, y2)
    assert torch.equal(x.grad, x2.grad)
    assert torch.equal(fc.grad, fc2.grad)
    assert torch.equal(proj.grad, proj2.grad)
    assert fc.grad.dtype == torch.float32
    # and close to the bf16 MLP it replaces
    ref = torch.relu(x_in.float() @ fc_in.t()).square() @ proj_in.t()
    assert rel(y.float(), ref) < 0.06


def test_relu_square_mlp_takes_prequantized_input():
    """x_mx: the input already quantized by the residual step; x then only carries autograd (fp8.h:49-50)."""
    N, C = 256, 256
    g = torch.Generator(device="cuda").manual_seed(6)
    x = torch.randn(N, C, device="cuda", generator=g).to(torch.bfloat16)
    r = torch.randn(N, C, device="cuda", generator=g).to(torch.bfloat16)
    fc = (torch.randn(4 * C, C, device="cuda", generator=g) * C ** -0.5).requires_grad_()
    proj = (torch.randn(C, 4 * C, device="cuda", generator=g) * (4 * C) ** -0.5).requires_grad_()
    res, n, n_mx, rstd, s = nc.residual_norm_mx(x, r, gate_cols=C)
    y = nc.fp8_relu_square_mlp(n, fc, proj, x_mx=n_mx)
    y2 = nc.fp8_relu_square_mlp(n, fc, proj)
    assert torch.equal(y, y2)


def test_qkv_takes_prequantized_input():
    """x_mx from the residual step feeds the merged q/k/v GEMM directly (mx_attention.cpp:45); the gate's columns come
    from the bf16 n the same kernel writes."""
    N, C, gate_cols = 256, 256, 16
    g = torch.Generator(device="cuda").manual_seed(8)
    x = torch.randn(N, C, device="cuda", generator=g).to(torch.bfloat16)
    r = torch.randn(N, C, device="cuda", generator=g).to(torch.bfloat16)
    ws = [(torch.randn(128, C, device="cuda", generator=g) * 0.05).requires_grad_() for _ in range(3)]
    res, n, n_mx, rstd, s = nc.residual_norm_mx(x, r, gate_cols=gate_cols)
    full = nc.residual_norm_mx(x, r, gate_cols=C)[1]
    a = nc.fp8_qkv(n, *ws, gate_cols=gate_cols, x_mx=n_mx)
    b = nc.fp8_qkv(full, *ws, gate_cols=gate_cols)
    assert all(torch.equal(u, v) for u, v in zip(a, b))


def test_shape_errors():
    x = torch.zeros(128, 192, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(128, 192, device="cuda")
    with pytest.raises(RuntimeError):
        nc.fp8_qkv(x, w, w, w)
    with pytest.raises(RuntimeError):
        nc.fp8_relu_square_mlp(x, w, w)
