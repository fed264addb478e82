"""GPU: the benchmark's step (nanochat_cpp_b200/dp_step.py) in its variants, on a small model: the weight gradients as
one bf16 write into the reference's stacked send buffers against fp32 `+=` into .grad followed by the cast
(src/nanochat/model/fp8/fp8.cpp:470-514, src/nanochat/train/optim.cpp:459), the same GEMM list through cuBLASLt, and
the step fed by the fused residual step and the softcap loss kernels instead of ready-made tensors."""
import pytest
import torch

import nanochat_cpp_b200 as nc
from nanochat_cpp_b200.dp_step import DpStep, StepConfig

pytestmark = pytest.mark.gpu


def small(**kw):
    return StepConfig(n_layer=2, n_embd=256, vocab=512, tokens=512, chunk_rows=256, **kw)


def rel(a, b):
    a64, b64 = a.double(), b.double()
    return ((a64 - b64).norm() / (b64.norm() + 1e-30)).item()


def test_bf16_bucket_equals_fp32_accumulate_then_cast():
    dev = torch.device("cuda", 0)
    a = DpStep(small(), dev)
    a.run_step(0)
    direct = a.bucket.buffer.clone()
    b = DpStep(small(wgrad_fp32_accumulate=True), dev)
    b.run_step(0)
    assert torch.equal(b.bucket.buffer, direct)  # one rounding of the same fp32 accumulators either way
    first = [g.clone() for g in b.grads[1]]
    b.run_step(0)  # a second micro-step accumulates
    for g, f in zip(b.grads[1], first):
        assert torch.equal(g, 2 * f)
    # the layout: layer 1's merged QKV gradient sits in entries 4..6 of the (C, C) stack, attention out in entry 7
    C = a.cfg.n_embd
    assert torch.equal(a.bucket.stacks["muon_CxC"][4:7].reshape(3 * C, C), a.bucket.matrix(1, 0))
    assert a.bucket.matrix(1, 1).data_ptr() == a.bucket.stacks["muon_CxC"][7].data_ptr()
    assert nc.capi.device_status() == 0


def test_gemm_list_through_cublaslt_agrees():
    dev = torch.device("cuda", 0)
    s = DpStep(small(), dev)
    s.run_step(0)
    s.run_gemms_only("b200")
    ours = (s.qkv.clone(), s.dx.clone(), s.bucket.matrix(0, 2).clone(), s.bucket.lm_head().clone())
    s.run_gemms_only("cublaslt")
    theirs = (s.qkv, s.dx, s.bucket.matrix(0, 2), s.bucket.lm_head())
    for x, y in zip(ours, theirs):
        assert rel(x, y) < 2e-3


def test_step_with_real_producers():
    dev = torch.device("cuda", 0)
    s = DpStep(small(real_producers=True), dev)
    s.run_step(0)
    s.run_step(1)
    st = s._producers()
    # the fused residual step's MX output is what the quantizer gives for its normalized rows
    res, n, n_mx, rstd, summed = st["mlp_out"][1]
    assert n_mx is s.xq_mlp[1]
    which = (1 + 1) % len(s.x_mlp)  # the input set of layer 1 in step 1
    x, r = s.x_mlp[which], s.resid[which]
    want_res = (x.float() + r.float()).to(torch.bfloat16)
    assert torch.equal(res, want_res)
    normed = (want_res.float() * rstd[:, None]).to(torch.bfloat16)
    want = nc.quantize_mx(normed)
    assert torch.equal(n_mx.data.view(torch.uint8), want.data.view(torch.uint8))
    assert torch.equal(n_mx.inv_scale_t.view(torch.uint8), want.inv_scale_t.view(torch.uint8))
    assert torch.isfinite(st["loss"]).all() and float(st["loss"].mean()) > 0
    assert torch.isfinite(s.bucket.buffer.float()).all()
    assert nc.capi.device_status() == 0


def test_graph_replay_equals_eager_launches():
    """capture() records the step once per phase of the input rotation; a replay writes the bytes the eager launches
    write, for both phases and for the fp32-accumulate form after a re-capture."""
    dev = torch.device("cuda", 0)
    s = DpStep(small(), dev)
    eager = []
    for k in range(2):
        s.run_step(k, eager=True)
        eager.append((s.bucket.buffer.clone(), s.qkv.clone(), s.dx.clone(), s.gq_4c.data_t.clone().view(torch.uint8)))
    s.capture()
    assert s.launches_per_step > 0
    for k in (0, 1, 2, 3):
        s.bucket.buffer.zero_()
        s.run_step(k)
        want = eager[k % 2]
        got = (s.bucket.buffer, s.qkv, s.dx, s.gq_4c.data_t.view(torch.uint8))
        for g, w in zip(got, want):
            assert torch.equal(g, w)
    s.set_wgrad_fp32_accumulate(True)  # drops the graphs: the next step is launched eagerly
    s.run_step(0)
    s.capture()
    base = [g.clone() for g in s.grads[1]]
    s.run_step(0)
    for g, b in zip(s.grads[1], base):
        assert torch.equal(g, 2 * b)
    assert torch.equal(s.bucket.buffer, 2 * eager[0][0])  # the cast of gradients accumulated over two micro-steps
    assert nc.capi.device_status() == 0
