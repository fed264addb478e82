"""GPU parity of the fused residual add + lambda blend + RMS norm with MX output, through the C ABI: bit-exact
against the reference's own CUDA kernels compiled from their source, and against the CPU oracle (with the device's
rstd handed to the oracle, since the device's rsqrt is approximate). Shapes and input combinations follow
ResidualNorm.MxMatchesQuantize (tests/test_residual_norm.cpp:161-200)."""
import numpy as np
import pytest
import torch

import nanochat_cpp_b200 as nc
import refkernel
from helpers import assert_quantized_equal, np_f32, np_u8, residual_norm_inputs
from oracle import mx_oracle as mo

pytestmark = pytest.mark.gpu
SHAPES = [(256, 768), (256, 1536), (384, 256)]          # tests/test_residual_norm.cpp:170
COMBOS = [(False, False), (True, False), (True, True)]  # (add, blend), tests/test_residual_norm.cpp:171


def run(inp, gate_cols=0):
    c = lambda t: None if t is None else t.cuda()
    return nc.residual_norm_mx(c(inp["x"]), c(inp["r"]), c(inp["x0"]), c(inp["lr"]), c(inp["l0"]), inp["layer"],
                               gate_cols)


def bits(t):
    return t.detach().view(torch.int16).cpu().numpy()


@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("add,blend", COMBOS)
@pytest.mark.parametrize("gate_cols", [0, 12])
def test_matches_reference_kernel(rows, cols, add, blend, gate_cols):
    if not refkernel.available():
        pytest.skip("reference kernel library not built")
    inp = residual_norm_inputs(rows, cols, add, blend)
    res, n, n_mx, rstd, s = run(inp, gate_cols)
    c = lambda t: None if t is None else t.cuda()
    ref = refkernel.residual_norm(c(inp["x"]), c(inp["r"]), c(inp["x0"]), c(inp["lr"]), c(inp["l0"]), inp["layer"],
                                  gate_cols)
    what = f"{rows}x{cols} add={add} blend={blend} gate={gate_cols}"
    assert np.array_equal(bits(res), bits(ref["res"])), what
    assert np.array_equal(np_f32(rstd).view(np.uint32), np_f32(ref["rstd"]).view(np.uint32)), what
    assert (s is None) == (ref["s"] is None)
    if s is not None:
        assert np.array_equal(bits(s), bits(ref["s"])), what
    want = {k: np_u8(ref[k]) for k in ("data", "scale", "data_t", "scale_t")}
    assert_quantized_equal(n_mx, want, what)
    if gate_cols:
        assert np.array_equal(bits(n[:, :gate_cols]), bits(ref["n"][:, :gate_cols])), what


@pytest.mark.parametrize("rows,cols", SHAPES + [(128, 2048), (128, 128)])
@pytest.mark.parametrize("add,blend", COMBOS + [(False, True)])
def test_matches_oracle(rows, cols, add, blend):
    inp = residual_norm_inputs(rows, cols, add, blend, seed=3)
    res, n, n_mx, rstd, s = run(inp, cols)
    f = lambda t: None if t is None else np_f32(t)
    lr, l0 = (float(inp["lr"][inp["layer"]]), float(inp["l0"][inp["layer"]])) if blend else (1.0, 0.0)
    eps = float(torch.finfo(torch.float32).eps)
    o_s, o_res, o_rstd, _ = mo.residual_norm(f(inp["x"]), f(inp["r"]), f(inp["x0"]), lr, l0, eps)
    what = f"{rows}x{cols} add={add} blend={blend}"
    assert np.array_equal(np_f32(res), o_res), what
    if s is not None:
        assert np.array_equal(np_f32(s), o_s), what
    # rsqrt.approx is within 2 ulp of the correctly rounded value
    assert np.allclose(np_f32(rstd), o_rstd, rtol=3e-7, atol=0), what
    _, _, _, o_n = mo.residual_norm(f(inp["x"]), f(inp["r"]), f(inp["x0"]), lr, l0, eps, rstd=np_f32(rstd))
    assert np.array_equal(np_f32(n), o_n), what
    assert_quantized_equal(n_mx, mo.quantize_mx(o_n), what)


@pytest.mark.parametrize("add,blend", COMBOS)
def test_special_values_match_reference_kernel(add, blend):
    """NaN, infinities, bf16 subnormals, values whose squares overflow, an all-zero row: the packed bf16 add and
    blend and the packed maximum must still give the reference kernel's bits."""
    if not refkernel.available():
        pytest.skip("reference kernel library not built")
    rows, cols = 128, 512
    inp = residual_norm_inputs(rows, cols, add, blend, seed=9)
    x = inp["x"].float()
    x[5, 17] = float("nan")
    x[6, 300] = float("inf")
    x[7, 40] = float("-inf")
    x[8, :] = 0
    x[9, 0:64] = 1e-39
    x[9, 64:128] = -3e-40
    x[10, :] = x[10, :] * 1e-38
    x[11, 100:132] = 3e38
    x[12, :] = x[12, :] * 1e19
    x[13, 33] = -0.0
    inp["x"] = x.to(torch.bfloat16)
    if add:
        r = inp["r"].float()
        r[9, 0:64] = -1e-39          # exact cancellation of subnormals
        r[10, :] = r[10, :] * 1e-38
        r[8, :] = 0
        r[14, 7] = float("nan")
        inp["r"] = r.to(torch.bfloat16)
    if blend:
        x0 = inp["x0"].float()
        x0[8, :] = 0
        x0[10, :] = x0[10, :] * 1e-37
        x0[15, 9] = float("inf")
        inp["x0"] = x0.to(torch.bfloat16)
    res, n, n_mx, rstd, s = run(inp, cols)
    c = lambda t: None if t is None else t.cuda()
    ref = refkernel.residual_norm(c(inp["x"]), c(inp["r"]), c(inp["x0"]), c(inp["lr"]), c(inp["l0"]), inp["layer"], cols)
    assert np.array_equal(bits(res), bits(ref["res"]))
    assert np.array_equal(np_f32(rstd).view(np.uint32), np_f32(ref["rstd"]).view(np.uint32))
    if s is not None:
        assert np.array_equal(bits(s), bits(ref["s"]))
    assert np.array_equal(bits(n), bits(ref["n"]))
    assert_quantized_equal(n_mx, {k: np_u8(ref[k]) for k in ("data", "scale", "data_t", "scale_t")}, "special values")


def test_mx_is_quantize_of_n_at_full_size():
    """The reference's property (tests/test_residual_norm.cpp:179-186) on the d24 activation: the MX output is
    quantize_mx of the bf16 n, both layouts."""
    rows, cols = 32 * 2048, 1536
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(rows, cols, device="cuda", generator=g).to(torch.bfloat16)
    r = torch.randn(rows, cols, device="cuda", generator=g).to(torch.bfloat16)
    x0 = torch.randn(rows, cols, device="cuda", generator=g).to(torch.bfloat16)
    lr = torch.full((24,), 0.97, device="cuda")
    l0 = torch.full((24,), 0.11, device="cuda")
    res, n, n_mx, rstd, s = nc.residual_norm_mx(x, r, x0, lr, l0, 5, cols)
    q = nc.quantize_mx(n)
    for a, b in ((n_mx.data, q.data), (n_mx.inv_scale, q.inv_scale), (n_mx.data_t, q.data_t),
                 (n_mx.inv_scale_t, q.inv_scale_t)):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    want_s = x + r
    assert torch.equal(s, want_s)
    want_res = lr[5].to(torch.bfloat16) * want_s + l0[5].to(torch.bfloat16) * x0
    assert torch.equal(res, want_res)
    want_n = torch.nn.functional.rms_norm(res.float(), (cols,), eps=torch.finfo(torch.float32).eps)
    assert (n.float() - want_n).abs().max().item() <= 2 ** -6  # one bf16 rounding of values up to ~5


def test_rejects_bad_arguments():
    x = torch.zeros(128, 192, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        nc.residual_norm_mx(x)
    x = torch.zeros(128, 2176, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        nc.residual_norm_mx(x)
    x = torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        nc.residual_norm_mx(x, x0=x)  # blend without lambdas
    with pytest.raises(RuntimeError):
        nc.residual_norm_mx(x, gate_cols=257)
    assert not nc.residual_norm_mx_fits(128, 2176) and nc.residual_norm_mx_fits(128, 2048)
