"""Writes the golden fixtures of tests/golden/ on a machine with a B200.

    make -C oracle && python tests/golden/make_golden.py [outdir]

quantize_*.npz: a seeded CPU-drawn input and the bytes the reference's OWN CUDA quantizer
(nanochat_mx_quantize_* of src/nanochat/model/fp8/fp8_kernel.cu, compiled unmodified by oracle/Makefile into
oracle/_ref/) wrote for it on the GPU, both layouts. gemm_*.npz: quantized operands and the fp32 result of
cuBLASLt's MXFP8 GEMM (torch._scaled_mm, the arithmetic of the reference's --gemm=cublas backend,
src/nanochat/model/fp8/mx_gemm.cpp:158). residual_norm_*.npz: seeded inputs of the fused residual step and what the
reference's own nanochat_residual_norm_mx_fwd_c* / nanochat_residual_norm_fwd_c* kernels
(src/nanochat/model/ops/residual_norm_kernel.cu, compiled unmodified) wrote for them: s, res, rstd, the MX bytes of n in
both layouts, and n itself from the plain kernel. softcap_ce_*.npz: bf16 logits, targets and per-row scales with what
the reference's nanochat_softcap_ce_loss / nanochat_softcap_ce_loss_grad / nanochat_softcap_ce_grad_mx kernels
(src/nanochat/model/ops/softcap_ce_kernel.cu, compiled unmodified) gave: loss, lse, the bf16 gradient and its MX bytes.
The CPU test suite checks the oracle against these files.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import refkernel  # noqa: E402
from helpers import gemm_operands, quantizer_input, residual_norm_inputs  # noqa: E402


def bits(t):
    return t.view(torch.int16).numpy().view(np.uint16)


def main():
    out = sys.argv[1] if len(sys.argv) > 1 else HERE
    os.makedirs(out, exist_ok=True)
    assert refkernel.available(), "build oracle/_ref first (make -C oracle)"
    cases = [("bf16_128x128", 128, 128, torch.bfloat16, 0), ("bf16_256x384", 256, 384, torch.bfloat16, 0),
             ("relu2_256x384", 256, 384, torch.bfloat16, 1), ("f32_128x256", 128, 256, torch.float32, 0),
             ("relu2bwd_128x256", 128, 256, torch.bfloat16, 2)]
    for name, R, C, dtype, pro in cases:
        x = quantizer_input(R, C, seed=100 + R + C + pro).to(dtype)
        x[2, 3] = float("nan")
        x[3, 70] = float("inf")
        rec = {"prologue": np.int32(pro)}
        h = None
        if pro == 2:
            h = torch.randn(R, C, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
            rec["h_bf16_bits"] = bits(h)
        if dtype == torch.bfloat16:
            rec["x_bf16_bits"] = bits(x)
        else:
            rec["x_f32"] = x.numpy()
        data, scale, data_t, scale_t = refkernel.quantize_mx(x.cuda(), pro == 1, None if h is None else h.cuda())
        torch.cuda.synchronize()
        rec.update(data=data.cpu().numpy(), scale=scale.cpu().numpy(), data_t=data_t.cpu().numpy(), scale_t=scale_t.cpu().numpy())
        np.savez_compressed(os.path.join(out, f"quantize_{name}.npz"), **rec)
        print("wrote", name)
    for R, C, add, blend in [(128, 256, True, True), (128, 384, True, False), (128, 128, False, False)]:
        inp = residual_norm_inputs(R, C, add, blend, seed=21)
        c = lambda t: None if t is None else t.cuda()
        args = (c(inp["x"]), c(inp["r"]), c(inp["x0"]), c(inp["lr"]), c(inp["l0"]), inp["layer"])
        mx = refkernel.residual_norm(*args, gate_cols=0, mx=True)
        plain = refkernel.residual_norm(*args, mx=False)
        torch.cuda.synchronize()
        assert torch.equal(mx["res"], plain["res"]) and torch.equal(mx["rstd"], plain["rstd"])
        rec = {"x_bf16_bits": bits(inp["x"]), "eps": np.float32(torch.finfo(torch.float32).eps),
               "lr": np.float32(inp["lr"][inp["layer"]] if blend else 1), "l0": np.float32(inp["l0"][inp["layer"]] if blend else 0),
               "res_bf16_bits": bits(mx["res"].cpu()), "n_bf16_bits": bits(plain["n"].cpu()), "rstd": mx["rstd"].cpu().numpy()}
        if add:
            rec["r_bf16_bits"] = bits(inp["r"])
        if blend:
            rec["x0_bf16_bits"] = bits(inp["x0"])
        if mx["s"] is not None:
            rec["s_bf16_bits"] = bits(mx["s"].cpu())
        rec.update({k: mx[k].cpu().numpy() for k in ("data", "scale", "data_t", "scale_t")})
        name = f"{R}x{C}" + ("_add" if add else "") + ("_blend" if blend else "")
        np.savez_compressed(os.path.join(out, f"residual_norm_{name}.npz"), **rec)
        print("wrote residual_norm", name)
    for rows, padded, vocab, per_row in [(128, 256, 250, True), (128, 128, 128, False)]:
        g = torch.Generator().manual_seed(31 + padded)
        logits = (torch.randn(rows, padded, generator=g) * 8).to(torch.bfloat16)
        targets = torch.randint(vocab, (rows,), generator=g, dtype=torch.int64)
        targets[:5] = -1
        grad_scale = torch.rand(rows, generator=g) + 0.5
        z, t = logits.cuda(), targets.cuda()
        scale = grad_scale.cuda() if per_row else None
        valid = None if per_row else (t >= 0).sum()
        loss, lse, _ = refkernel.softcap_ce(z, t, vocab, 15.0)
        _, _, grad = refkernel.softcap_ce(z, t, vocab, 15.0, True, scale, valid)
        mx = refkernel.softcap_ce_grad_mx(z, t, lse, vocab, 15.0, scale, valid)
        torch.cuda.synchronize()
        lse = torch.where(t >= 0, lse, torch.zeros_like(lse))  # unset for ignored rows
        rec = {"logits_bf16_bits": bits(logits), "targets": targets.numpy(), "vocab": np.int32(vocab),
               "softcap": np.float32(15.0), "loss": loss.cpu().numpy(), "lse": lse.cpu().numpy(),
               "grad_bf16_bits": bits(grad.cpu()), "num_valid": np.int64(0 if per_row else int(valid.item()))}
        if per_row:
            rec["grad_scale"] = grad_scale.numpy()
        rec.update({k: v.cpu().numpy() for k, v in zip(("data", "scale", "data_t", "scale_t"), mx)})
        np.savez_compressed(os.path.join(out, f"softcap_ce_{rows}x{padded}.npz"), **rec)
        print("wrote softcap_ce", rows, padded)
    for M, N, K in [(128, 128, 128), (256, 384, 512)]:
        a, b = gemm_operands(M, N, K)
        qa = refkernel.quantize_mx(a.cuda())
        qb = refkernel.quantize_mx(b.cuda())
        e4, e8 = torch.float8_e4m3fn, torch.float8_e8m0fnu
        d = torch._scaled_mm(qa[0].view(e4), qb[0].view(e4).t(), qa[1].view(e8), qb[1].view(e8), None, None, torch.float32, False)
        np.savez_compressed(os.path.join(out, f"gemm_{M}x{N}x{K}.npz"), a=qa[0].cpu().numpy(), a_scale=qa[1].cpu().numpy(),
                            b=qb[0].cpu().numpy(), b_scale=qb[1].cpu().numpy(), d_f32=d.cpu().numpy())
        print("wrote gemm", M, N, K)


if __name__ == "__main__":
    main()
