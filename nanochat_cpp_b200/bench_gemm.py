"""Per-shape timing of the MXFP8 path, the counterpart of nanochat-cpp's tools/bench_gemm.cpp.

    python -m nanochat_cpp_b200.bench_gemm --tokens 16384 --embd 1536 [--vocab 32768] [--chunk 2048]
                                           [--only mlp_fc.fwd] [--iters 20] [--warmup 5] [--no-cublas]

Builds the GEMM shapes of one micro-step from --tokens/--embd as the reference does (tools/bench_gemm.cpp:
301-314): forward, dgrad and wgrad of the merged QKV, attention-out, MLP fc and proj Linears and of one
lm_head chunk. For each it times this library (median of 20 after 5 warm-ups, CUDA events on the launching
stream, tools/bench_gemm.cpp:46-67) next to cuBLASLt through torch._scaled_mm on the same operands, prints
microseconds, TFLOP/s (2MNK/t), the maximum absolute difference against cuBLASLt and whether two runs give
identical bits. The two MLP GEMMs whose epilogue also quantizes (relu^2 forward, relu^2 backward) are listed a second
time in that form ("+q"). It also times the quantizer on the activation shapes and the fused residual step with
achieved GB/s. --only keeps the rows whose name contains the given text (and skips the layer total), which with small
--iters/--warmup gives a profiler a short run of one kernel.
"""
from __future__ import annotations

import argparse
import json
import statistics

import torch

from . import engine as nc
from . import capi


WARMUP, ITERS = [5], [20]


def time_us(fn, warmup: int = 0, iters: int = 0) -> float:
    """Microseconds per call: `iters` back-to-back calls between one pair of CUDA events on the launching stream
    (so the host's launch cost hides behind the queue, as it does in a training step), median of three such groups."""
    warmup, iters = warmup or WARMUP[0], iters or ITERS[0]
    for _ in range(warmup):
        fn()
    groups = []
    for _ in range(3):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        b.synchronize()
        groups.append(a.elapsed_time(b) * 1e3 / iters)
    return statistics.median(groups)


def step_shapes(T: int, C: int, V: int, chunk: int):
    """(name, M, N, K, out dtype) of every GEMM of a micro-step."""
    shapes = []
    for name, n_out, k_in in (("qkv", 3 * C, C), ("attn_out", C, C), ("mlp_fc", 4 * C, C), ("mlp_proj", C, 4 * C)):
        shapes.append((f"{name}.fwd", T, n_out, k_in, torch.bfloat16))
        shapes.append((f"{name}.dgrad", T, k_in, n_out, torch.bfloat16))
        shapes.append((f"{name}.wgrad", n_out, k_in, T, torch.float32))
    rows = min(chunk, T)
    shapes.append(("lm_head.fwd_chunk", rows, V, C, torch.bfloat16))
    shapes.append(("lm_head.dgrad_chunk", rows, C, V, torch.bfloat16))
    shapes.append(("lm_head.wgrad", V, C, T, torch.float32))
    return shapes


def fused_row(name: str, M: int, N: int, K: int, kind: str, g, dev) -> dict:
    """One GEMM whose epilogue quantizes: timed, and checked bit for bit against the GEMM followed by the quantizer."""
    a = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
    b = torch.randn(N, K, generator=g, device=dev).to(torch.bfloat16)
    qa, qb = nc.quantize_mx(a, True, False), nc.quantize_mx(b, True, False)
    del a, b
    h = torch.randn(M, N, generator=g, device=dev).to(torch.bfloat16)
    q = nc.empty_mx(M, N, dev)
    if kind == "relu_square":
        def ours():
            nc.mx_gemm_relu_square(h, q.data, q.inv_scale, q.data_t, q.inv_scale_t, qa.data, qa.inv_scale, qb.data, qb.inv_scale)
    else:
        def ours():
            nc.mx_gemm_relu_square_bwd(qa.data, qa.inv_scale, qb.data, qb.inv_scale, h, q.data, q.inv_scale, q.data_t, q.inv_scale_t)
    us = time_us(ours)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    nc.mx_gemm_out(out, qa.data, qa.inv_scale, qb.data, qb.inv_scale)
    want = nc.quantize_mx(out, True, True, True) if kind == "relu_square" else nc.quantize_mx_relu_square_bwd(out, h)
    same = all(torch.equal(x.view(torch.uint8), y.view(torch.uint8)) for x, y in
               ((q.data, want.data), (q.inv_scale, want.inv_scale), (q.data_t, want.data_t), (q.inv_scale_t, want.inv_scale_t)))
    flops = 2.0 * M * N * K
    print(f"{name:22s} {M:6d} {N:6d} {K:6d} {1:6d} {us:9.1f} {flops / us / 1e6:9.1f} {'':>10s} {'':>9s} {'':>9s} "
          f"{'== gemm then quantize' if same else 'DIFFERS from gemm then quantize'}", flush=True)
    return dict(name=name, M=M, N=N, K=K, splits=1, us=us, tflops=flops / us / 1e6, cublas_us=float("nan"),
                cublas_tflops=float("nan"), maxdiff=0.0 if same else float("nan"), deterministic=same)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--embd", type=int, default=1536)
    ap.add_argument("--vocab", type=int, default=32768)
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--no-cublas", action="store_true")
    ap.add_argument("--json", type=str, default="")
    ap.add_argument("--only", type=str, default="")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args(argv)
    WARMUP[0], ITERS[0] = max(args.warmup, 1), max(args.iters, 1)
    capi.lib.mxb200_set_gemm_config(args.tile_n, 0)
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    rows = []
    print(f"{'gemm':22s} {'M':>6s} {'N':>6s} {'K':>6s} {'splits':>6s} {'us':>9s} {'TFLOP/s':>9s} {'cublas us':>10s} {'TFLOP/s':>9s} {'maxdiff':>9s} det")
    shapes = step_shapes(args.tokens, args.embd, args.vocab, args.chunk)
    # the MLP GEMMs in the form the step runs them: h = x . Wfc^T with relu(h)^2 quantized in the epilogue, and
    # dh = (dy . Wproj) * 2h quantized in the epilogue without ever being written
    T, C = args.tokens, args.embd
    shapes += [("mlp_fc.fwd+q", T, 4 * C, C, "relu_square"), ("mlp_proj.dgrad+q", T, 4 * C, C, "relu_square_bwd")]
    for name, M, N, K, dtype in shapes:
        if args.only and args.only not in name:
            continue
        if isinstance(dtype, str):
            rows.append(fused_row(name, M, N, K, dtype, g, dev))
            continue
        a = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
        b = torch.randn(N, K, generator=g, device=dev).to(torch.bfloat16)
        qa, qb = nc.quantize_mx(a, True, False), nc.quantize_mx(b, True, False)
        del a, b
        out = torch.empty(M, N, dtype=dtype, device=dev)
        splits = capi.lib.mxb200_gemm_splits(M, N, K)

        def ours():
            nc.mx_gemm_out(out, qa.data, qa.inv_scale, qb.data, qb.inv_scale, splits=splits)
        us = time_us(ours)
        first = out.clone()
        ours()
        det = torch.equal(first, out)
        cu_us, diff = float("nan"), float("nan")
        if not args.no_cublas:
            def cublas():
                return torch._scaled_mm(qa.data, qb.data.t(), qa.inv_scale, qb.inv_scale, None, None, dtype, False)
            cu_us = time_us(cublas)
            diff = (cublas().float() - first.float()).abs().max().item()
        flops = 2.0 * M * N * K
        rows.append(dict(name=name, M=M, N=N, K=K, splits=splits, us=us, tflops=flops / us / 1e6, cublas_us=cu_us,
                         cublas_tflops=flops / cu_us / 1e6, maxdiff=diff, deterministic=det))
        print(f"{name:22s} {M:6d} {N:6d} {K:6d} {splits:6d} {us:9.1f} {flops / us / 1e6:9.1f} {cu_us:10.1f} "
              f"{flops / cu_us / 1e6:9.1f} {diff:9.3g} {det}", flush=True)
        del qa, qb, out, first
    tot = t_ours = 1.0
    if not args.only:
        tot = sum(2.0 * r["M"] * r["N"] * r["K"] for r in rows[:12])
        t_ours = sum(r["us"] for r in rows[:12])
        t_cu = sum(r["cublas_us"] for r in rows[:12])
        print(f"layer total (12 GEMMs): {t_ours:.1f} us = {tot / t_ours / 1e6:.1f} TFLOP/s; cuBLASLt {t_cu:.1f} us = {tot / t_cu / 1e6:.1f} TFLOP/s")

    print(f"\n{'quantize (both layouts)':28s} {'rows':>6s} {'cols':>6s} {'us':>9s} {'GB/s':>9s}")
    qrows = []
    for name, R, Ccols in (("quantize x", args.tokens, args.embd), ("quantize dy_qkv", args.tokens, 3 * args.embd),
                           ("quantize h / dh", args.tokens, 4 * args.embd)):
        if args.only and args.only not in name:
            continue
        xs = [torch.randn(R, Ccols, generator=g, device=dev).to(torch.bfloat16) for _ in range(3)]  # > L2 in rotation
        q = nc.empty_mx(R, Ccols, dev)
        out, out_t = nc.mx_outs(q)
        i = [0]

        def quant():
            nc.quantize_mx_into(xs[i[0] % 3], False, out, out_t)
            i[0] += 1
        us = time_us(quant)
        nbytes = R * Ccols * (2 + 2 * (1 + 1 / 32))
        qrows.append(dict(name=name, rows=R, cols=Ccols, us=us, gbs=nbytes / us / 1e3))
        print(f"{name:28s} {R:6d} {Ccols:6d} {us:9.1f} {nbytes / us / 1e3:9.1f}", flush=True)
        del xs, q
    if nc.residual_norm_mx_fits(args.tokens, args.embd):
        print(f"\n{'residual step -> MX':28s} {'rows':>6s} {'cols':>6s} {'us':>9s} {'GB/s':>9s}")
        R, Ccols = args.tokens, args.embd
        lr, l0 = torch.full((4,), 0.97, device=dev), torch.full((4,), 0.11, device=dev)
        for name, n_in, n_out in (("residual_norm add+blend", 3, 2), ("residual_norm add", 2, 1), ("residual_norm plain", 1, 1)):
            if args.only and args.only not in name:
                continue
            sets = [[torch.randn(R, Ccols, generator=g, device=dev).to(torch.bfloat16) for _ in range(n_in)] for _ in range(2)]
            outs = nc.residual_norm_mx(*sets[0], lr, l0, 1) if n_in == 3 else nc.residual_norm_mx(*sets[0])
            i = [0]

            def norm():
                x = sets[i[0] % 2]
                i[0] += 1
                if n_in == 3:
                    nc.residual_norm_mx(x[0], x[1], x[2], lr, l0, 1, out=outs)
                else:
                    nc.residual_norm_mx(*x, out=outs)
            us = time_us(norm)
            nbytes = R * Ccols * (2 * n_in + 2 * n_out + 2 * (1 + 1 / 32))  # inputs, res (+ s), MX both ways
            qrows.append(dict(name=name, rows=R, cols=Ccols, us=us, gbs=nbytes / us / 1e3))
            print(f"{name:28s} {R:6d} {Ccols:6d} {us:9.1f} {nbytes / us / 1e3:9.1f}", flush=True)
            del sets
    if args.json:
        with open(args.json, "w") as f:
            json.dump(dict(gemm=rows, quantize=qrows, layer_tflops=tot / t_ours / 1e6), f, indent=1)


if __name__ == "__main__":
    main()
