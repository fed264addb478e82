"""Device time of the benchmark step per kernel class.

    python -m nanochat_cpp_b200.step_breakdown [--steps 5]

Runs one rank's d24 step (dp_step.DpStep, the workload of bench.py) with a CUDA event on either side of every GEMM and
quantizer launch and prints, per class of launch (qkv.fwd, mlp_fc.fwd + quantize, ... in the order the step issues
them), launches per step, microseconds per launch and milliseconds per step. A launch's bracket includes the gap
before it, so the classes add up to the step. The counterpart of reading nanochat-cpp's NVTX ranges off a timeline
(src/nanochat/train/trainer.cpp:284-312) where no timeline tool is at hand.
"""
from __future__ import annotations

import argparse
import collections

import torch

from .dp_step import DpStep, StepConfig


def class_labels(cfg: StepConfig, n_weight_launches: int):
    L, chunks = cfg.n_layer, cfg.tokens // cfg.chunk_rows
    fc, pd = ("mlp_fc.fwd+q", "mlp_proj.dgrad+q") if cfg.fused_mlp else ("mlp_fc.fwd", "mlp_proj.dgrad")
    gemm = ["qkv.fwd", "attn_out.fwd", fc, "mlp_proj.fwd"] * L + ["lm_head.fwd", "lm_head.dgrad"] * chunks + ["lm_head.wgrad"]
    gemm += ["mlp_proj.wgrad", pd, "mlp_fc.dgrad", "mlp_fc.wgrad", "attn_out.dgrad", "attn_out.wgrad", "qkv.dgrad",
             "qkv.wgrad"] * L
    fwd_q = ["quantize x_attn", "quantize y_att", "quantize x_mlp"] + ([] if cfg.fused_mlp else ["quantize relu2(h)"])
    bwd_q = ["quantize dy_proj"] + ([] if cfg.fused_mlp else ["quantize dh"]) + ["quantize dy_o", "quantize dy_qkv"]
    quant = ["quantize weights"] * n_weight_launches + fwd_q * L + ["quantize x_lm"] + ["quantize dlogits"] * chunks + bwd_q * L
    return gemm, quant


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=5)
    args = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    cfg = StepConfig()
    events = {"gemm": [], "quant": []}
    on = [False]

    def hook(kind):
        def h(begin):
            if on[0]:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                events[kind].append(e)
        return h

    step = DpStep(cfg, dev, gemm_hook=hook("gemm"), quant_hook=hook("quant"))
    for i in range(3):
        step.run_step(i)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for i in range(10):
        step.run_step(3 + i)
    b.record()
    b.synchronize()
    print(f"step without per-launch events: {a.elapsed_time(b) / 10:.2f} ms")
    on[0] = True
    for i in range(args.steps):
        step.run_step(20 + i)
    torch.cuda.synchronize()
    n_quant = len(events["quant"]) // 2 // args.steps
    fixed = len(class_labels(cfg, 0)[1])
    labels = dict(zip(("gemm", "quant"), class_labels(cfg, n_quant - fixed)))
    totals = {}
    for kind, ev in events.items():
        n = len(ev) // 2 // args.steps
        assert n == len(labels[kind]), (kind, n, len(labels[kind]))
        per = collections.OrderedDict()
        for s in range(args.steps):
            for i in range(n):
                t = ev[2 * (s * n + i)].elapsed_time(ev[2 * (s * n + i) + 1])
                c = per.setdefault(labels[kind][i], [0.0, 0])
                c[0] += t
                c[1] += 1
        totals[kind] = sum(t for t, _ in per.values()) / args.steps
        for name, (t, c) in per.items():
            print(f"{name:20s} {c // args.steps:4d} launches/step {t / c * 1e3:8.1f} us each {t / args.steps:7.3f} ms/step")
    print(f"gemm {totals['gemm']:.2f} ms/step, quantize {totals['quant']:.2f} ms/step")


if __name__ == "__main__":
    main()
