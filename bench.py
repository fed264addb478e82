"""Benchmark of the MXFP8 Linear path on B200: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is one rank's data-parallel GEMM workload of a d24 nanochat training step: every Linear of 24 layers
(merged QKV, attention out, MLP fc, MLP proj) plus the lm_head in 2048-row chunks, each forward, dgrad and
wgrad, with all MX quantizations of activations, gradients and (once per step) weights, weight gradients
written as bf16 into the reference's stacked send buffers and, for N > 1, reduce-scattered segment by segment
(whole matrices per rank) over NCCL while backward continues
(71.74 TFLOP of GEMM per rank and step). Inputs are seeded synthetic tensors of the BASELINE shapes and
distributions; there is no dataset or checkpoint on this path.

value: GEMM TFLOP/s of the whole job (all ranks), from device time of the timed steps, inputs resident in HBM. The
timed steps replay CUDA graphs of the step, captured after eager warm-up steps (--no-graph launches every kernel from
the host instead). The steps are then run a second time, launched from the host, with CUDA events around every launch,
which gives the per-kernel durations.
e2e: the same with one full set of every per-step input (activations, residual, incoming gradients, lm_head
activations and logit gradients: everything but the weights) copied from pinned host memory inside the timed region
(on a copy stream, one step ahead, as a loader would) and a slice of the result read back every step. roofline: the GEMM kernel alone, bracketed by CUDA events on its stream.
cpu_baseline / --impl reference: the reference's CPU formulation of the path (libtorch quantize -> dequantize ->
fp32 matmul, oracle/torch_reference.py) on a bounded sample, on the host cores.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "MXFP8 linear TFLOP/s/GPU, d24 fwd+dgrad+wgrad shapes, % of FP8 tensor peak"
WORKLOAD = "d24 data-parallel step GEMM set: 24 x (QKV, attn-out, MLP fc, MLP proj) + lm_head in 2048-row chunks, fwd+dgrad+wgrad, M=16384 tokens/rank"
# 2MNK over the step's 305 GEMMs: 24 layers x 3 x 2 x 16384 x 12 x 1536^2 + lm_head 3 x 2 x 16384 x 32768 x 1536
STEP_TFLOP = (24 * 3 * 2.0 * 16384 * 12 * 1536 ** 2 + 3 * 2.0 * 16384 * 32768 * 1536) / 1e12
NCCL_MAX_CTAS = 0  # cap on the CTAs NCCL may use per collective (0: NCCL's default, which measured best: a cap of 8
                   # or 4 slows the collective more than it frees SMs for the GEMMs it overlaps)
FP8_SPEC_TFLOPS = 4500.0  # B200 dense FP8, 2x the 2.25e15 bf16 figure
# dram__bytes_read.sum + dram__bytes_write.sum of one captured launch of the GEMM kernel, the merged-QKV forward
# (M=16384, N=4608, K=1536, bf16 out: 45.2 MB read + 100.2 MB written), from the ncu summary of the CTA-pair kernels kept
# under profiles/ (ncu cannot run inside this benchmark, so the figure is carried here). Its algorithmic bytes: 184.3e6.
GEMM_TRAFFIC_BYTES = 145.4e6
GEMM_TRAFFIC_LAUNCH = "qkv.fwd 16384x4608x1536 (algorithmic 184.3 MB; the step's other launches differ in shape)"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "200"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])), mx.append(float(f[2])), power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [s for s, p in zip(sm, power) if p > 300] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------------------------- CPU arm

def cpu_reference_sample(min_seconds: float = 10.0, max_seconds: float = 30.0):
    """The reference's CPU formulation on a bounded sample of the workload: the merged-QKV Linear of one d24
    layer (N = 4608, K = 1536) on a 2048-token slice, forward + dgrad + wgrad, repeated until min_seconds.
    Returns (TFLOP/s, cores, description)."""
    import torch
    from oracle import torch_reference as tr
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)
    M, N, K = 2048, 4608, 1536
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g) / K ** 0.5
    dy = (torch.randn(M, N, generator=g) * 1e-3).to(torch.bfloat16)
    flops = 3 * 2.0 * M * N * K
    tr.linear_forward(x, w)  # warm-up
    t0, reps = time.perf_counter(), 0
    while True:
        tr.linear_forward(x, w)
        tr.linear_backward(x, w, dy)
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= min_seconds or dt >= max_seconds:
            break
    return flops * reps / dt / 1e12, cores, (f"d24 merged-QKV Linear (N=4608, K=1536) on a 2048-token slice, fwd+dgrad+wgrad incl. "
                                             f"quantize/dequantize, x{reps} in {dt:.1f} s")


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times = []
    tflops = cores = sample = None
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        tflops, cores, sample = cpu_reference_sample(min_seconds=2.0, max_seconds=6.0)
        if i >= args.warmup:
            times.append((time.perf_counter() - t0, tflops))
    value = statistics.mean(t for _, t in times)
    sample_ms = statistics.mean(d for d, _ in times) * 1e3
    step_tflop = STEP_TFLOP
    ms = step_tflop / value * 1e3  # what one whole step would take at the sampled rate
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "tflop_per_rank_step": step_tflop,
                       "note": "CPU formulation timed on a bounded sample per step; ms_per_step = the step's flops at the sampled rate",
                       "sample_ms_per_step": sample_ms},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------- GPU arm

def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    import nanochat_cpp_b200 as nc
    from nanochat_cpp_b200.dp_step import DpStep, StepConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the MXFP8 engine has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    nccl_max_ctas = int(os.environ.get("MXB200_NCCL_MAX_CTAS", str(NCCL_MAX_CTAS)))
    if world > 1:
        # The collective overlaps GEMMs that want every SM (one CTA pair per TPC, all of shared memory): cap the CTAs
        # NCCL's reduce-scatter kernel may take, so that it delays few tiles while it runs.
        opts = dist.ProcessGroupNCCL.Options()
        if nccl_max_ctas > 0:
            opts.config.max_ctas = nccl_max_ctas
        if os.environ.get("MXB200_NCCL_CGA"):
            opts.config.cga_cluster_size = int(os.environ["MXB200_NCCL_CGA"])
        dist.init_process_group("nccl", device_id=device, pg_options=opts)

    cfg = StepConfig()
    gemm_events, quant_events = [], []
    collect = [False]
    last_end = [None]

    def make_hook(store):
        # One event per launch boundary: the event that ends a launch doubles as the start of the next one (the step's
        # launches follow each other on one stream), which halves what the instrumentation adds to the stream.
        def h(begin: bool):
            if not collect[0]:
                return
            if begin and last_end[0] is not None:
                ev = last_end[0]
            else:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
            store.append(ev)
            last_end[0] = None if begin else ev
        return h

    hook, qhook = make_hook(gemm_events), make_hook(quant_events)
    step = DpStep(cfg, device, rank, world, gemm_hook=hook, quant_hook=qhook)
    flops = cfg.flops_per_step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: the timed region carries no per-launch events (an event record per launch boundary
    # costs a few percent of a step)
    # The timed steps replay CUDA graphs of the step (one per phase of the input rotation; captured after eager steps
    # have configured the kernels): the same launches, and at N > 1 the same collectives on their side stream, without
    # the host between them. Warm-up runs both forms.
    use_graph = not args.no_graph
    for i in range(max(args.warmup, 1) if use_graph else args.warmup):  # a capture needs one eager step before it
        step.run_step(i, eager=True)
    if use_graph:
        barrier()
        try:
            step.capture()
            captured = 1
        except Exception as e:  # a driver or library that cannot capture the step: fall back to host launches
            print(f"bench.py: graph capture failed on rank {rank} ({e!r:.300}); launching from the host", file=sys.stderr)
            step.release()
            captured = 0
        if world > 1:  # all ranks run the same form
            agreed = torch.tensor([captured], device=device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            captured = int(agreed.item())
        if not captured:
            step.release()
            use_graph = False
        for i in range(args.warmup):
            step.run_step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = nc.capi.launch_count()
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_begin.record()
    for i in range(args.steps):
        step.run_step(args.warmup + i)
    t_end.record()
    barrier()
    # a replayed graph launches the kernels counted while it was captured
    launches = step.launches_per_step * args.steps if use_graph else nc.capi.launch_count() - launches0
    ms_total = t_begin.elapsed_time(t_end)

    # ---- the same steps once more with CUDA events around every GEMM and quantizer launch: the per-kernel durations
    # behind `roofline` and `quantizer` (clocks are still being sampled, so both regions share one clock record)
    collect[0] = True
    i_begin, i_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    i_begin.record()
    for i in range(args.steps):
        step.run_step(args.warmup + args.steps + i, eager=True)
    i_end.record()
    barrier()
    collect[0] = False
    clocks = sampler.stop() if rank == 0 else None
    instrumented_ms = i_begin.elapsed_time(i_end)
    gemm_ms = sum(gemm_events[i].elapsed_time(gemm_events[i + 1]) for i in range(0, len(gemm_events), 2))
    n_gemm = len(gemm_events) // 2
    quant_ms = sum(quant_events[i].elapsed_time(quant_events[i + 1]) for i in range(0, len(quant_events), 2))
    n_quant = len(quant_events) // 2
    watchdog = nc.capi.device_status()

    # ---- comparators, one rank only: (1) the step's GEMMs alone, back to back, through this library and through
    # cuBLASLt's MXFP8 GEMM (torch._scaled_mm, what the reference's --gemm=cublas calls) on the same operands;
    # (2) cuBLASLt MXFP8 at 8192^3 run for about two seconds: a measured FP8 GEMM rate of this GPU under its power cap;
    # (3) the step with the reference's default weight-gradient form (fp32 += into .grad, then the cast into the bucket)
    extra = {}
    if world == 1 and not args.no_comparators:
        def timed_ms(fn, reps):
            fn()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            for _ in range(reps):
                fn()
            b.record()
            b.synchronize()
            return a.elapsed_time(b) / reps
        extra["gemm_only_ms"] = timed_ms(lambda: step.run_gemms_only("b200"), 3)
        try:
            extra["cublaslt_ms"] = timed_ms(lambda: step.run_gemms_only("cublaslt"), 3)
        except Exception as e:  # a torch build without the MXFP8 _scaled_mm path
            extra["cublaslt_error"] = repr(e)[:200]
        try:
            n = 8192
            qa = nc.quantize_mx(torch.randn(n, n, device=device).to(torch.bfloat16), True, False)
            qb = nc.quantize_mx(torch.randn(n, n, device=device).to(torch.bfloat16), True, False)
            out = torch.empty(n, n, dtype=torch.bfloat16, device=device)

            def burst():
                for _ in range(50):
                    torch._scaled_mm(qa.data, qb.data.t(), qa.inv_scale, qb.inv_scale, None, None, torch.bfloat16, False, out=out)
            ms50 = timed_ms(burst, 1)
            reps = max(int(2000.0 / max(ms50, 1e-3)), 2)
            extra["fp8_cublaslt_8192_tflops"] = 50 * 2.0 * n ** 3 / (timed_ms(burst, reps) * 1e-3) / 1e12
            del qa, qb, out
        except Exception as e:
            extra["fp8_cublaslt_error"] = repr(e)[:200]
        k = [0]

        def acc_step():
            step.run_step(k[0])
            k[0] += 1

        def other_form_ms():  # the step in another form, launched as the timed steps are
            step.run_step(0, eager=True)
            if use_graph:
                step.capture()
            return timed_ms(acc_step, min(args.steps, 5))
        step.set_wgrad_fp32_accumulate(True)
        extra["fp32_accumulate_ms"] = other_form_ms()
        step.set_wgrad_fp32_accumulate(False)
        step.cfg.real_producers = True
        extra["real_producers_ms"] = other_form_ms()
        step.cfg.real_producers = False
        step.release()
        if use_graph:
            step.capture()
        watchdog = watchdog or nc.capi.device_status()

    # ---- end to end: one full set of every per-step input of the path (the activations and residual each Linear
    # reads, the gradients each backward reads, the lm_head's activations and a chunk of logit gradients; everything but
    # the weights, which are parameters) comes from pinned host memory and a result slice goes back. As a training
    # loop's loader would, the copy of step i + 1's inputs runs on a copy stream into staging buffers while step i
    # computes; the step then takes them with a device-side copy. All of it is inside the timed region.
    targets = (step.x_attn[0], step.y_att[0], step.x_mlp[0], step.resid[0], step.dy_proj[0], step.dy_o[0], step.dy_qkv[0],
               step.x_lm, step.dlogits[0])
    host_in = [t.cpu().pin_memory() for t in targets]
    staging = [torch.empty_like(t) for t in targets]
    host_out = torch.empty(4096, dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = host_out.numel() * host_out.element_size()
    copy_stream = torch.cuda.Stream(device=device)
    staged = torch.cuda.Event()
    taken = torch.cuda.Event()

    def prefetch():
        copy_stream.wait_event(taken)  # the staging buffers' previous contents have been consumed
        with torch.cuda.stream(copy_stream):
            for dst, src in zip(staging, host_in):
                dst.copy_(src, non_blocking=True)
            staged.record()

    def e2e_step(i, last):
        torch.cuda.current_stream().wait_event(staged)
        for dst, src in zip(targets, staging):
            dst.copy_(src)
        taken.record()
        if not last:
            prefetch()
        step.run_step(0)
        host_out.copy_((step.bucket.shards[0] if world > 1 else step.bucket.buffer)[:4096], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    taken.record()
    prefetch()
    e2e_step(0, False)
    barrier()
    e_begin, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_begin.record()
    for i in range(args.steps):
        e2e_step(i, i == args.steps - 1)
    e_end.record()
    barrier()
    e2e_ms = e_begin.elapsed_time(e_end)

    times = torch.tensor([ms_total, e2e_ms, gemm_ms, quant_ms, instrumented_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, gemm_ms, quant_ms, instrumented_ms = times.tolist()

    if rank == 0:
        peaks = measured_peaks()
        ms_per_step = ms_total / args.steps
        value = flops * world / (ms_per_step * 1e-3) / 1e12
        e2e_value = flops * world / (e2e_ms / args.steps * 1e-3) / 1e12
        achieved = flops * args.steps / (gemm_ms * 1e-3) / 1e12
        fp8_2x = 2.0 * peaks["bf16_sustained"]
        fp8_lt = extra.get("fp8_cublaslt_8192_tflops")
        # denominator: the larger of the two measured stand-ins for this GPU's sustained FP8 GEMM rate
        fp8_peak = max(fp8_2x, fp8_lt or 0.0)
        peak_source = (f"cuBLASLt MXFP8 8192^3 run for ~2 s in this process ({fp8_lt:.0f} TFLOP/s)" if fp8_lt and fp8_lt >= fp8_2x
                       else f"2 x bf16_tflops_sustained of {peaks['source']} ({fp8_2x:.0f} TFLOP/s)")
        cpu = None
        if world == 1 and not args.no_comparators:
            v, cores, sample = cpu_reference_sample()
            cpu = {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample}
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8_e4m3 (ue8m0 block scales, fp32 accumulate)", "data": "synthetic",
            "config": {"workload": WORKLOAD, "tflop_per_rank_step": flops / 1e12, "global_tokens": cfg.tokens * world,
                       "parallelism": f"dp{world}",
                       "launch": "CUDA graph replay of the step" if use_graph else "every kernel launched from the host",
                       "l2": "operands and outputs of every launch exceed or rotate past the 126 MB L2 (9+ GB touched per step)",
                       "collective": (f"bf16 reduce-scatter (avg) of whole matrices per rank in the reference's stack segments over NCCL "
                                      f"({'NCCL default CTAs' if nccl_max_ctas <= 0 else 'max ' + str(nccl_max_ctas) + ' CTAs'}), overlapped with backward") if world > 1 else "none (1 rank)"},
            "per_gpu_tflops": value / world,
            "pct_of_fp8_spec_peak": 100.0 * value / world / FP8_SPEC_TFLOPS,
            "pct_of_2x_measured_bf16_sustained": 100.0 * value / world / fp8_2x,
            "value_is": "whole-job aggregate over n_gpus; per_gpu_tflops is the metric's per-GPU figure",
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "kernel": "mxb200_gemm_pair_256x256 / _256x192 (+ _relu_square, _relu_square_bwd)", "achieved": achieved, "peak": fp8_peak,
                         "unit": "TFLOP/s", "frac": achieved / fp8_peak, "traffic": GEMM_TRAFFIC_BYTES,
                         "traffic_launch": GEMM_TRAFFIC_LAUNCH,
                         "peak_source": peak_source, "peak_2x_bf16_sustained": fp8_2x, "peak_cublaslt_mxfp8_8192": fp8_lt,
                         "frac_of_fp8_spec_4500": achieved / FP8_SPEC_TFLOPS,
                         "launches": n_gemm, "avg_launch_us": gemm_ms * 1e3 / max(n_gemm, 1)},
            "quantizer": {"bound": "hbm", "kernel": "mxb200_quantize_bf16_stream / mxb200_quantize_batch_f32", "achieved": cfg.quantized_bytes_per_step() * args.steps / (quant_ms * 1e-3) / 1e9,
                          "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": cfg.quantized_bytes_per_step() * args.steps / (quant_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                          "launches": n_quant, "ms_per_step": quant_ms / args.steps, "gb_per_step": cfg.quantized_bytes_per_step() / 1e9},
            "ms_per_step_split": {"gemm": gemm_ms / args.steps, "quantize": quant_ms / args.steps,
                                  "other": instrumented_ms / args.steps - (gemm_ms + quant_ms) / args.steps,
                                  "instrumented_ms_per_step": instrumented_ms / args.steps,
                                  "note": "from a second pass over the same steps with CUDA events around every launch; value and ms_per_step come from the pass without them"},
            "watchdog": watchdog,
        }
        if "gemm_only_ms" in extra:
            line["roofline"]["gemm_only_tflops"] = flops / (extra["gemm_only_ms"] * 1e-3) / 1e12
            line["roofline"]["gemm_only_note"] = ("the step's 305 GEMMs back to back, plain epilogues, no quantizer launches; "
                                                  "cublaslt_tflops is the same list through torch._scaled_mm (no residual add)")
        if "cublaslt_ms" in extra:
            line["roofline"]["cublaslt_tflops"] = flops / (extra["cublaslt_ms"] * 1e-3) / 1e12
            line["roofline"]["frac_of_cublaslt"] = extra["cublaslt_ms"] / extra["gemm_only_ms"]
        for key in ("cublaslt_error", "fp8_cublaslt_error"):
            if key in extra:
                line["roofline"][key] = extra[key]
        if "fp32_accumulate_ms" in extra:
            line["wgrad_fp32_accumulate"] = {"ms_per_step": extra["fp32_accumulate_ms"],
                                             "value": flops / (extra["fp32_accumulate_ms"] * 1e-3) / 1e12, "unit": "TFLOP/s",
                                             "note": "the same step with every weight gradient as fp32 += into .grad and a cast into the bucket; "
                                                     "`value` above uses the single bf16 write into the bucket"}
        if "real_producers_ms" in extra:
            line["real_producers"] = {"ms_per_step": extra["real_producers_ms"],
                                      "value": flops / (extra["real_producers_ms"] * 1e-3) / 1e12, "unit": "TFLOP/s",
                                      "note": "the same step with the kernels a training step runs in front of the GEMMs: the fused residual "
                                              "add + blend + RMS norm emitting MX for the QKV and MLP-fc inputs, and in the lm_head the softcap "
                                              "loss pass + gradient quantized from the logits; `value` above uses BASELINE's ready-made tensors "
                                              "and the plain quantizer"}
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if watchdog != 0:
            line["invalid"] = f"a bounded device wait ran out (status word {watchdog:#x}): results are not trusted"
        print(json.dumps(line), flush=True)
    # the graphs hold the collectives they captured: they go before the communicator does
    step.release()
    gc.collect()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if watchdog != 0:
        raise SystemExit(3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", type=str, default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every kernel of the timed steps from the host instead of replaying CUDA graphs of the step")
    ap.add_argument("--no-comparators", action="store_true",
                    help="skip the cuBLASLt / fp32-accumulate / CPU legs (a short run of the step alone, for a profiler)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
