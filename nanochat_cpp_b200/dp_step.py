"""The data-parallel GEMM workload of one nanochat training step, on one rank.

Every Linear of a depth-`n_layer` nanochat model (merged QKV, attention out, MLP fc, MLP proj; then the
chunked lm_head) runs forward, dgrad and wgrad through the MXFP8 engine on this rank's own micro-batch, the
weight gradients leave as bf16 straight into the reference's stacked send buffers, and every segment of whole
matrices is reduce-scattered (average) across ranks as soon as backward has produced it, while backward goes on. Nothing else of the model runs:
attention, norms and the loss are outside this path, so their outputs are seeded synthetic tensors of the
right shape and distribution.

Call sites mirrored (paths within nanochat-cpp): the per-Linear sequence of src/nanochat/model/fp8/fp8.cpp:
240-260 (Float8Matmul), 424-462 (MxQkv), 265-338 (Fp8ReluSquareMlp, MX branch), the chunked lm_head of
src/nanochat/model/ops/softcap_ce.cpp:27-110, and the gradient reduce-scatter of
src/nanochat/train/optim.cpp:425-431, 459-468.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional

import contextlib

import torch
import torch.distributed as dist

from . import engine as nc


@contextlib.contextmanager
def nvtx_range(name: str):
    """A named range on profiler timelines, as the reference's trainer marks its phases
    (src/nanochat/train/trainer.cpp:284-312); a no-op without a profiler attached or a CUDA device."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


@dataclass
class StepConfig:
    """Shapes of config_from_depth (src/nanochat/model/gpt.cpp:25-39): n_embd = 64 * depth."""
    n_layer: int = 24
    n_embd: int = 1536
    vocab: int = 32768
    tokens: int = 16384          # per rank: batch 8 x sequence 2048
    chunk_rows: int = 2048       # lm_head row chunk
    fused_mlp: bool = True       # relu^2 / relu^2-backward quantization inside the fc / proj-dgrad GEMM epilogues
    batched_weights: bool = True  # the step's weight quantization as a few batched launches instead of one per matrix
    # Weight gradients: False = one bf16 write per matrix straight into the reduce-scatter bucket (a step without
    # gradient accumulation); True = the reference's default, fp32 `+=` into the weights' .grad buffers
    # (src/nanochat/model/fp8/fp8.cpp:470-514) followed by the cast of each layer's gradients into the bucket
    # (src/nanochat/train/optim.cpp:459).
    wgrad_fp32_accumulate: bool = False
    # Producers of the quantized GEMM inputs: False = the plain quantizer on ready-made bf16 tensors everywhere (the
    # BASELINE configurations' form: they time Linears, not what feeds them); True = the kernels the reference's
    # training step actually runs there: the fused residual add + lambda blend + RMS norm that emits MX for the QKV
    # and MLP-fc inputs (src/nanochat/model/ops/residual_norm.cpp:33-96) and, in the lm_head, the softcap loss pass
    # and the gradient quantized straight from the logits (ops/softcap_ce.cpp:66-92) instead of synthetic dlogits.
    real_producers: bool = False

    @property
    def linear_shapes(self):
        C = self.n_embd
        return [("qkv", 3 * C, C), ("attn_out", C, C), ("mlp_fc", 4 * C, C), ("mlp_proj", C, 4 * C)]

    @property
    def layer_params(self) -> int:
        return sum(n * k for _, n, k in self.linear_shapes)

    @property
    def lm_head_params(self) -> int:
        return self.vocab * self.n_embd

    def quantized_bytes_per_step(self) -> float:
        """Algorithmic HBM bytes of every quantizer launch of a step: input read once (2 B bf16, 4 B fp32 weights,
        two bf16 inputs for the relu^2 backward) plus (1 + 1/32) B per element and written layout."""
        M, C, V = self.tokens, self.n_embd, self.vocab
        both = 2 * (1 + 1 / 32)
        act = (3 * M * C) * (2 + both)                                             # x_attn, y_att, x_mlp
        grad = (2 * M * C + M * 3 * C) * (2 + both)                                # dy_proj, dy_o, dy_qkv
        if not self.fused_mlp:                                                     # relu^2(h) and dh as own passes
            act += (M * 4 * C) * (2 + both)
            grad += (M * 4 * C) * (4 + both)
        weights = self.layer_params * (4 + both)
        lm = (M * C) * (2 + both) + (M * V) * (2 + both) + self.lm_head_params * (4 + both)
        return self.n_layer * (act + grad + weights) + lm

    def flops_per_step(self) -> float:
        """2MNK over every GEMM: forward, dgrad and wgrad of each Linear."""
        layer = sum(3 * 2.0 * self.tokens * n * k for _, n, k in self.linear_shapes)
        return self.n_layer * layer + 3 * 2.0 * self.tokens * self.vocab * self.n_embd


@dataclass
class BucketSegment:
    """One reduce-scatter: `count` matrices per rank out of world * count consecutive entries of a stack (or, for the
    lm_head, one row slice per rank)."""
    stack: str          # name of the stack, or "lm_head"
    first: int          # first stack entry of the segment (world * entries-per-rank before it)
    count: int          # entries each rank receives
    out_first: int      # where they land in the rank's chunk of the stack
    ready_layer: int    # backward has produced the segment once this layer's weight gradients are written


class GradBucket:
    """The bf16 send buffers of the step's one collective, laid out as the reference's optimizer lays its gradients
    out (src/nanochat/train/optim.cpp:699-714, 222-233, 437-472): the matrices of the transformer blocks are grouped
    by shape, each group stacked as (K_pad, m, n) in forward order with K_pad a multiple of the world size,

        muon_CxC   : per layer c_q, c_k, c_v, c_proj        (4 * n_layer entries; q, k, v adjacent, so the merged
                                                             QKV weight gradient is one (3C, C) GEMM output)
        muon_Cx4C  : per layer the MLP's c_proj             (n_layer entries)
        muon_4CxC  : per layer the MLP's c_fc               (n_layer entries)

    and every stack is reduce-scattered in at most eight segments: a segment is world * c consecutive entries, rank r
    receives entries [r * c, (r + 1) * c) of it, so a rank always ends up with WHOLE matrices (Muon orthogonalises
    per matrix). The lm_head gradient (an AdamW group) is scattered as row slices (optim.cpp:425-431). The weight
    gradient GEMMs write their bf16 output straight into the stacks, so no cast pass precedes the collective (the
    reference casts the stacked fp32 buffer first, optim.cpp:459)."""

    MAX_SEGMENTS = 8  # kMuonSegments, optim.cpp:21

    def __init__(self, cfg: StepConfig, device, world: int = 1):
        self.cfg, self.world = cfg, world
        C, L, V = cfg.n_embd, cfg.n_layer, cfg.vocab
        if V % world:
            raise ValueError("lm_head rows must divide evenly across ranks")
        shapes = [("muon_CxC", 4 * L, C, C), ("muon_Cx4C", L, C, 4 * C), ("muon_4CxC", L, 4 * C, C)]
        self.stack_info = {}
        off = 0
        for name, count, m, n in shapes:
            padded = (count + world - 1) // world * world
            self.stack_info[name] = dict(count=count, padded=padded, m=m, n=n, offset=off)
            off += padded * m * n
        self.lm_offset = off
        off += V * C
        self.numel = off
        self.buffer = torch.zeros(off, dtype=torch.bfloat16, device=device)  # zeros: the padding entries stay zero
        self.stacks = {name: self.buffer[i["offset"]:i["offset"] + i["padded"] * i["m"] * i["n"]].view(i["padded"], i["m"], i["n"])
                       for name, i in self.stack_info.items()}
        # this rank's chunks: (K_pad / world, m, n) per stack, (V / world, C) of the lm_head
        self.chunks = {name: torch.empty((i["padded"] // world, i["m"], i["n"]), dtype=torch.bfloat16, device=device)
                       for name, i in self.stack_info.items()}
        self.lm_chunk = torch.empty((V // world, C), dtype=torch.bfloat16, device=device)
        per_layer = {"muon_CxC": 4, "muon_Cx4C": 1, "muon_4CxC": 1}
        self.segments: List[BucketSegment] = []
        for name, i in self.stack_info.items():
            chunk = i["padded"] // world
            n_seg = min(self.MAX_SEGMENTS, chunk) if world > 1 else 1
            counts = [chunk // n_seg + (1 if s < chunk % n_seg else 0) for s in range(n_seg)]
            o = 0
            for c in counts:
                first = world * o
                self.segments.append(BucketSegment(name, first, c, o, min(first // per_layer[name], L - 1)))
                o += c
        self.segments.append(BucketSegment("lm_head", 0, V // world, 0, L))
        self.shards = [self.output(i).reshape(-1) for i in range(len(self.segments))]

    # ---- where the GEMMs write
    def matrix(self, layer: int, index: int) -> torch.Tensor:
        """The (out, in) gradient of Linear `index` of `layer` (0 merged QKV, 1 attention out, 2 MLP fc, 3 MLP proj) as a
        view of its stack."""
        C = self.cfg.n_embd
        if index == 0:
            return self.stacks["muon_CxC"][4 * layer:4 * layer + 3].view(3 * C, C)
        if index == 1:
            return self.stacks["muon_CxC"][4 * layer + 3]
        if index == 2:
            return self.stacks["muon_4CxC"][layer]
        if index == 3:
            return self.stacks["muon_Cx4C"][layer]
        raise IndexError(index)

    def lm_head(self) -> torch.Tensor:
        return self.buffer[self.lm_offset:].view(self.cfg.vocab, self.cfg.n_embd)

    # ---- the collective
    def input(self, i: int) -> torch.Tensor:
        """Segment i as sent: world * count whole matrices (or all rows of the lm_head)."""
        seg = self.segments[i]
        if seg.stack == "lm_head":
            return self.lm_head()
        return self.stacks[seg.stack][seg.first:seg.first + self.world * seg.count]

    def output(self, i: int) -> torch.Tensor:
        """Where this rank's share of segment i lands: entries [out_first, out_first + count) of its chunk."""
        seg = self.segments[i]
        if seg.stack == "lm_head":
            return self.lm_chunk
        return self.chunks[seg.stack][seg.out_first:seg.out_first + seg.count]

    def owned_entries(self, stack: str, rank: int) -> List[int]:
        """The stack entries rank `rank` holds after the scatter, in chunk order (optim.cpp:263-273)."""
        rows = []
        for seg in self.segments:
            if seg.stack == stack:
                rows += [seg.first + rank * seg.count + t for t in range(seg.count)]
        return rows

    def ready_after_layer(self, layer: int) -> List[int]:
        """Segments that are complete once backward has finished `layer` (it walks the layers downwards; n_layer stands
        for the lm_head, which comes first)."""
        return [i for i, seg in enumerate(self.segments) if seg.ready_layer == layer]

    def reduce_scatter(self, i: int, group=None, async_op: bool = False):
        """Average segment i across ranks into this rank's chunk. world == 1: a copy."""
        if self.world == 1 or not dist.is_initialized():
            self.output(i).copy_(self.input(i)[:self.output(i).size(0)])
            return None
        return dist.reduce_scatter_tensor(self.output(i), self.input(i), op=dist.ReduceOp.AVG, group=group,
                                          async_op=async_op)


def _student_t(shape, nu: float, gen, device) -> torch.Tensor:
    """N(0,1) / sqrt(chi2_nu / nu) from the seeded generator."""
    z = torch.randn(shape, generator=gen, device=device)
    chi2 = torch.zeros(shape, device=device)
    for _ in range(int(nu)):
        chi2 += torch.randn(shape, generator=gen, device=device) ** 2
    return z / torch.sqrt(chi2 / nu)


class DpStep:
    """Buffers and launch sequence of one rank's step. `gemm_hook(begin: bool)` and `quant_hook(begin: bool)`
    (optional) are called right before and right after every GEMM / quantizer launch so a benchmark can bracket
    them with events."""

    def __init__(self, cfg: StepConfig, device, rank: int = 0, world: int = 1, input_sets: int = 2,
                 gemm_hook: Optional[Callable[[bool], None]] = None,
                 quant_hook: Optional[Callable[[bool], None]] = None):
        self.cfg, self.device, self.rank, self.world = cfg, device, rank, world
        self.hook = gemm_hook
        self.qhook = quant_hook
        M, C, V = cfg.tokens, cfg.n_embd, cfg.vocab
        gen = torch.Generator(device=device).manual_seed(1000 + rank)
        bf = torch.bfloat16

        def randn(shape, std=1.0):
            return (torch.randn(shape, generator=gen, device=device) * std).to(bf)

        # fp32 master weights, one set per layer, ~N(0, 1/sqrt(K)); identical on every rank (seed without rank)
        wgen = torch.Generator(device=device).manual_seed(7)
        self.weights = [[torch.randn((n, k), generator=wgen, device=device) / k ** 0.5 for _, n, k in cfg.linear_shapes]
                        for _ in range(cfg.n_layer)]
        self.w_lm = torch.randn((V, C), generator=wgen, device=device) / C ** 0.5
        self.wq: List[List[nc.Fp8Tensor]] = [[nc.empty_mx(n, k, device) for _, n, k in cfg.linear_shapes]
                                             for _ in range(cfg.n_layer)]
        self.wq_lm = nc.empty_mx(V, C, device)

        # synthetic activations / incoming gradients, a few sets used in rotation
        self.x_attn = [randn((M, C)) for _ in range(input_sets)]
        self.y_att = [randn((M, C)) for _ in range(input_sets)]
        self.x_mlp = [randn((M, C)) for _ in range(input_sets)]
        self.resid = [randn((M, C)) for _ in range(input_sets)]
        self.dy_proj = [randn((M, C), 1e-3) for _ in range(input_sets)]
        self.dy_o = [randn((M, C), 1e-3) for _ in range(input_sets)]
        self.dy_qkv = [randn((M, 3 * C), 1e-3) for _ in range(input_sets)]
        self.x_lm = (0.5 * _student_t((M, C), 3.0, gen, device)).to(bf)
        self.dlogits = [randn((cfg.chunk_rows, V), 1e-3) for _ in range(input_sets)]

        # saved for backward, per layer: the transposed (column-wise) quantizations and the MLP hidden
        L = cfg.n_layer
        self.xq_attn = [nc.empty_mx(M, C, device) for _ in range(L)]
        self.yq_att = [nc.empty_mx(M, C, device) for _ in range(L)]
        self.xq_mlp = [nc.empty_mx(M, C, device) for _ in range(L)]
        self.aq = [nc.empty_mx(M, 4 * C, device) for _ in range(L)]
        self.h = [torch.empty((M, 4 * C), dtype=bf, device=device) for _ in range(L)]
        # outputs and scratch shared by all layers
        self.qkv = torch.empty((M, 3 * C), dtype=bf, device=device)
        self.out_c = torch.empty((M, C), dtype=bf, device=device)
        self.gq_c = nc.empty_mx(M, C, device)
        self.gq_3c = nc.empty_mx(M, 3 * C, device)
        self.gq_4c = nc.empty_mx(M, 4 * C, device)
        self.da = torch.empty((M, 4 * C), dtype=bf, device=device)
        self.dx = torch.empty((M, C), dtype=bf, device=device)
        # lm_head
        self.xq_lm = nc.empty_mx(M, C, device)
        self.logits = torch.empty((cfg.chunk_rows, V), dtype=bf, device=device)
        self.gq_lm = nc.empty_mx(M, V, device)
        self.dx_lm = torch.empty((M, C), dtype=bf, device=device)

        self.bucket = GradBucket(cfg, device, world)
        # fp32 .grad buffers, only for the accumulate form
        self.grads = self.grad_lm = None
        self.set_wgrad_fp32_accumulate(cfg.wgrad_fp32_accumulate)
        # inputs of the real producers (StepConfig.real_producers), allocated on first use
        self._producer_state = None
        # "b200": this library; "cublaslt": the same GEMMs through torch._scaled_mm, the arithmetic of the
        # reference's --gemm=cublas (src/nanochat/model/fp8/mx_gemm.cpp:158); gemm_only: replay the GEMMs over the
        # operands quantized by an earlier step, no quantizer launches
        self.gemm_impl = "b200"
        self.gemm_only = False
        self.comm_stream = torch.cuda.Stream(device=device) if (device.type == "cuda" and world > 1) else None
        self._pending: list = []
        self._graphs = None            # CUDA graphs of the step, one per phase of the input rotation (capture())
        self.launches_per_step = None  # library kernels in one captured step

    def set_wgrad_fp32_accumulate(self, on: bool):
        """Switches the weight-gradient form (StepConfig.wgrad_fp32_accumulate); the fp32 .grad buffers (4 bytes per
        parameter) are allocated on first use."""
        self._graphs = None  # a captured step has the other form baked in
        self.cfg.wgrad_fp32_accumulate = on
        if on and self.grads is None:
            cfg, device = self.cfg, self.device
            self.grads = [[torch.zeros((n, k), dtype=torch.float32, device=device) for _, n, k in cfg.linear_shapes]
                          for _ in range(cfg.n_layer)]
            self.grad_lm = torch.zeros((cfg.vocab, cfg.n_embd), dtype=torch.float32, device=device)

    def _producers(self):
        """Buffers of the real-producer form: a residual stream x0 and lambdas for the blend, outputs of the two fused
        residual steps per layer, targets and per-row loss buffers of the lm_head."""
        if self._producer_state is None:
            cfg, dev = self.cfg, self.device
            M, C = cfg.tokens, cfg.n_embd
            g = torch.Generator(device=dev).manual_seed(77 + self.rank)
            bf = torch.bfloat16
            st = {}
            st["x0"] = torch.randn((M, C), generator=g, device=dev).to(bf)
            st["lr"] = torch.rand(cfg.n_layer, generator=g, device=dev) + 0.5
            st["l0"] = torch.rand(cfg.n_layer, generator=g, device=dev) * 0.3
            st["targets"] = torch.randint(0, cfg.vocab, (M,), generator=g, device=dev)
            st["loss"] = torch.empty(M, dtype=torch.float32, device=dev)
            st["lse"] = torch.empty(cfg.chunk_rows, dtype=torch.float32, device=dev)
            st["scale"] = torch.full((1,), 1.0 / M, device=dev)
            # (res, n, n_mx, rstd, s) per fused residual step; n_mx is replaced by the layer's saved MX buffers
            st["attn_out"] = [None] * cfg.n_layer
            st["mlp_out"] = [None] * cfg.n_layer
            self._producer_state = st
        return self._producer_state

    def _residual_norm(self, key: str, l: int, x, r, x0, q: nc.Fp8Tensor):
        """One fused residual step whose MX output lands in the saved-for-backward buffers q."""
        st = self._producers()
        if self.gemm_only:
            return
        if self.qhook:
            self.qhook(True)
        prev = st[key][l]
        if prev is None:
            res, n, n_mx, rstd, s_ = nc.residual_norm_mx(x, r, x0, st["lr"], st["l0"], l)
            prev = (res, n, q, rstd, s_)  # from now on the kernel writes MX straight into q
            del n_mx
        st[key][l] = nc.residual_norm_mx(x, r, x0, st["lr"], st["l0"], l, out=prev)
        if self.qhook:
            self.qhook(False)

    def _grad(self, layer: int, index: int):
        return self.grads[layer][index] if self.cfg.wgrad_fp32_accumulate else None

    def _cast_grads(self, layer: int):
        """The accumulate form's last step before the collective: fp32 .grad -> the bf16 bucket."""
        if not self.cfg.wgrad_fp32_accumulate or self.gemm_impl == "cublaslt":
            return
        if layer == self.cfg.n_layer:
            self.bucket.lm_head().copy_(self.grad_lm)
            return
        for j in range(4):
            self.bucket.matrix(layer, j).copy_(self.grads[layer][j])

    # ------------------------------------------------------------------ pieces
    def _gemm(self, out, a, a_scale, b, b_scale, resid=None):
        if self.hook:
            self.hook(True)
        if self.gemm_impl == "cublaslt":
            # the library call the reference's cuBLAS backend makes; its residual add is a separate kernel of the
            # residual step and is left out here (in cuBLASLt's favour)
            torch._scaled_mm(a, b.t(), a_scale, b_scale, None, None, out.dtype, False, out=out)
        else:
            nc.mx_gemm_out(out, a, a_scale, b, b_scale, resid)
        if self.hook:
            self.hook(False)

    def _wgrad(self, bucket_view, grad, a, a_scale, b, b_scale):
        """One weight gradient: bf16 straight into the bucket, or fp32 += into .grad (cast to the bucket later)."""
        if grad is None or self.gemm_impl == "cublaslt":
            self._gemm(bucket_view, a, a_scale, b, b_scale)
            return
        if self.hook:
            self.hook(True)
        nc.mx_gemm_f32(a, a_scale, b, b_scale, grad, True)
        if self.hook:
            self.hook(False)

    def _quant(self, x, q: nc.Fp8Tensor, relu_square=False):
        out, out_t = nc.mx_outs(q)
        self._quant_into(x, relu_square, out, out_t)

    def _quant_into(self, x, relu_square, out, out_t):
        if self.gemm_only:
            return
        if self.qhook:
            self.qhook(True)
        nc.quantize_mx_into(x, relu_square, out, out_t)
        if self.qhook:
            self.qhook(False)

    def quantize_weights(self):
        """Once per optimizer step (the reference's weight cache, fp8.cpp:516-536): fp32 masters -> both layouts."""
        if self.gemm_only:
            return
        if not self.cfg.batched_weights:
            for ws, qs in zip(self.weights, self.wq):
                for w, q in zip(ws, qs):
                    self._quant(w, q)
            self._quant(self.w_lm, self.wq_lm)
            return
        # all of them in a few launches: a launch per weight matrix (one or two waves of tiles) is bound by its own
        # ramp-up and tail
        jobs = [(w, *nc.mx_outs(q)) for ws, qs in zip(self.weights, self.wq) for w, q in zip(ws, qs)]
        jobs.append((self.w_lm, *nc.mx_outs(self.wq_lm)))
        if self.qhook:
            self.qhook(True)
        nc.quantize_mx_batch_into(jobs)
        if self.qhook:
            self.qhook(False)

    def layer_forward(self, l: int, s: int):
        wq = self.wq[l]
        if self.cfg.real_producers:  # s = x + r, res = lr s + l0 x0, n = rms_norm(res) -> MX (the QKV input)
            self._residual_norm("attn_out", l, self.x_attn[s], self.resid[s], self._producers()["x0"], self.xq_attn[l])
        else:
            self._quant(self.x_attn[s], self.xq_attn[l])
        self._gemm(self.qkv, self.xq_attn[l].data, self.xq_attn[l].inv_scale, wq[0].data, wq[0].inv_scale)
        self._quant(self.y_att[s], self.yq_att[l])
        self._gemm(self.out_c, self.yq_att[l].data, self.yq_att[l].inv_scale, wq[1].data, wq[1].inv_scale, self.resid[s])
        if self.cfg.real_producers:  # res = x + r, n = rms_norm(res) -> MX (the MLP fc input)
            self._residual_norm("mlp_out", l, self.x_mlp[s], self.resid[s], None, self.xq_mlp[l])
        else:
            self._quant(self.x_mlp[s], self.xq_mlp[l])
        if self.cfg.fused_mlp and not self.gemm_only:
            # fc GEMM writes h and, from the same epilogue, MX(relu(h)^2) in both layouts (fp8.cpp:279-284)
            if self.hook:
                self.hook(True)
            nc.mx_gemm_relu_square(self.h[l], self.aq[l].data, self.aq[l].inv_scale, self.aq[l].data_t,
                                   self.aq[l].inv_scale_t, self.xq_mlp[l].data, self.xq_mlp[l].inv_scale, wq[2].data,
                                   wq[2].inv_scale)
            if self.hook:
                self.hook(False)
        else:
            self._gemm(self.h[l], self.xq_mlp[l].data, self.xq_mlp[l].inv_scale, wq[2].data, wq[2].inv_scale)
            self._quant(self.h[l], self.aq[l], relu_square=True)
        self._gemm(self.out_c, self.aq[l].data, self.aq[l].inv_scale, wq[3].data, wq[3].inv_scale, self.resid[s])

    def layer_backward(self, l: int, s: int):
        wq, b = self.wq[l], self.bucket
        # MLP proj: dA = dY . W, dW = dY^T . A
        self._quant(self.dy_proj[s], self.gq_c)
        # the reference's order (fp8.cpp:299-337): proj weight gradient, then the dgrad whose epilogue quantizes dh,
        # then fc's dgrad and weight gradient, which read that dh while it is still in L2
        self._wgrad(b.matrix(l, 3), self._grad(l, 3), self.gq_c.data_t, self.gq_c.inv_scale_t, self.aq[l].data_t, self.aq[l].inv_scale_t)
        if self.cfg.fused_mlp and not self.gemm_only:
            # dgrad GEMM whose epilogue reads h and emits MX(dh) directly; dA is never written (fp8.cpp:318-323)
            if self.hook:
                self.hook(True)
            nc.mx_gemm_relu_square_bwd(self.gq_c.data, self.gq_c.inv_scale, wq[3].data_t, wq[3].inv_scale_t, self.h[l],
                                       self.gq_4c.data, self.gq_4c.inv_scale, self.gq_4c.data_t, self.gq_4c.inv_scale_t)
            if self.hook:
                self.hook(False)
        else:
            self._gemm(self.da, self.gq_c.data, self.gq_c.inv_scale, wq[3].data_t, wq[3].inv_scale_t)
            # relu^2 backward as a prologue of the quantizer: dh = bf16(h > 0 ? dA * 2h : 0)
            out, out_t = nc.mx_outs(self.gq_4c)
            if self.qhook and not self.gemm_only:
                self.qhook(True)
            if not self.gemm_only:
                nc.check(nc.lib.mxb200_quantize_mx_relu_square_bwd(
                    self.da.data_ptr(), self.h[l].data_ptr(), self.da.size(0), self.da.size(1), out, out_t,
                    nc.SCALE_REFERENCE, torch.cuda.current_stream().cuda_stream), "quantize dh")
            if self.qhook and not self.gemm_only:
                self.qhook(False)
        self._gemm(self.dx, self.gq_4c.data, self.gq_4c.inv_scale, wq[2].data_t, wq[2].inv_scale_t)
        self._wgrad(b.matrix(l, 2), self._grad(l, 2), self.gq_4c.data_t, self.gq_4c.inv_scale_t, self.xq_mlp[l].data_t, self.xq_mlp[l].inv_scale_t)
        # attention out
        self._quant(self.dy_o[s], self.gq_c)
        self._gemm(self.dx, self.gq_c.data, self.gq_c.inv_scale, wq[1].data_t, wq[1].inv_scale_t)
        self._wgrad(b.matrix(l, 1), self._grad(l, 1), self.gq_c.data_t, self.gq_c.inv_scale_t, self.yq_att[l].data_t, self.yq_att[l].inv_scale_t)
        # merged QKV
        self._quant(self.dy_qkv[s], self.gq_3c)
        self._gemm(self.dx, self.gq_3c.data, self.gq_3c.inv_scale, wq[0].data_t, wq[0].inv_scale_t)
        self._wgrad(b.matrix(l, 0), self._grad(l, 0), self.gq_3c.data_t, self.gq_3c.inv_scale_t, self.xq_attn[l].data_t, self.xq_attn[l].inv_scale_t)

    def lm_head(self):
        """Chunked logits GEMM, gradient quantized per chunk into row/column ranges of one MX buffer, dX per chunk,
        one wgrad GEMM over all tokens (softcap_ce.cpp:46-109)."""
        cfg = self.cfg
        self._quant(self.x_lm, self.xq_lm)
        K = cfg.n_embd
        for c, begin in enumerate(range(0, cfg.tokens, cfg.chunk_rows)):
            rows = cfg.chunk_rows
            xa = self.xq_lm.data[begin:begin + rows]
            xs = self.xq_lm.inv_scale[begin * K // 32:(begin + rows) * K // 32]
            self._gemm(self.logits, xa, xs, self.wq_lm.data, self.wq_lm.inv_scale)
            out_rows = nc.mx_out(self.gq_lm.data, self.gq_lm.inv_scale, begin, 0)
            out_cols = nc.mx_out(self.gq_lm.data_t, self.gq_lm.inv_scale_t, 0, begin)
            if self.cfg.real_producers and not self.gemm_only:
                st = self._producers()
                if self.qhook:
                    self.qhook(True)
                t = st["targets"][begin:begin + rows]
                nc.softcap_ce_loss(self.logits, t, cfg.vocab, 15.0, loss=st["loss"][begin:begin + rows], lse=st["lse"])
                nc.softcap_ce_grad_mx(self.logits, t, st["lse"], cfg.vocab, 15.0, out_rows, out_cols, grad_scale=st["scale"])
                if self.qhook:
                    self.qhook(False)
            else:
                g = self.dlogits[c % len(self.dlogits)]
                self._quant_into(g, False, out_rows, out_cols)
            ga = self.gq_lm.data[begin:begin + rows]
            gs = self.gq_lm.inv_scale[begin * cfg.vocab // 32:(begin + rows) * cfg.vocab // 32]
            self._gemm(self.dx_lm[begin:begin + rows], ga, gs, self.wq_lm.data_t, self.wq_lm.inv_scale_t)
        self._wgrad(self.bucket.lm_head(), self.grad_lm if self.cfg.wgrad_fp32_accumulate else None, self.gq_lm.data_t,
                    self.gq_lm.inv_scale_t, self.xq_lm.data_t, self.xq_lm.inv_scale_t)

    def _reduce_segment(self, i: int):
        """Reduce-scatter segment i on the communication stream once the compute stream has produced it."""
        if self.world == 1 or self.gemm_only:
            return
        ev = torch.cuda.Event()
        ev.record()
        self.comm_stream.wait_event(ev)
        seg = self.bucket.segments[i]
        with nvtx_range(f"reduce_scatter {seg.stack}[{seg.first}:+{self.world * seg.count}]"), \
                torch.cuda.stream(self.comm_stream):
            self._pending.append(self.bucket.reduce_scatter(i, async_op=True))

    def run_gemms_only(self, impl: str = "b200"):
        """The step's 305 GEMMs again, back to back, over the operands an earlier run_step quantized: no quantizer
        launches, plain epilogues (the two MLP GEMMs without their fused quantization), no collective. impl
        "cublaslt" sends the same operands through torch._scaled_mm."""
        self.gemm_only, self.gemm_impl = True, impl
        try:
            self.run_step(0)
        finally:
            self.gemm_only, self.gemm_impl = False, "b200"

    def finish_collectives(self):
        for w in self._pending:
            if w is not None:
                w.wait()
        self._pending.clear()
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)

    # ------------------------------------------------------------------ the step
    def capture(self) -> None:
        """Records the step as CUDA graphs, one per phase of the input rotation (step k reads input set (k + layer) %
        n_sets), after which run_step replays them: the step's 555 launches, and with more than one rank its
        collectives with their side stream and events, are then issued by the device's front end without the host
        between them, which takes the gaps between launches (1 to 1.5 ms of a 41 ms step) out. Call it after an eager
        step (first launches configure kernels and allocate the split-K workspace) and again after changing the
        step's form; `release()` or a form change drops the graphs."""
        n_sets = len(self.x_attn)
        self._graphs = None
        stream = torch.cuda.Stream(device=self.device)
        graphs, pool = [], None
        for phase in range(n_sets):
            g = torch.cuda.CUDAGraph()
            before = nc.capi.launch_count()
            # thread_local: NCCL's watchdog thread and the clock sampler make CUDA calls of their own meanwhile
            with torch.cuda.graph(g, pool=pool, stream=stream, capture_error_mode="thread_local"):
                self._run_step_eager(phase)
            self.launches_per_step = nc.capi.launch_count() - before
            pool = g.pool()
            graphs.append(g)
        self._graphs = graphs

    def release(self) -> None:
        self._graphs = None

    def run_step(self, step: int = 0, eager: bool = False):
        """One step. Replays the captured graph of this step's phase when `capture()` has been called, unless `eager`
        (per-launch hooks only see eager launches) or the GEMM-only comparator form is on."""
        if self._graphs is not None and not eager and not self.gemm_only:
            with nvtx_range("step (graph replay)"):
                self._graphs[step % len(self._graphs)].replay()
            return
        self._run_step_eager(step)

    def _run_step_eager(self, step: int = 0):
        cfg = self.cfg
        n_sets = len(self.x_attn)
        with nvtx_range("quantize_weights"):
            self.quantize_weights()
        for l in range(cfg.n_layer):
            with nvtx_range(f"layer{l}.forward"):
                self.layer_forward(l, (step + l) % n_sets)
        with nvtx_range("lm_head"):
            self.lm_head()
            self._cast_grads(cfg.n_layer)
        for i in self.bucket.ready_after_layer(cfg.n_layer):
            self._reduce_segment(i)
        for l in reversed(range(cfg.n_layer)):
            with nvtx_range(f"layer{l}.backward"):
                self.layer_backward(l, (step + l) % n_sets)
                self._cast_grads(l)
            for i in self.bucket.ready_after_layer(l):
                self._reduce_segment(i)
        with nvtx_range("finish_collectives"):
            self.finish_collectives()
