"""Host-side mirror of nanochat-cpp's MXFP8 Linear interface over libmxb200.so.

Same names, argument meaning and error behaviour as the reference's fp8.h / mx_gemm.h (file:line cited per
function, paths within nanochat-cpp), with torch tensors used only as owners of device memory. Every call
goes to the CUDA library through the C ABI; nothing here computes on the CPU and nothing falls back.
"""
from __future__ import annotations

import ctypes
import enum
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch

from . import capi
from .capi import MxOut, check, lib

__all__ = [
    "Fp8Tensor", "Fp8WeightCache", "MxGemmBackend", "set_mx_gemm_backend", "mx_gemm_backend", "mx_fits",
    "empty_mx", "empty_mx_scale", "mx_out", "mx_outs", "quantize_mx", "quantize_mx_into", "quantize_mx_batch_into",
    "quantize_mx_relu_square_bwd", "residual_norm_mx", "residual_norm_mx_fits", "quantize_fp8_weight", "mx_qkv_weights", "mx_gemm", "mx_gemm_out",
    "mx_gemm_f32", "mx_gemm_relu_square", "mx_gemm_relu_square_bwd", "mx_grad_direct", "mx_grad_weights", "fp8_matmul", "fp8_qkv", "fp8_relu_square_mlp", "relu_square_mlp_mx", "fp8_eligible",
    "softcap_ce_loss", "softcap_ce_grad_mx", "softcap_cross_entropy",
    "SCALE_REFERENCE", "SCALE_OCP_FLOOR",
]

SCALE_REFERENCE = capi.SCALE_REFERENCE
SCALE_OCP_FLOOR = capi.SCALE_OCP_FLOOR
E4M3 = torch.float8_e4m3fn
E8M0 = torch.float8_e8m0fnu


class MxGemmBackend(enum.Enum):
    """src/nanochat/model/fp8/mx_gemm.h:9 has {Cublas, Cutlass}; this library is the third value a
    ``--gemm=b200`` flag would select. It is the only one implemented here."""
    B200 = "b200"


_backend = MxGemmBackend.B200


def set_mx_gemm_backend(backend: MxGemmBackend) -> None:
    """src/nanochat/model/fp8/mx_gemm.cpp:134-136. Anything but B200 raises: there is no other backend."""
    global _backend
    if backend is not MxGemmBackend.B200:
        raise ValueError("only MxGemmBackend.B200 exists in this library")
    _backend = backend


def mx_gemm_backend() -> MxGemmBackend:
    return _backend


@dataclass
class Fp8Tensor:
    """A quantized 2-D tensor: data (R, C) scaled along its rows, data_t (C, R) scaled along its own rows,
    swizzled E8M0 scales for each (src/nanochat/model/fp8/fp8.h:68-77)."""
    data: Optional[torch.Tensor] = None
    data_t: Optional[torch.Tensor] = None
    inv_scale: Optional[torch.Tensor] = None
    inv_scale_t: Optional[torch.Tensor] = None


def mx_fits(rows: int, cols: int) -> bool:
    """src/nanochat/model/fp8/fp8.h:86-88."""
    return rows % 128 == 0 and cols % 128 == 0


def fp8_eligible(in_features: int, out_features: int) -> bool:
    """src/nanochat/model/fp8/fp8.h:127-130."""
    return in_features % 16 == 0 and out_features % 16 == 0 and min(in_features, out_features) >= 128


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what}: expected a CUDA tensor; this engine has no CPU path")


def empty_mx_scale(rows: int, cols: int, device) -> torch.Tensor:
    """src/nanochat/model/fp8/fp8.cpp:113-115."""
    return torch.empty(rows * cols // 32, dtype=E8M0, device=device)


def empty_mx(R: int, C: int, device, rows: bool = True, cols: bool = True) -> Fp8Tensor:
    """src/nanochat/model/fp8/fp8.cpp:122-133."""
    q = Fp8Tensor()
    if rows:
        q.data = torch.empty((R, C), dtype=E4M3, device=device)
        q.inv_scale = empty_mx_scale(R, C, device)
    if cols:
        q.data_t = torch.empty((C, R), dtype=E4M3, device=device)
        q.inv_scale_t = empty_mx_scale(C, R, device)
    return q


def mx_out(data: torch.Tensor, scale: torch.Tensor, row: int = 0, col: int = 0) -> MxOut:
    """The kernels' view of MX data (R, ld) from (row, col) on; row, col % 128 == 0
    (src/nanochat/model/fp8/fp8.cpp:117-120)."""
    if row % 128 or col % 128:
        raise RuntimeError("mx_out: row and col must be multiples of 128")
    ld = data.size(1)
    tiles = ld // 128
    return MxOut(data.data_ptr() + row * ld + col, ld, scale.data_ptr() + ((row // 128) * tiles + col // 128) * 512, tiles)


def mx_outs(q: Fp8Tensor):
    """src/nanochat/model/fp8/fp8.cpp:135-142."""
    out = mx_out(q.data, q.inv_scale) if q.data is not None else MxOut(None, 0, None, 0)
    out_t = mx_out(q.data_t, q.inv_scale_t) if q.data_t is not None else MxOut(None, 0, None, 0)
    return out, out_t


def quantize_mx_into(x: torch.Tensor, relu_square: bool, out: MxOut, out_t: MxOut,
                     scale_rule: int = SCALE_REFERENCE) -> None:
    """quantize_mx of x into given buffers (src/nanochat/model/fp8/fp8.cpp:144-153)."""
    _require_cuda(x, "quantize_mx")
    if not (x.dim() == 2 and x.is_contiguous() and mx_fits(x.size(0), x.size(1))
            and x.dtype in (torch.bfloat16, torch.float32) and (not relu_square or x.dtype == torch.bfloat16)):
        raise RuntimeError("MX: expected an aligned, contiguous 2D tensor with dims % 128")
    check(lib.mxb200_quantize_mx(x.data_ptr(), int(x.dtype == torch.bfloat16), x.size(0), x.size(1), out, out_t,
                                 capi.PROLOGUE_RELU_SQUARE if relu_square else capi.PROLOGUE_NONE, scale_rule,
                                 _stream()), "quantize_mx")


def quantize_mx_batch_into(jobs: Sequence[tuple], scale_rule: int = SCALE_REFERENCE) -> None:
    """quantize_mx_into(x, False, out, out_t) for every (x, out, out_t) of jobs, all bf16 or all fp32, in as few
    launches as possible: the same bytes as one call each. For runs of small tensors, e.g. the parts of the merged
    q/k/v weight (src/nanochat/model/fp8/fp8.cpp:155-171) or a model's weights after an optimizer step."""
    if not jobs:
        return
    x0 = jobs[0][0]
    _require_cuda(x0, "quantize_mx_batch")
    arr = (capi.QuantizeJob * len(jobs))()
    for i, (x, out, out_t) in enumerate(jobs):
        if not (x.is_cuda and x.dim() == 2 and x.is_contiguous() and mx_fits(x.size(0), x.size(1))
                and x.dtype == x0.dtype and x.dtype in (torch.bfloat16, torch.float32) and x.device == x0.device):
            raise RuntimeError("MX: expected aligned, contiguous 2D tensors of one dtype with dims % 128")
        arr[i] = capi.QuantizeJob(x.data_ptr(), x.size(0), x.size(1), out, out_t)
    check(lib.mxb200_quantize_mx_batch(arr, len(jobs), int(x0.dtype == torch.bfloat16), scale_rule, _stream()),
          "quantize_mx_batch")


def quantize_mx(x: torch.Tensor, rows: bool = True, cols: bool = True, relu_square: bool = False,
                scale_rule: int = SCALE_REFERENCE) -> Fp8Tensor:
    """MXFP8 E4M3 of a contiguous 2-D bf16 or fp32 x (src/nanochat/model/fp8/fp8.h:82-84,
    fp8.cpp:538-549)."""
    _require_cuda(x, "quantize_mx")
    q = empty_mx(x.size(0), x.size(1), x.device, rows, cols)
    out, out_t = mx_outs(q)
    quantize_mx_into(x, relu_square, out, out_t, scale_rule)
    return q


def quantize_mx_relu_square_bwd(g: torch.Tensor, h: torch.Tensor, rows: bool = True, cols: bool = True,
                                scale_rule: int = SCALE_REFERENCE) -> Fp8Tensor:
    """MX of dh = bf16(h > 0 ? g * 2h : 0) without writing dh
    (src/nanochat/model/fp8/fp8_kernel.h:41-43; caller fp8.cpp:318-323)."""
    _require_cuda(g, "quantize_mx_relu_square_bwd")
    if not (g.shape == h.shape and g.dtype == h.dtype == torch.bfloat16 and g.is_contiguous() and h.is_contiguous()
            and mx_fits(g.size(0), g.size(1))):
        raise RuntimeError("MX: expected two contiguous bf16 2D tensors of one shape with dims % 128")
    q = empty_mx(g.size(0), g.size(1), g.device, rows, cols)
    out, out_t = mx_outs(q)
    check(lib.mxb200_quantize_mx_relu_square_bwd(g.data_ptr(), h.data_ptr(), g.size(0), g.size(1), out, out_t,
                                                 scale_rule, _stream()), "quantize_mx_relu_square_bwd")
    return q


def residual_norm_mx_fits(rows: int, cols: int) -> bool:
    """Whether residual_norm_mx handles (rows, cols): both % 128 and cols within the kernel's row-in-registers limit
    (the reference's is 1536, src/nanochat/model/ops/residual_norm_kernel.h:15; this kernel's is 2048)."""
    return mx_fits(rows, cols) and cols <= 2048


def residual_norm_mx(x: torch.Tensor, r: Optional[torch.Tensor] = None, x0: Optional[torch.Tensor] = None,
                     lr: Optional[torch.Tensor] = None, l0: Optional[torch.Tensor] = None, layer: int = 0,
                     gate_cols: int = 0, eps: float = torch.finfo(torch.float32).eps, out: Optional[tuple] = None):
    """Forward of the reference's fused residual step with MX output (src/nanochat/model/ops/residual_norm.cpp:36-96,
    the `mx` branch): s = x + r, res = lr[layer] * s + l0[layer] * x0 (with the op path's bf16 roundings),
    n = rms_norm(res). Returns (res, n, n_mx, rstd, s): n holds only its first gate_cols columns; n_mx is
    quantize_mx(n) in both layouts, bit for bit; s is None unless both r and x0 are given. out: a tuple this function
    returned earlier for the same shapes and inputs present, whose buffers are written again instead of new ones."""
    _require_cuda(x, "residual_norm_mx")
    cols = x.size(-1)
    rows = x.numel() // cols
    if not (x.dtype == torch.bfloat16 and x.is_contiguous() and residual_norm_mx_fits(rows, cols)
            and 0 <= gate_cols <= cols):
        raise RuntimeError("residual_norm_mx: shape")
    for t in (r, x0):
        if t is not None and not (t.dtype == torch.bfloat16 and t.is_contiguous() and t.shape == x.shape):
            raise RuntimeError("residual_norm_mx: expected contiguous bf16 of x's shape")
    blend = x0 is not None
    if blend and not (lr is not None and l0 is not None and lr.dtype == l0.dtype == torch.float32
                      and 0 <= layer < lr.numel() == l0.numel() and lr.is_contiguous() and l0.is_contiguous()):
        raise RuntimeError("residual_norm_mx: the blend needs fp32 lambdas")
    if out is not None:
        res, n, n_mx, rstd, s = out
        if not (res.shape == x.shape and n.shape == x.shape and rstd.numel() == rows and n_mx.data.shape == (rows, cols)
                and (s is not None) == (r is not None and blend)):
            raise RuntimeError("residual_norm_mx: out does not match")
    else:
        res = torch.empty_like(x)
        n = torch.empty_like(x)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        s = torch.empty_like(x) if (r is not None and blend) else None
        n_mx = empty_mx(rows, cols, x.device)
    out, out_t = mx_outs(n_mx)
    args = capi.ResidualNormMx(x.data_ptr(), r.data_ptr() if r is not None else None,
                               x0.data_ptr() if blend else None,
                               lr.data_ptr() + 4 * layer if blend else None, l0.data_ptr() + 4 * layer if blend else None,
                               s.data_ptr() if s is not None else None, res.data_ptr(), n.data_ptr(), rstd.data_ptr(),
                               rows, cols, eps, out, out_t, gate_cols)
    check(lib.mxb200_residual_norm_mx_fwd(ctypes.byref(args), _stream()), "residual_norm_mx")
    return res, n, n_mx, rstd, s


class Fp8WeightCache:
    """FP8 copies of weights, remade only when a weight changes: in-place updates bump the tensor's version
    (src/nanochat/model/fp8/fp8.h:18-38, fp8.cpp:516-536)."""

    def __init__(self, enabled: bool = False):
        self.enabled = enabled
        self._kind = -1
        self._keys: list = []
        self._value: list = []

    def get(self, kind: int, weights: Sequence[torch.Tensor], make: Callable[[], List[torch.Tensor]]):
        if not self.enabled:
            return make()
        keys = [(id(w), w.data_ptr(), w._version) for w in weights]
        if kind != self._kind or keys != self._keys:
            self._value = make()
            self._kind, self._keys = kind, keys
        return self._value


def quantize_fp8_weight(w: torch.Tensor, cache: Optional[Fp8WeightCache] = None) -> Fp8Tensor:
    """A weight's E4M3 copy under MX, from cache while w is unchanged
    (src/nanochat/model/fp8/fp8.cpp:551-558)."""
    def make():
        q = quantize_mx(w.detach().contiguous())
        return [q.data, q.data_t, q.inv_scale, q.inv_scale_t]
    v = cache.get(1, [w], make) if cache is not None else make()
    return Fp8Tensor(v[0], v[1], v[2], v[3])


def mx_qkv_weights(wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, cache: Optional[Fp8WeightCache] = None):
    """Merged q/k/v weights: {w_cat (n, C), w_cat^T (C, n), their scales}; each part quantized into its row
    range of one buffer (src/nanochat/model/fp8/fp8.cpp:155-171)."""
    C = wq.size(1)
    n = wq.size(0) + wk.size(0) + wv.size(0)

    def make():
        out = [torch.empty((n, C), dtype=E4M3, device=wq.device), torch.empty((C, n), dtype=E4M3, device=wq.device),
               empty_mx_scale(n, C, wq.device), empty_mx_scale(C, n, wq.device)]
        row, jobs = 0, []
        for w in (wq, wk, wv):
            if w.size(1) != C:
                raise RuntimeError("q/k/v weights must share the input dim")
            jobs.append((w.detach().contiguous(), mx_out(out[0], out[2], row, 0), mx_out(out[1], out[3], 0, row)))
            row += w.size(0)
        if len({j[0].dtype for j in jobs}) == 1:
            quantize_mx_batch_into(jobs)  # the three parts in one launch
        else:
            for x, o, o_t in jobs:
                quantize_mx_into(x, False, o, o_t)
        return out
    return cache.get(1, [wq, wk, wv], make) if cache is not None else make()


# ------------------------------------------------------------------------------------------------ GEMMs

_workspaces: dict = {}


def _workspace(device, nbytes: int) -> torch.Tensor:
    """Split-K scratch, grown on demand and kept per (device, stream): split-K GEMMs on different streams may
    overlap on the GPU and must not share partial tiles and counters, while launches on one stream are ordered
    and reuse theirs (the reference's cuBLASLt path likewise borrows torch's per-stream workspace,
    src/nanochat/model/fp8/mx_gemm.cpp:236-237). A replaced tensor is handed back to the caching allocator, which
    keeps it for the stream it was allocated on until that stream's queued work has run."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (index, torch.cuda.current_stream(index).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _check_operands(a, a_scale, b, b_scale, what):
    for t in (a, a_scale, b, b_scale):
        _require_cuda(t, what)
    if not (a.dim() == 2 and b.dim() == 2 and a.is_contiguous() and b.is_contiguous() and a.dtype == E4M3
            and b.dtype == E4M3 and a.size(1) == b.size(1)):
        raise RuntimeError(f"{what}: shape mismatch")
    M, N, K = a.size(0), b.size(0), a.size(1)
    if a_scale.numel() != M * K // 32 or b_scale.numel() != N * K // 32:
        raise RuntimeError(f"{what}: expected e4m3 operands with their MX scales")
    return M, N, K


def mx_gemm_out(out: torch.Tensor, a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor, b_scale: torch.Tensor,
                resid: Optional[torch.Tensor] = None, splits: Optional[int] = None) -> None:
    """mx_gemm into out, bf16 or fp32 (src/nanochat/model/fp8/mx_gemm.h:26-27, mx_gemm.cpp:164-173).
    resid: optional bf16 (M, N) residual fused into the bf16 epilogue. splits: None lets the library decide."""
    M, N, K = _check_operands(a, a_scale, b, b_scale, "mx_gemm")
    if not (out.is_contiguous() and out.size(0) == M and out.size(1) == N and out.dtype in (torch.bfloat16, torch.float32)):
        raise RuntimeError("mx_gemm: shape mismatch")
    kind = capi.OUT_BF16 if out.dtype == torch.bfloat16 else capi.OUT_F32
    if resid is not None and not (kind == capi.OUT_BF16 and resid.shape == out.shape and resid.dtype == torch.bfloat16
                                  and resid.is_contiguous()):
        raise RuntimeError("mx_gemm: the residual must be a contiguous bf16 tensor of the output's shape")
    s = lib.mxb200_gemm_splits(M, N, K) if splits is None else splits
    rp = resid.data_ptr() if resid is not None else None
    if s <= 1:
        if kind == capi.OUT_BF16:
            st = lib.mxb200_gemm_bf16(a.data_ptr(), a_scale.data_ptr(), b.data_ptr(), b_scale.data_ptr(), out.data_ptr(),
                                      rp, M, N, K, _stream())
        else:
            st = lib.mxb200_gemm_f32(a.data_ptr(), a_scale.data_ptr(), b.data_ptr(), b_scale.data_ptr(), out.data_ptr(),
                                     M, N, K, None, 0, _stream())
    else:
        nbytes = lib.mxb200_gemm_workspace_bytes(M, N, K, s)
        ws = _workspace(out.device, nbytes)
        st = lib.mxb200_gemm_splitk(a.data_ptr(), a_scale.data_ptr(), b.data_ptr(), b_scale.data_ptr(), out.data_ptr(),
                                    kind, rp, M, N, K, None, 0, s, ws.data_ptr(), ws.numel(), _stream())
    check(st, "mx_gemm")


def mx_gemm(a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor, b_scale: torch.Tensor,
            out_dtype: torch.dtype = torch.bfloat16, resid: Optional[torch.Tensor] = None,
            splits: Optional[int] = None) -> torch.Tensor:
    """a (M, K) . b (N, K)^T as out_dtype (src/nanochat/model/fp8/mx_gemm.h:18-24, mx_gemm.cpp:154-162)."""
    out = torch.empty((a.size(0), b.size(0)), dtype=out_dtype, device=a.device)
    mx_gemm_out(out, a, a_scale, b, b_scale, resid, splits)
    return out


def mx_gemm_f32(a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor, b_scale: torch.Tensor, out: torch.Tensor,
                accumulate: bool, alpha: Optional[torch.Tensor] = None, splits: Optional[int] = None) -> None:
    """out (M, N) fp32 (+)= alpha * a . b^T; alpha a device fp32 scalar (None: 1)
    (src/nanochat/model/fp8/mx_gemm.h:44-50, mx_gemm.cpp:214-319)."""
    M, N, K = _check_operands(a, a_scale, b, b_scale, "mx_gemm_f32")
    if not (out.is_cuda and out.is_contiguous() and out.dtype == torch.float32 and out.size(0) == M and out.size(1) == N):
        raise RuntimeError("mx_gemm_f32: expected a contiguous fp32 (M, N) output")
    if alpha is not None and not (alpha.is_cuda and alpha.dtype == torch.float32 and alpha.numel() == 1):
        raise RuntimeError("mx_gemm_f32: alpha must be a device fp32 scalar")
    ap = alpha.data_ptr() if alpha is not None else None
    s = lib.mxb200_gemm_splits(M, N, K) if splits is None else splits
    if s <= 1:
        st = lib.mxb200_gemm_f32(a.data_ptr(), a_scale.data_ptr(), b.data_ptr(), b_scale.data_ptr(), out.data_ptr(),
                                 M, N, K, ap, int(accumulate), _stream())
    else:
        nbytes = lib.mxb200_gemm_workspace_bytes(M, N, K, s)
        ws = _workspace(out.device, nbytes)
        st = lib.mxb200_gemm_splitk(a.data_ptr(), a_scale.data_ptr(), b.data_ptr(), b_scale.data_ptr(), out.data_ptr(),
                                    capi.OUT_F32, None, M, N, K, ap, int(accumulate), s, ws.data_ptr(), ws.numel(),
                                    _stream())
    check(st, "mx_gemm_f32")


def _check_mx_out(t: torch.Tensor, scale: torch.Tensor, rows: int, cols: int, what: str) -> None:
    """src/nanochat/model/fp8/mx_gemm.cpp:125-130."""
    if not (t.is_cuda and t.is_contiguous() and t.dtype == E4M3 and t.size(0) == rows and t.size(1) == cols
            and scale.numel() == rows * cols // 32):
        raise RuntimeError(f"{what}: expected e4m3 ({rows}, {cols}) with its MX scales")


def mx_gemm_relu_square(h: torch.Tensor, q: torch.Tensor, q_scale: torch.Tensor, q_t: torch.Tensor,
                        q_t_scale: torch.Tensor, a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor,
                        b_scale: torch.Tensor) -> bool:
    """h = mx_gemm(a, ..., bf16) into h and q = quantize_mx(h, True, True, True) into q, q_t (N, M) in one GEMM
    (src/nanochat/model/fp8/mx_gemm.h:29-35, mx_gemm.cpp:175-192). Returns True, as the reference does when its
    fused backend applies; there is no unfused fallback to report here."""
    M, N, K = _check_operands(a, a_scale, b, b_scale, "mx_gemm_relu_square")
    if not (h.is_cuda and h.is_contiguous() and h.dtype == torch.bfloat16 and h.size(0) == M and h.size(1) == N):
        raise RuntimeError("mx_gemm_relu_square: shape mismatch")
    _check_mx_out(q, q_scale, M, N, "mx_gemm_relu_square")
    _check_mx_out(q_t, q_t_scale, N, M, "mx_gemm_relu_square")
    check(lib.mxb200_gemm_relu_square(a.data_ptr(), a_scale.data_ptr(), b.data_ptr(), b_scale.data_ptr(), h.data_ptr(),
                                      q.data_ptr(), q_scale.data_ptr(), q_t.data_ptr(), q_t_scale.data_ptr(), M, N, K,
                                      _stream()), "mx_gemm_relu_square")
    return True


def mx_gemm_relu_square_bwd(a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor, b_scale: torch.Tensor,
                            h: torch.Tensor, dh: torch.Tensor, dh_scale: torch.Tensor, dh_t: torch.Tensor,
                            dh_t_scale: torch.Tensor) -> bool:
    """relu^2's backward from its dgrad GEMM in one GEMM: ga = mx_gemm(a, ..., bf16) (not written) and h (M, N) bf16
    -> quantize_mx_relu_square_bwd's outputs (src/nanochat/model/fp8/mx_gemm.h:37-42, mx_gemm.cpp:194-212)."""
    M, N, K = _check_operands(a, a_scale, b, b_scale, "mx_gemm_relu_square_bwd")
    if not (h.is_cuda and h.is_contiguous() and h.dtype == torch.bfloat16 and h.size(0) == M and h.size(1) == N):
        raise RuntimeError("mx_gemm_relu_square_bwd: shape mismatch")
    _check_mx_out(dh, dh_scale, M, N, "mx_gemm_relu_square_bwd")
    _check_mx_out(dh_t, dh_t_scale, N, M, "mx_gemm_relu_square_bwd")
    check(lib.mxb200_gemm_relu_square_bwd(a.data_ptr(), a_scale.data_ptr(), b.data_ptr(), b_scale.data_ptr(),
                                          h.data_ptr(), dh.data_ptr(), dh_scale.data_ptr(), dh_t.data_ptr(),
                                          dh_t_scale.data_ptr(), M, N, K, _stream()), "mx_gemm_relu_square_bwd")
    return True


# ------------------------------------------------------------------------------------------------ Linear

def mx_grad_direct(w: torch.Tensor) -> bool:
    """Whether backward may write w's gradient straight into w.grad: a contiguous fp32 leaf that requires
    grad (src/nanochat/model/fp8/fp8.h:114-116)."""
    return w.is_leaf and w.requires_grad and w.dtype == torch.float32 and w.is_contiguous()


def mx_grad_weights(go_t: torch.Tensor, go_scale_t: torch.Tensor, in_t: torch.Tensor, in_scale_t: torch.Tensor,
                    ws: Sequence[torch.Tensor], alpha: Optional[torch.Tensor] = None) -> None:
    """dW = alpha * go_t (n, N) . in_t (C, N)^T into the .grad of ws, whose rows concatenate to n: allocated (=)
    when undefined, else accumulated (+=). Several ws share one buffer, so one GEMM serves
    (src/nanochat/model/fp8/fp8.h:118-125, fp8.cpp:470-514)."""
    n, C = go_t.size(0), in_t.size(0)
    if sum(w.size(0) for w in ws) != n or any(w.size(1) != C for w in ws):
        raise RuntimeError("mx_grad_weights: weight rows must concatenate to the gradient's")
    merged = None
    if all(w.grad is not None for w in ws):
        g0 = ws[0].grad
        base = g0.data_ptr()
        contiguous, row = True, 0
        for w in ws:
            contiguous &= w.grad.data_ptr() == base + row * C * 4 and w.grad.is_contiguous() and w.grad.dtype == torch.float32
            row += w.size(0)
        if contiguous and len(ws) > 1 and g0._base is not None and g0._base.numel() == n * C:
            merged = g0._base.view(n, C)
        elif contiguous and len(ws) == 1:
            merged = g0
    if merged is not None:
        mx_gemm_f32(go_t, go_scale_t, in_t, in_scale_t, merged, True, alpha)
        return
    buf = torch.empty((n, C), dtype=torch.float32, device=go_t.device)
    mx_gemm_f32(go_t, go_scale_t, in_t, in_scale_t, buf, False, alpha)
    row = 0
    for w in ws:
        part = buf.narrow(0, row, w.size(0))
        if w.grad is None:
            w.grad = part  # row blocks of one buffer, as the reference's merged q/k/v
        else:
            w.grad.add_(part)
        row += w.size(0)


class _Float8Matmul(torch.autograd.Function):
    """One Linear under MX: y = x . w^T, dX = dY . w, dW = dY^T . x, every operand E4M3 with per-32 scales
    along the contraction (src/nanochat/model/fp8/fp8.cpp:240-260)."""

    @staticmethod
    def forward(ctx, x, w, cache):
        xq = quantize_mx(x)
        wq = quantize_fp8_weight(w, cache)
        ctx.save_for_backward(xq.data_t, xq.inv_scale_t, wq.data_t, wq.inv_scale_t)
        ctx.w = w
        ctx.direct = mx_grad_direct(w)
        return mx_gemm(xq.data, xq.inv_scale, wq.data, wq.inv_scale, torch.bfloat16)

    @staticmethod
    def backward(ctx, go):
        x_t, x_scale_t, w_t, w_scale_t = ctx.saved_tensors
        gq = quantize_mx(go.contiguous())
        dx = mx_gemm(gq.data, gq.inv_scale, w_t, w_scale_t, torch.bfloat16)
        if ctx.direct:
            mx_grad_weights(gq.data_t, gq.inv_scale_t, x_t, x_scale_t, [ctx.w])
            return dx, None, None
        dw = mx_gemm(gq.data_t, gq.inv_scale_t, x_t, x_scale_t, torch.float32)
        return dx, dw.to(ctx.w.dtype), None


class _MxQkv(torch.autograd.Function):
    """q, k, v = x . w_i^T with x quantized once and one GEMM each for the forward, the input gradient and the weight
    gradients: MX scales run along K, so the three weights concatenate along their rows and the three output
    gradients along their columns (src/nanochat/model/fp8/fp8.cpp:424-462)."""

    @staticmethod
    def forward(ctx, x, wq, wk, wv, gate_cols, cache, x_mx):
        sizes = (wq.size(0), wk.size(0), wv.size(0))
        xq = x_mx if x_mx is not None else quantize_mx(x)
        w, w_t, w_scale, w_scale_t = mx_qkv_weights(wq, wk, wv, cache)
        qkv = mx_gemm(xq.data, xq.inv_scale, w, w_scale, torch.bfloat16)
        ctx.save_for_backward(xq.data_t, xq.inv_scale_t, w_t, w_scale_t)
        ctx.ws, ctx.gate_cols, ctx.sizes = (wq, wk, wv), gate_cols, sizes
        ctx.direct = all(mx_grad_direct(t) for t in (wq, wk, wv))
        out = [qkv.narrow(1, 0, sizes[0]), qkv.narrow(1, sizes[0], sizes[1]), qkv.narrow(1, sizes[0] + sizes[1], sizes[2])]
        if gate_cols > 0:
            out.append(x.narrow(1, 0, gate_cols).contiguous())
        return tuple(out)

    @staticmethod
    def backward(ctx, *grads):
        x_t, x_scale_t, w_t, w_scale_t = ctx.saved_tensors
        N, sizes = x_t.size(1), ctx.sizes
        n = sum(sizes)
        dev = x_t.device
        g = torch.empty((N, n), dtype=E4M3, device=dev)
        g_t = torch.empty((n, N), dtype=E4M3, device=dev)
        g_scale, g_scale_t = empty_mx_scale(N, n, dev), empty_mx_scale(n, N, dev)
        row = 0
        for i in range(3):
            gi = grads[i] if grads[i] is not None else torch.zeros((N, sizes[i]), dtype=torch.bfloat16, device=dev)
            quantize_mx_into(gi.contiguous(), False, mx_out(g, g_scale, 0, row), mx_out(g_t, g_scale_t, row, 0))
            row += sizes[i]
        dx = mx_gemm(g, g_scale, w_t, w_scale_t, torch.bfloat16)
        if ctx.gate_cols > 0 and grads[3] is not None:
            dx.narrow(1, 0, ctx.gate_cols).add_(grads[3])
        if ctx.direct:
            mx_grad_weights(g_t, g_scale_t, x_t, x_scale_t, list(ctx.ws))
            return dx, None, None, None, None, None, None
        dw = mx_gemm(g_t, g_scale_t, x_t, x_scale_t, torch.float32)
        parts, row = [], 0
        for w, rows in zip(ctx.ws, sizes):
            parts.append(dw.narrow(0, row, rows).to(w.dtype))
            row += rows
        return (dx, *parts, None, None, None)


def fp8_qkv(x_2d: torch.Tensor, wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, gate_cols: int = 0,
            cache: Optional[Fp8WeightCache] = None, x_mx: Optional[Fp8Tensor] = None):
    """Attention's c_q, c_k, c_v as fp8_matmuls of the same x_2d (N, in) bf16, merged
    (src/nanochat/model/fp8/fp8.h:58-66, MX branch). Returns (q, k, v), views of one (N, q + k + v) buffer, plus
    x_2d[:, :gate_cols] when gate_cols > 0 (the value-embedding gate's input; its gradient is added to dx in the
    same pass). x_mx: x_2d already quantized in both layouts (residual_norm_mx), as the reference's attention path
    takes it (src/nanochat/model/attention/mx_attention.h:20, mx_attention.cpp:45); x_2d then carries autograd and the
    gate's columns only."""
    n = wq.size(0) + wk.size(0) + wv.size(0)
    if not (mx_fits(x_2d.size(0), x_2d.size(1)) and n % 128 == 0 and all(w.size(0) % 128 == 0 for w in (wq, wk, wv))
            and 0 <= gate_cols <= x_2d.size(1)):
        raise RuntimeError("fp8_qkv: MX needs N, in and every weight's rows % 128")
    if x_mx is not None and (x_mx.data is None or x_mx.data_t is None):
        raise RuntimeError("fp8_qkv: x_mx needs both layouts")
    return _MxQkv.apply(x_2d.contiguous(), wq, wk, wv, gate_cols, cache, x_mx)


class _Fp8ReluSquareMlp(torch.autograd.Function):
    """c_proj(relu(c_fc(x))^2) as two MX Linears with relu^2 folded into the GEMM epilogues: the forward quantizes
    relu(h)^2 in c_fc's epilogue, the backward quantizes dh = (go . w_proj) * 2h in the dgrad GEMM's epilogue without
    writing it; h is what is saved (src/nanochat/model/fp8/fp8.cpp:262-338, MX branch)."""

    @staticmethod
    def forward(ctx, x, w_fc, w_proj, fc_cache, proj_cache, x_mx):
        xq = x_mx if x_mx is not None else quantize_mx(x)
        fcq = quantize_fp8_weight(w_fc, fc_cache)
        h = torch.empty((x.size(0), w_fc.size(0)), dtype=torch.bfloat16, device=x.device)
        aq = empty_mx(h.size(0), h.size(1), h.device)
        mx_gemm_relu_square(h, aq.data, aq.inv_scale, aq.data_t, aq.inv_scale_t, xq.data, xq.inv_scale, fcq.data,
                            fcq.inv_scale)
        projq = quantize_fp8_weight(w_proj, proj_cache)
        ctx.save_for_backward(xq.data_t, xq.inv_scale_t, fcq.data_t, fcq.inv_scale_t, h, aq.data_t, aq.inv_scale_t,
                              projq.data_t, projq.inv_scale_t)
        ctx.w_fc, ctx.w_proj = w_fc, w_proj
        return mx_gemm(aq.data, aq.inv_scale, projq.data, projq.inv_scale, torch.bfloat16)

    @staticmethod
    def backward(ctx, grad_output):
        x_t, x_scale_t, fc_t, fc_scale_t, h, a_t, a_scale_t, proj_t, proj_scale_t = ctx.saved_tensors
        go = quantize_mx(grad_output.contiguous())

        def weight_grad(g_t, g_scale_t, in_t, in_scale_t, w):
            if mx_grad_direct(w):
                mx_grad_weights(g_t, g_scale_t, in_t, in_scale_t, [w])
                return None
            return mx_gemm(g_t, g_scale_t, in_t, in_scale_t, torch.float32).to(w.dtype)

        grad_proj = weight_grad(go.data_t, go.inv_scale_t, a_t, a_scale_t, ctx.w_proj)
        dhq = empty_mx(h.size(0), h.size(1), h.device)
        mx_gemm_relu_square_bwd(go.data, go.inv_scale, proj_t, proj_scale_t, h, dhq.data, dhq.inv_scale, dhq.data_t,
                                dhq.inv_scale_t)
        grad_x = mx_gemm(dhq.data, dhq.inv_scale, fc_t, fc_scale_t, torch.bfloat16)
        grad_fc = weight_grad(dhq.data_t, dhq.inv_scale_t, x_t, x_scale_t, ctx.w_fc)
        return grad_x, grad_fc, grad_proj, None, None, None


def relu_square_mlp_mx(N: int, cin: int, w_fc: torch.Tensor, w_proj: torch.Tensor) -> bool:
    """Whether fp8_relu_square_mlp of an (N, in) input runs under MX: every dim % 128
    (src/nanochat/model/fp8/fp8.h:56-58)."""
    return (mx_fits(N, cin) and mx_fits(w_fc.size(0), w_fc.size(1)) and mx_fits(w_proj.size(0), w_proj.size(1))
            and w_fc.size(1) == cin and w_proj.size(1) == w_fc.size(0))


def fp8_relu_square_mlp(x_2d: torch.Tensor, w_fc: torch.Tensor, w_proj: torch.Tensor,
                        fc_cache: Optional[Fp8WeightCache] = None, proj_cache: Optional[Fp8WeightCache] = None,
                        x_mx: Optional[Fp8Tensor] = None) -> torch.Tensor:
    """The MLP's c_proj(relu(c_fc(x)).square()) with both matmuls as fp8_matmul, bit for bit
    (src/nanochat/model/fp8/fp8.h:46-54). x_2d (N, in) bf16, w_fc (hidden, in), w_proj (out, hidden) -> (N, out).
    x_mx: x_2d already quantized in both layouts (residual_norm_mx); x_2d then only carries autograd."""
    if not relu_square_mlp_mx(x_2d.size(0), x_2d.size(1), w_fc, w_proj):
        raise RuntimeError("fp8_relu_square_mlp: MX needs N, in, hidden, out % 128")
    if x_mx is not None and (x_mx.data is None or x_mx.data_t is None):
        raise RuntimeError("fp8_relu_square_mlp: x_mx needs both layouts")
    return _Fp8ReluSquareMlp.apply(x_2d.contiguous(), w_fc, w_proj, fc_cache, proj_cache, x_mx)


def fp8_matmul(input_2d: torch.Tensor, weight: torch.Tensor, cache: Optional[Fp8WeightCache] = None) -> torch.Tensor:
    """input_2d (N, in) bf16, weight (out, in) -> (N, out) bf16 under the MX recipe
    (src/nanochat/model/fp8/fp8.h:40-44, fp8.cpp:566-571). Dims must be % 128: the reference falls back to its
    tensorwise recipe otherwise, which is outside this library."""
    if not (mx_fits(input_2d.size(0), input_2d.size(1)) and mx_fits(weight.size(0), weight.size(1))):
        raise RuntimeError("fp8_matmul: MX needs N, in, out % 128")
    return _Float8Matmul.apply(input_2d.contiguous(), weight, cache)


# ------------------------------------------------------------------------------------------------ chunked lm_head loss

def softcap_ce_loss(logits: torch.Tensor, targets: torch.Tensor, vocab: int, softcap: float,
                    loss: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None):
    """Per row of bf16 logits (rows, padded): lse of the soft-capped logits and loss = lse - capped[target]; rows with
    target < 0 get loss 0 (src/nanochat/model/ops/softcap_ce_kernel.h:13-22 with grad = false). Returns (loss, lse),
    written into the given fp32 tensors when present."""
    _require_cuda(logits, "softcap_ce_loss")
    rows, padded = logits.shape
    if not (logits.dtype == torch.bfloat16 and logits.stride(1) == 1 and targets.dtype == torch.int64
            and targets.is_contiguous() and targets.numel() == rows):
        raise RuntimeError("softcap_ce_loss: expected bf16 logits (rows, padded) and int64 targets (rows)")
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device) if loss is None else loss
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device) if lse is None else lse
    check(lib.mxb200_softcap_ce_loss(logits.data_ptr(), rows, logits.stride(0), targets.data_ptr(), vocab, padded,
                                     softcap, loss.data_ptr(), lse.data_ptr(), _stream()), "softcap_ce_loss")
    return loss, lse


def softcap_ce_grad_mx(logits: torch.Tensor, targets: torch.Tensor, lse: torch.Tensor, vocab: int, softcap: float,
                       out: MxOut, out_t: MxOut, grad_scale: Optional[torch.Tensor] = None,
                       num_valid: Optional[torch.Tensor] = None, scale_rule: int = SCALE_REFERENCE) -> None:
    """The loss's gradient with respect to the logits, MX-quantized (as quantize_mx of its bf16) into out / out_t
    without being written, from the logits and softcap_ce_loss's lse
    (src/nanochat/model/ops/softcap_ce_kernel.h:24-29). grad_scale: fp32 (rows) or one element (every row);
    num_valid: int64 scalar on the device that divides the scale."""
    _require_cuda(logits, "softcap_ce_grad_mx")
    rows, padded = logits.shape
    stride = 0
    if grad_scale is not None:
        if grad_scale.dtype != torch.float32 or not grad_scale.is_contiguous():
            raise RuntimeError("softcap_ce_grad_mx: grad_scale must be contiguous fp32")
        stride = 1 if grad_scale.dim() == 1 and grad_scale.numel() == rows and rows > 1 else 0
    if num_valid is not None and num_valid.dtype != torch.int64:
        raise RuntimeError("softcap_ce_grad_mx: num_valid must be int64")
    check(lib.mxb200_softcap_ce_grad_mx(logits.data_ptr(), rows, logits.stride(0), targets.data_ptr(), lse.data_ptr(),
                                        vocab, padded, softcap,
                                        grad_scale.data_ptr() if grad_scale is not None else None, stride,
                                        num_valid.data_ptr() if num_valid is not None else None, out, out_t,
                                        scale_rule, _stream()), "softcap_ce_grad_mx")


def _run_chunks(x, weight, targets, vocab, softcap, chunk_rows, losses, grad_x, grad_scale, num_valid, cache):
    """The MX branch of the reference's run_chunks (src/nanochat/model/ops/softcap_ce.cpp:27-110): per chunk of rows
    logits = xq[chunk] . wq^T, the loss pass, the gradient quantized straight from the logits (row-wise into a chunk
    buffer, transposed into one (padded, N) buffer), grad_x[chunk] = gq . wq_t^T. Returns (xq, g_all) whose transposes
    are the operands of the single weight-gradient GEMM, or (None, None) without grad_x."""
    N, C = x.shape
    padded = weight.size(0)
    grad = grad_x is not None
    xq = quantize_mx(x, True, grad)
    wq = quantize_fp8_weight(weight, cache)
    rows_max = min(N, chunk_rows)
    logits = torch.empty((rows_max, padded), dtype=torch.bfloat16, device=x.device)
    lse = torch.empty(rows_max, dtype=torch.float32, device=x.device)
    loss_scratch = torch.empty(rows_max, dtype=torch.float32, device=x.device) if losses is None else None
    g_all = empty_mx(N, padded, x.device, False, True) if grad else None
    blocks = C // 32
    for begin in range(0, N, chunk_rows):
        end = min(N, begin + chunk_rows)
        rows = end - begin
        buf = logits[:rows]
        mx_gemm_out(buf, xq.data[begin:end], xq.inv_scale[begin * blocks:end * blocks], wq.data, wq.inv_scale)
        softcap_ce_loss(buf, targets[begin:end], vocab, softcap,
                        losses[begin:end] if losses is not None else loss_scratch[:rows], lse[:rows])
        if not grad:
            continue
        gq = empty_mx(rows, padded, x.device, True, False)
        scale = None
        if grad_scale is not None:
            scale = grad_scale[begin:end] if grad_scale.dim() == 1 and grad_scale.numel() == N else grad_scale
        softcap_ce_grad_mx(buf, targets[begin:end], lse[:rows], vocab, softcap, mx_out(gq.data, gq.inv_scale, 0, 0),
                           mx_out(g_all.data_t, g_all.inv_scale_t, 0, begin), scale, num_valid)
        mx_gemm_out(grad_x[begin:end], gq.data, gq.inv_scale, wq.data_t, wq.inv_scale_t)
    return (xq, g_all) if grad else (None, None)


class _SoftcapCrossEntropy(torch.autograd.Function):
    """src/nanochat/model/ops/softcap_ce.cpp:118-205, MX branch: for mean/sum the incoming gradient is a scalar, so the
    forward computes grad_x and the weight gradient's operands at once and the backward only scales (one GEMM with
    alpha = the incoming gradient, straight into .grad when the weight is an fp32 leaf); for none the backward re-runs
    the chunks with the per-row gradient."""

    @staticmethod
    def forward(ctx, x, weight, targets, vocab, softcap, chunk_rows, reduction, needs_grad, cache):
        num_valid = (targets >= 0).sum()
        losses = torch.empty(x.size(0), dtype=torch.float32, device=x.device)
        precompute = needs_grad and reduction != "none"
        grad_x = torch.empty_like(x) if precompute else None
        xq, g_all = _run_chunks(x, weight, targets, vocab, softcap, chunk_rows, losses, grad_x, None,
                                num_valid if reduction == "mean" else None, cache)
        ctx.precomputed, ctx.weight = precompute, weight
        ctx.args = (vocab, softcap, chunk_rows, cache)
        if precompute:
            ctx.save_for_backward(grad_x, g_all.data_t, g_all.inv_scale_t, xq.data_t, xq.inv_scale_t)
        elif needs_grad:
            ctx.save_for_backward(x, weight, targets)
        if reduction == "mean":
            return losses.sum() / num_valid  # ignored targets have loss 0
        if reduction == "sum":
            return losses.sum()
        return losses

    @staticmethod
    def backward(ctx, g):
        saved = ctx.saved_tensors
        if not saved:
            raise RuntimeError("softcap_cross_entropy: backward without grad mode in forward")
        weight = ctx.weight
        if ctx.precomputed:
            grad_x, g_t, g_scale_t, x_t, x_scale_t = saved
            gw = g.to(torch.float32).reshape(1)
            if mx_grad_direct(weight):  # .grad (+)= g * dlogits^T . x, one GEMM
                mx_grad_weights(g_t, g_scale_t, x_t, x_scale_t, [weight], gw)
                return grad_x * g, None, None, None, None, None, None, None, None
            dw = torch.empty(weight.shape, dtype=torch.float32, device=weight.device)
            mx_gemm_f32(g_t, g_scale_t, x_t, x_scale_t, dw, False, gw)
            return grad_x * g, dw.to(weight.dtype), None, None, None, None, None, None, None
        x, weight, targets = saved
        vocab, softcap, chunk_rows, cache = ctx.args
        grad_x = torch.empty_like(x)
        xq, g_all = _run_chunks(x, weight, targets, vocab, softcap, chunk_rows, None, grad_x,
                                g.to(torch.float32).contiguous(), None, cache)
        dw = torch.empty(weight.shape, dtype=torch.float32, device=weight.device)
        mx_gemm_f32(g_all.data_t, g_all.inv_scale_t, xq.data_t, xq.inv_scale_t, dw, False)
        return grad_x, dw.to(weight.dtype), None, None, None, None, None, None, None


def softcap_cross_entropy(x: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, vocab_size: int,
                          softcap: float, chunk_rows: int, reduction: str = "mean",
                          cache: Optional[Fp8WeightCache] = None) -> torch.Tensor:
    """lm_head + logit softcap + cross-entropy a chunk of rows at a time under the MX recipe, so that the full
    (N, vocab) logits never exist (src/nanochat/model/ops/softcap_ce.h:16-24, recipe Mx). x: (N, C) bf16; weight:
    (V_padded, C) fp32 lm_head weight; targets: (N) int64, -1 = ignored; logits are cropped to vocab_size and capped as
    softcap * tanh(z / softcap); mean divides by the number of targets that are not ignored. MX needs N, C, chunk_rows
    and V_padded % 128 (the reference falls back to other recipes otherwise, which are outside this library)."""
    if x.dim() != 2 or targets.dim() != 1 or targets.size(0) != x.size(0):
        raise ValueError("softcap_cross_entropy expects x (N, C) and targets (N)")
    if chunk_rows < 1:
        raise ValueError("chunk_rows must be positive")
    if not x.is_cuda or x.dtype != torch.bfloat16:
        raise ValueError("softcap_cross_entropy expects bf16 CUDA activations")
    if reduction not in ("mean", "sum", "none"):
        raise ValueError("reduction must be mean, sum or none")
    if not (mx_fits(x.size(0), x.size(1)) and chunk_rows % 128 == 0 and weight.size(0) % 128 == 0
            and weight.size(0) >= vocab_size and weight.size(1) == x.size(1)):
        raise RuntimeError("softcap_cross_entropy: MX needs N, C, chunk_rows and the padded vocab % 128")
    needs_grad = torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad)
    return _SoftcapCrossEntropy.apply(x.contiguous(), weight, targets.to(torch.int64).contiguous(), int(vocab_size),
                                      float(softcap), int(chunk_rows), reduction, needs_grad, cache)
