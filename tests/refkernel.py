"""ctypes door to the reference's own CUDA quantizer (oracle/_ref/libnanochat_ref_quant.so), built by
oracle/Makefile from the unmodified reference source. A checker for GPU tests; absent when the reference
tree was not available at build time."""
from __future__ import annotations

import ctypes
import os

import torch

_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                     "libnanochat_ref_quant.so")
_lib = None


def available() -> bool:
    return os.path.exists(_PATH)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_PATH)
        vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
        _lib.ref_quantize_mx.argtypes = [vp, i32, i64, i64, vp, i64, vp, i64, vp, i64, vp, i64, i32, vp]
        _lib.ref_quantize_mx_relu_square_bwd.argtypes = [vp, vp, i64, i64, vp, i64, vp, i64, vp, i64, vp, i64, vp]
    return _lib


def quantize_mx(x: torch.Tensor, relu_square: bool = False, h: torch.Tensor | None = None):
    """Runs nanochat::kernels::quantize_mx (or the relu^2 backward variant when h is given) on the GPU and
    returns (data, scale, data_t, scale_t) uint8 tensors."""
    R, C = x.shape
    dev = x.device
    data = torch.zeros((R, C), dtype=torch.uint8, device=dev)
    data_t = torch.zeros((C, R), dtype=torch.uint8, device=dev)
    scale = torch.zeros(R * C // 32, dtype=torch.uint8, device=dev)
    scale_t = torch.zeros(R * C // 32, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    if h is None:
        err = lib().ref_quantize_mx(x.data_ptr(), int(x.dtype == torch.bfloat16), R, C, data.data_ptr(), C,
                                    scale.data_ptr(), C // 128, data_t.data_ptr(), R, scale_t.data_ptr(), R // 128,
                                    int(relu_square), stream)
    else:
        err = lib().ref_quantize_mx_relu_square_bwd(x.data_ptr(), h.data_ptr(), R, C, data.data_ptr(), C,
                                                    scale.data_ptr(), C // 128, data_t.data_ptr(), R,
                                                    scale_t.data_ptr(), R // 128, stream)
    assert err == 0, f"reference kernel launch failed: cudaError {err}"
    return data, scale, data_t, scale_t


def _bind_residual_norm(l):
    vp, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
    l.ref_residual_norm_fwd.argtypes = [vp] * 9 + [i64, i32, f32, vp]
    l.ref_residual_norm_mx_fwd.argtypes = [vp] * 9 + [i64, i32, f32, vp, i64, vp, i64, vp, i64, vp, i64, i32, vp]


def residual_norm(x, r=None, x0=None, lr=None, l0=None, layer=0, gate_cols=0, mx=True,
                  eps=float(torch.finfo(torch.float32).eps)):
    """Runs nanochat::kernels::residual_norm_mx_fwd (mx) or residual_norm_fwd on the GPU. Returns a dict of
    res, s (None unless r and x0), rstd, n (bf16, full width: only the first gate_cols columns are written with mx)
    and, with mx, data / scale / data_t / scale_t."""
    l = lib()
    if not hasattr(l, "_rn_bound"):
        _bind_residual_norm(l)
        l._rn_bound = True
    R, C = x.shape
    dev = x.device
    blend = x0 is not None
    res = torch.zeros_like(x)
    n = torch.zeros_like(x)
    s = torch.zeros_like(x) if (r is not None and blend) else None
    rstd = torch.zeros(R, dtype=torch.float32, device=dev)
    ptr = lambda t: t.data_ptr() if t is not None else None
    lam = lambda t: t.data_ptr() + 4 * layer if blend else None
    stream = torch.cuda.current_stream().cuda_stream
    base = [x.data_ptr(), ptr(r), ptr(x0), lam(lr), lam(l0), ptr(s), res.data_ptr(), n.data_ptr(), rstd.data_ptr(),
            R, C, eps]
    out = {"res": res, "s": s, "rstd": rstd, "n": n}
    if mx:
        data = torch.zeros((R, C), dtype=torch.uint8, device=dev)
        data_t = torch.zeros((C, R), dtype=torch.uint8, device=dev)
        scale = torch.zeros(R * C // 32, dtype=torch.uint8, device=dev)
        scale_t = torch.zeros(R * C // 32, dtype=torch.uint8, device=dev)
        err = l.ref_residual_norm_mx_fwd(*base, data.data_ptr(), C, scale.data_ptr(), C // 128, data_t.data_ptr(), R,
                                         scale_t.data_ptr(), R // 128, gate_cols, stream)
        out.update(data=data, scale=scale, data_t=data_t, scale_t=scale_t)
    else:
        err = l.ref_residual_norm_fwd(*base, stream)
    assert err == 0, f"reference kernel launch failed: {err}"
    return out


def _bind_softcap(l):
    vp, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
    l.ref_softcap_ce.argtypes = [vp, i64, i64, vp, i32, i32, f32, vp, vp, i64, vp, i32, vp, vp]
    l.ref_softcap_ce_grad_mx.argtypes = [vp, i64, i64, vp, vp, i32, i32, f32, vp, i64, vp, vp, i64, vp, i64, vp, i64, vp,
                                         i64, vp]


def softcap_ce(logits, targets, vocab, softcap, grad=False, grad_scale=None, num_valid=None):
    """Runs nanochat::kernels::softcap_ce on a copy of the logits. Returns (loss, lse, grad): grad is the bf16 gradient
    the kernel wrote over the logits when grad is set, else None."""
    l = lib()
    if not hasattr(l, "_ce_bound"):
        _bind_softcap(l)
        l._ce_bound = True
    z = logits.clone()
    rows, padded = z.shape
    loss = torch.zeros(rows, dtype=torch.float32, device=z.device)
    lse = torch.zeros(rows, dtype=torch.float32, device=z.device)
    err = l.ref_softcap_ce(z.data_ptr(), rows, padded, targets.data_ptr(), vocab, padded, softcap, loss.data_ptr(),
                           grad_scale.data_ptr() if grad_scale is not None else None, 1,
                           num_valid.data_ptr() if num_valid is not None else None, int(grad), lse.data_ptr(),
                           torch.cuda.current_stream().cuda_stream)
    assert err == 0, f"reference kernel launch failed: {err}"
    return loss, lse, (z if grad else None)


def softcap_ce_grad_mx(logits, targets, lse, vocab, softcap, grad_scale=None, num_valid=None):
    """Runs nanochat::kernels::softcap_ce_grad_mx. Returns (data, scale, data_t, scale_t)."""
    l = lib()
    if not hasattr(l, "_ce_bound"):
        _bind_softcap(l)
        l._ce_bound = True
    R, C = logits.shape
    dev = logits.device
    data = torch.zeros((R, C), dtype=torch.uint8, device=dev)
    data_t = torch.zeros((C, R), dtype=torch.uint8, device=dev)
    scale = torch.zeros(R * C // 32, dtype=torch.uint8, device=dev)
    scale_t = torch.zeros(R * C // 32, dtype=torch.uint8, device=dev)
    err = l.ref_softcap_ce_grad_mx(logits.data_ptr(), R, C, targets.data_ptr(), lse.data_ptr(), vocab, C, softcap,
                                   grad_scale.data_ptr() if grad_scale is not None else None, 1,
                                   num_valid.data_ptr() if num_valid is not None else None, data.data_ptr(), C,
                                   scale.data_ptr(), C // 128, data_t.data_ptr(), R, scale_t.data_ptr(), R // 128,
                                   torch.cuda.current_stream().cuda_stream)
    assert err == 0, f"reference kernel launch failed: {err}"
    return data, scale, data_t, scale_t
