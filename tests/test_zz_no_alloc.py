"""mxb200_gemm_splitk_static, the split-K entry point for callers that cannot allocate device memory.

A backend plugged in at nanochat-cpp's kernel seam receives pointers and a stream but no workspace, is called
from autograd worker threads mid-backward, and may run in a process whose allocator already holds all of HBM;
none of these can afford a cudaMalloc. The entry point therefore keeps its scratch in an array inside the
library's device image. This file checks, through the C ABI, that it gives the same result as the
caller-workspace entry point on two calls in a row (the array is shared and keeps the first call's contents),
and that it refuses problems larger than the array. Collected last on purpose.
"""
import pytest
import torch

import nanochat_cpp_b200 as nc

pytestmark = pytest.mark.gpu


def _operands(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(M, K, generator=g) * torch.logspace(-1, 1, K)).to(torch.bfloat16).cuda()
    b = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    return nc.quantize_mx(a, True, False), nc.quantize_mx(b, True, False)


def _with_caller_workspace(qa, qb, out, kind, M, N, K, splits, alpha=None, accumulate=0):
    lib = nc.capi.lib
    need = lib.mxb200_gemm_workspace_bytes(M, N, K, splits)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    st = lib.mxb200_gemm_splitk(qa.data.data_ptr(), qa.inv_scale.data_ptr(), qb.data.data_ptr(), qb.inv_scale.data_ptr(),
                                out.data_ptr(), kind, None, M, N, K, alpha, accumulate, splits, ws.data_ptr(), need,
                                torch.cuda.current_stream().cuda_stream)
    assert st == nc.capi.OK, nc.capi.strerror(st)


def _static(qa, qb, out, kind, M, N, K, splits, alpha=None, accumulate=0):
    return nc.capi.lib.mxb200_gemm_splitk_static(
        qa.data.data_ptr(), qa.inv_scale.data_ptr(), qb.data.data_ptr(), qb.inv_scale.data_ptr(), out.data_ptr(), kind,
        None, M, N, K, alpha, accumulate, splits, torch.cuda.current_stream().cuda_stream)


def test_static_scratch_matches_caller_workspace_twice_in_a_row():
    nc.capi.lib.mxb200_set_gemm_config(0, 0)
    # first call: a weight-gradient-like shape, fp32 output, 4 slices
    M, N, K = 512, 768, 4096
    qa, qb = _operands(M, N, K, seed=31)
    want = torch.empty(M, N, device="cuda")
    _with_caller_workspace(qa, qb, want, nc.capi.OUT_F32, M, N, K, 4)
    got = torch.full((M, N), float("nan"), device="cuda")
    assert _static(qa, qb, got, nc.capi.OUT_F32, M, N, K, 4) == nc.capi.OK
    torch.cuda.synchronize()
    assert torch.equal(got, want)  # same kernel, fixed summation order: identical bits (tests elsewhere allow 1e-6)

    # second call right after, other shape and slice count, += with a device alpha: the array still holds the
    # first call's partial tiles and must not leak them
    M2, N2, K2 = 256, 384, 2048
    qa2, qb2 = _operands(M2, N2, K2, seed=32)
    alpha = torch.full((1,), 0.25, device="cuda")
    base = torch.randn(M2, N2, generator=torch.Generator().manual_seed(33)).cuda()
    want2 = base.clone()
    _with_caller_workspace(qa2, qb2, want2, nc.capi.OUT_F32, M2, N2, K2, 2, alpha.data_ptr(), 1)
    got2 = base.clone()
    assert _static(qa2, qb2, got2, nc.capi.OUT_F32, M2, N2, K2, 2, alpha.data_ptr(), 1) == nc.capi.OK
    torch.cuda.synchronize()
    assert torch.equal(got2, want2)
    rel = ((got2.double() - want2.double()).norm() / want2.double().norm()).item()
    assert rel < 1e-6

    # and a bf16 output, as the gradient bucket takes it
    want3 = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    _with_caller_workspace(qa, qb, want3, nc.capi.OUT_BF16, M, N, K, 2)
    got3 = torch.empty_like(want3)
    assert _static(qa, qb, got3, nc.capi.OUT_BF16, M, N, K, 2) == nc.capi.OK
    torch.cuda.synchronize()
    assert torch.equal(got3, want3)
    assert nc.capi.device_status() == 0


def test_static_scratch_refuses_what_does_not_fit():
    M, N, K = 4608, 1536, 16384  # needs 216 tiles x 2 slices x 128 KB > 32 MiB
    need = nc.capi.lib.mxb200_gemm_workspace_bytes(M, N, K, 2)
    assert need > nc.capi.STATIC_SCRATCH_BYTES
    dummy = torch.empty(16, dtype=torch.uint8, device="cuda")
    p = dummy.data_ptr()
    st = nc.capi.lib.mxb200_gemm_splitk_static(p, p, p, p, p, nc.capi.OUT_F32, None, M, N, K, None, 0, 2,
                                               torch.cuda.current_stream().cuda_stream)
    assert st == nc.capi.ERR_WORKSPACE
    assert "workspace" in nc.capi.strerror(st)


def test_static_scratch_calls_take_no_device_memory():
    """What the entry point is for: across its calls the device's free memory does not move (no cudaMalloc by the
    library, the runtime or an allocator on its behalf). Outputs are allocated beforehand; the first call on the
    device, which looks up the array's address, is made before the measurement."""
    M, N, K = 512, 768, 4096
    qa, qb = _operands(M, N, K, seed=34)
    got = torch.empty(M, N, device="cuda")
    again = torch.empty(M, N, device="cuda")
    assert _static(qa, qb, got, nc.capi.OUT_F32, M, N, K, 2) == nc.capi.OK
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    reserved_before = torch.cuda.memory_reserved()
    assert _static(qa, qb, got, nc.capi.OUT_F32, M, N, K, 4) == nc.capi.OK
    assert _static(qa, qb, again, nc.capi.OUT_F32, M, N, K, 4) == nc.capi.OK
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.cuda.memory_reserved() == reserved_before
    assert torch.equal(got, again)
