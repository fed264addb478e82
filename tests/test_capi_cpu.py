"""CPU: the C-ABI library loads and exports every symbol include/mxb200.h declares; host-side logic of the
reference-interface mirror (views, cache, bucket layout). No compute calls: there is no GPU here."""
import os
import re

import pytest
import torch

import nanochat_cpp_b200 as nc
from nanochat_cpp_b200.dp_step import GradBucket, StepConfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "mxb200.h")).read()
    declared = set(re.findall(r"MXB200_API\s+[\w\s\*]+?\b(mxb200_\w+)\s*\(", header))
    assert len(declared) >= 12
    assert declared == set(nc.capi.SYMBOLS)
    for name in declared:
        assert hasattr(nc.capi.lib, name), name
    assert nc.capi.lib.mxb200_version() >= 100


def test_status_strings_and_no_cpu_fallback():
    for st in range(0, 10):
        assert nc.capi.strerror(st)
    assert "no CPU fallback" in nc.capi.strerror(nc.capi.ERR_DEVICE)
    if not torch.cuda.is_available():
        # without a device every entry point refuses instead of computing on the host
        assert nc.capi.lib.mxb200_gemm_bf16(None, None, None, None, None, None, 128, 128, 128, None) == nc.capi.ERR_DEVICE
        out = nc.capi.MxOut(None, 0, None, 0)
        assert nc.capi.lib.mxb200_quantize_mx(None, 1, 128, 128, out, out, 0, 0, None) == nc.capi.ERR_DEVICE
        with pytest.raises(RuntimeError):
            nc.quantize_mx(torch.zeros(128, 128, dtype=torch.bfloat16))


def test_mx_out_view_arithmetic():
    """fp8.cpp:117-120: data + row * ld + col, scale + ((row / 128) * tiles + col / 128) * 512."""
    data = torch.empty((512, 384), dtype=torch.uint8)
    scale = torch.empty(512 * 384 // 32, dtype=torch.uint8)
    v = nc.mx_out(data, scale, 256, 128)
    assert v.data == data.data_ptr() + 256 * 384 + 128
    assert v.ld == 384 and v.scale_tiles == 3
    assert v.scale == scale.data_ptr() + ((256 // 128) * 3 + 1) * 512
    with pytest.raises(RuntimeError):
        nc.mx_out(data, scale, 64, 0)
    assert nc.mx_fits(256, 384) and not nc.mx_fits(256, 96)
    assert nc.fp8_eligible(1536, 1536) and not nc.fp8_eligible(12, 1536)


def test_weight_cache_reuses_until_version_changes():
    """Fp8.WeightCacheReusesUntilWeightChanges (tests/test_fp8.cpp:73-90), host logic only."""
    w = torch.randn(256, 128)
    made = []

    def make():
        made.append(1)
        return [torch.zeros(1)]
    cache = nc.Fp8WeightCache(enabled=True)
    a = cache.get(1, [w], make)
    b = cache.get(1, [w], make)
    assert a is b and len(made) == 1
    with torch.no_grad():
        w.mul_(2)  # as an optimizer step: bumps the version
    c = cache.get(1, [w], make)
    assert c is not a and len(made) == 2
    cache.enabled = False
    assert cache.get(1, [w], make) is not cache.get(1, [w], make)


def test_bucket_layout():
    cfg = StepConfig(n_layer=2, n_embd=256, vocab=512, tokens=256, chunk_rows=128)
    b = GradBucket(cfg, torch.device("cpu"), world=1)
    assert b.numel == 2 * cfg.layer_params + cfg.lm_head_params
    assert cfg.layer_params == 12 * 256 * 256
    # the reference's stacks by shape: (C, C) x 4 per layer, then (C, 4C), then (4C, C); layer 1's MLP fc gradient is
    # entry 1 of the last one
    m = b.matrix(1, 2)
    assert m.shape == (1024, 256)
    cc, c4c = 8 * 256 * 256, 2 * 256 * 1024
    assert m.data_ptr() == b.buffer.data_ptr() + 2 * (cc + c4c + 1024 * 256)
    assert b.matrix(1, 0).data_ptr() == b.buffer.data_ptr() + 2 * (4 * 256 * 256)
    assert b.lm_head().shape == (512, 256)
    assert abs(StepConfig().flops_per_step() / 1e12 - 71.743) < 0.01
