"""Fused quantized gate/up projection + SwiGLU against the oracle (fp32 ground truth), through
the public wrappers and so through the C ABI.  Geometries are chosen to reach the direct
epilogue, the workspace split-K reduce and the cluster split-K reduce of the kernel."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from full_inference_engine_b200.kernels import swiglu, w4a16_format as w4, w4a16_linear, w8a16_linear
from full_inference_engine_b200.quantization import Int8Linear, W4A16Linear
from full_inference_engine_b200.quantization.fused_mlp import (
    FusedGateUpSwiGLU, install_fused_swiglu, uninstall_fused_swiglu,
)
from oracle import wq_oracle as oracle
from tests.helpers import assert_within_bar, to_np

pytestmark = pytest.mark.gpu
DEV = "cuda"

# (K, N per projection): direct epilogue (K too short to split), workspace split-K (narrow
# tiles, few of them), cluster split-K (wide tiles, few of them), ragged N
GEOMETRIES = [(512, 2560), (2048, 320), (4096, 512), (1024, 200)]
ROWS = [1, 5, 16, 48, 64, 144, 300]


def _truth(x, gate_deq, up_deq, gate_bias=None, up_bias=None):
    xf = to_np(x).astype(np.float32)
    g = oracle.linear_fp32(xf, gate_deq, None if gate_bias is None else to_np(gate_bias))
    u = oracle.linear_fp32(xf, up_deq, None if up_bias is None else to_np(up_bias))
    return oracle.swiglu_fp32(g, u)


def _weights(k, n, seed):
    torch.manual_seed(seed)
    return (torch.randn(n, k, device=DEV) * 0.05, torch.randn(n, k, device=DEV) * 0.05)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("k,n", GEOMETRIES)
def test_w4_reference_layout_pairs(k, n, dtype):
    wg, wu = _weights(k, n, k + n)
    (pg, sg), (pu, su) = w4.quantize_weight_w4_grouped(wg), w4.quantize_weight_w4_grouped(wu)
    packed, scales = swiglu.interleave_gate_up(pg, pu), swiglu.interleave_gate_up(sg, su)
    gate_deq = oracle.unpack_w4(to_np(pg), to_np(sg), k)
    up_deq = oracle.unpack_w4(to_np(pu), to_np(su), k)
    for m in ROWS:
        x = torch.randn(m, k, device=DEV).to(dtype)
        y = swiglu.w4a16_gate_up_swiglu(x, packed, scales)
        assert y.shape == (m, n) and y.dtype is dtype
        assert_within_bar(y, _truth(x, gate_deq, up_deq))


@pytest.mark.parametrize("k,n", GEOMETRIES)
def test_w4_asymmetric_layout_pairs_with_bias(k, n):
    wg, wu = _weights(k, n, 7 * k + n)
    qg, qu = w4.quantize_weight_w4_asym(wg + 0.01), w4.quantize_weight_w4_asym(wu - 0.01)
    packed, scales, zeros = (swiglu.interleave_gate_up(a, b) for a, b in zip(qg, qu))
    bg, bu = torch.randn(n, device=DEV).half() * 0.1, torch.randn(n, device=DEV).half() * 0.1
    bias = swiglu.interleave_gate_up(bg, bu)
    gate_deq = oracle.unpack_w4_asym(*(to_np(t) for t in qg), k)
    up_deq = oracle.unpack_w4_asym(*(to_np(t) for t in qu), k)
    for m in ROWS:
        x = torch.randn(m, k, device=DEV).half()
        y = swiglu.w4a16_gate_up_swiglu(x, packed, scales, bias, zeros_pairs=zeros)
        assert_within_bar(y, _truth(x, gate_deq, up_deq, bg, bu))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("k,n", GEOMETRIES)
def test_w8_pairs(k, n, dtype):
    wg, wu = _weights(k, n, 3 * k + n)
    (qg, sg), (qu, su) = (w8a16_linear.quantize_weight_per_channel_fp32_scales(w) for w in (wg, wu))
    qweight, scales = swiglu.interleave_gate_up(qg, qu), swiglu.interleave_gate_up(sg, su)
    gate_deq, up_deq = oracle.dequant_w8(to_np(qg), to_np(sg)), oracle.dequant_w8(to_np(qu), to_np(su))
    for m in ROWS:
        x = torch.randn(m, k, device=DEV).to(dtype)
        y = swiglu.w8a16_gate_up_swiglu(x, qweight, scales)
        assert y.shape == (m, n)
        assert_within_bar(y, _truth(x, gate_deq, up_deq))


def test_fused_equals_two_projections_then_swiglu():
    """The fused launch against this library's own unfused route (two forwards, torch SwiGLU):
    the only difference is that the fused one never rounds gate and up to fp16."""
    k, n, m = 2048, 1536, 33
    wg, wu = _weights(k, n, 11)
    (pg, sg), (pu, su) = w4.quantize_weight_w4_grouped(wg), w4.quantize_weight_w4_grouped(wu)
    x = torch.randn(m, k, device=DEV).half()
    unfused = swiglu.swiglu_reference(w4a16_linear.w4a16_linear(x, pg, sg), w4a16_linear.w4a16_linear(x, pu, su))
    fused = swiglu.w4a16_gate_up_swiglu(x, swiglu.interleave_gate_up(pg, pu), swiglu.interleave_gate_up(sg, su))
    scale = float(unfused.float().abs().max())
    assert float((fused.float() - unfused.float()).abs().max()) <= 2e-3 * scale


def test_errors():
    k, n = 512, 129          # odd number of rows cannot be pairs
    w = torch.randn(n, k, device=DEV) * 0.05
    p, s = w4.quantize_weight_w4_grouped(w)
    x = torch.randn(4, k, device=DEV).half()
    with pytest.raises(ValueError):
        w4a16_linear.w4a16_linear(x, p, s, swiglu_pairs=True)
    p2, s2 = w4.quantize_weight_w4_grouped(torch.randn(256, k, device=DEV) * 0.05)
    with pytest.raises(RuntimeError, match="unsupported"):
        w4a16_linear.w4a16_linear(x, p2, s2, kernel="gemv", swiglu_pairs=True)
    with pytest.raises(ValueError):
        swiglu.interleave_gate_up(p, p2)


class _FeedForward(torch.nn.Module):
    def __init__(self, hidden, inner):
        super().__init__()
        self.gate_proj = torch.nn.Linear(hidden, inner, bias=False)
        self.up_proj = torch.nn.Linear(hidden, inner, bias=False)
        self.down_proj = torch.nn.Linear(inner, hidden, bias=False)

    def forward(self, x):
        return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


@pytest.mark.parametrize("kind", ["w4a16", "int8"])
def test_installed_feed_forward(kind):
    torch.manual_seed(5)
    block = torch.nn.Sequential(_FeedForward(256, 1024), _FeedForward(256, 512)).to(DEV).half()
    for ff in block:
        for name in ("gate_proj", "up_proj", "down_proj"):
            linear = getattr(ff, name)
            if kind == "w4a16":
                shell = W4A16Linear(linear.in_features, linear.out_features, device=DEV)
                shell.quantize_from(linear.weight.data)
            else:
                shell = Int8Linear(linear)
            setattr(ff, name, shell)
    x = torch.randn(3, 7, 256, device=DEV).half()
    with torch.no_grad():
        before = block(x)
        assert install_fused_swiglu(block) == 2
        assert isinstance(block[0].fused_gate_up_swiglu, FusedGateUpSwiGLU) and block[0].gate_proj is None
        after = block(x)
        assert install_fused_swiglu(block) == 2          # idempotent
        for ff in block:
            ff.fused_gate_up_swiglu.reference = True
        reference = block(x)
        assert uninstall_fused_swiglu(block) == 2
        restored = block(x)
    assert torch.equal(before, restored)
    scale = float(before.float().abs().max())
    assert float((after.float() - before.float()).abs().max()) <= 1e-2 * scale
    assert float((after.float() - reference.float()).abs().max()) <= 1e-2 * scale
