"""Host-side logic of the fused gate/up + SwiGLU layer: row interleaving, module construction
and its error behaviour, reference-mode arithmetic, install/uninstall.  The CUDA quantizers are
swapped for the CPU oracle so nothing here needs a GPU."""

from __future__ import annotations

import re
import os

import numpy as np
import pytest
import torch
from torch import nn

from full_inference_engine_b200 import _lib
from full_inference_engine_b200.kernels import swiglu
from full_inference_engine_b200.quantization import Int8Linear, W4A16Linear
from full_inference_engine_b200.quantization import int8 as int8_mod
from full_inference_engine_b200.quantization import w4a16 as w4_mod
from full_inference_engine_b200.quantization.fused_mlp import (
    FusedGateUpSwiGLU, install_fused_swiglu, uninstall_fused_swiglu,
)
from oracle import wq_oracle as oracle

GROUP = 32


@pytest.fixture(autouse=True)
def oracle_quantizers(monkeypatch):
    def w4(weight, group_size):
        p, s = oracle.quantize_w4_grouped(weight.float().numpy(), group_size)
        return torch.from_numpy(p), torch.from_numpy(s)

    def w8(weight):
        q, s = oracle.quantize_w8_int8linear(weight.float().numpy())
        return torch.from_numpy(q), torch.from_numpy(s)

    monkeypatch.setattr(w4_mod, "_quantize", w4)
    monkeypatch.setattr(int8_mod, "_quantize", w8)


def _w4(linear: nn.Linear) -> W4A16Linear:
    shell = W4A16Linear(linear.in_features, linear.out_features, group_size=GROUP, bias=linear.bias is not None)
    shell.quantize_from(linear.weight.data)
    shell.set_bias(None if linear.bias is None else linear.bias.data)
    return shell


def test_interleave_matches_the_oracle_and_commutes_with_quantization():
    torch.manual_seed(0)
    gate, up = torch.randn(6, 64), torch.randn(6, 64)
    rows = swiglu.interleave_gate_up(gate, up)
    assert torch.equal(rows[0::2], gate) and torch.equal(rows[1::2], up)
    assert np.array_equal(rows.numpy(), oracle.interleave_rows(gate.numpy(), up.numpy()))
    # quantize-then-interleave == interleave-then-quantize (row-wise statistics)
    pg, sg = oracle.quantize_w4_grouped(gate.numpy(), GROUP)
    pu, su = oracle.quantize_w4_grouped(up.numpy(), GROUP)
    pj, sj = oracle.quantize_w4_grouped(rows.numpy(), GROUP)
    assert np.array_equal(oracle.interleave_rows(pg, pu), pj)
    assert np.array_equal(oracle.interleave_rows(sg, su).view(np.uint16), sj.view(np.uint16))
    with pytest.raises(ValueError):
        swiglu.interleave_gate_up(gate, up[:5])


def test_flag_value_matches_the_header():
    header = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "b200q.h")
    text = open(header).read()
    value = int(re.search(r"#define\s+B200Q_FLAG_SWIGLU_PAIRS\s+(0x[0-9a-fA-F]+)", text).group(1), 16)
    assert value == _lib.FLAG_SWIGLU_PAIRS
    assert value & _lib.FLAG_STATIC_WEIGHTS == 0 and value & 0xFF == 0


@pytest.mark.parametrize("bias", [False, True])
def test_reference_mode_equals_the_two_modules_and_the_reference_swiglu(bias):
    torch.manual_seed(1)
    gate, up = nn.Linear(64, 96, bias=bias), nn.Linear(64, 96, bias=bias)
    qg, qu = _w4(gate), _w4(up)
    qg.reference = qu.reference = True
    fused = FusedGateUpSwiGLU(qg, qu)
    fused.reference = True
    x = torch.randn(2, 5, 64)
    expected = swiglu.swiglu_reference(qg(x), qu(x))
    assert torch.equal(fused(x), expected)
    assert fused.packed.shape == (192, 32) and fused.scales.shape == (192, 2)
    with pytest.raises(RuntimeError):
        fused.reference = False
        fused(x)                       # CPU tensors never reach a kernel


def test_int8_pair_and_construction_errors():
    torch.manual_seed(2)
    gate, up = nn.Linear(32, 48), nn.Linear(32, 48)
    a, b = Int8Linear(gate), Int8Linear(up)
    a.reference = b.reference = True
    fused = FusedGateUpSwiGLU(a, b)
    fused.reference = True
    x = torch.randn(4, 32)
    assert torch.allclose(fused(x), swiglu.swiglu_reference(a(x), b(x)), atol=1e-6)
    assert fused.qweight.shape == (96, 32) and fused.scales.dtype is torch.float32
    with pytest.raises(ValueError):
        FusedGateUpSwiGLU(a, _w4(nn.Linear(32, 48)))               # mixed kinds
    with pytest.raises(ValueError):
        FusedGateUpSwiGLU(a, Int8Linear(nn.Linear(32, 40)))        # geometry
    with pytest.raises(ValueError):
        FusedGateUpSwiGLU(a, Int8Linear(nn.Linear(32, 48, bias=False)))
    with pytest.raises(ValueError):
        FusedGateUpSwiGLU(gate, up)                                 # not quantized


class _FeedForward(nn.Module):
    def __init__(self):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = nn.Linear(64, 96), nn.Linear(64, 96), nn.Linear(96, 64)

    def forward(self, x):
        return self.down_proj(nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


def test_install_and_uninstall():
    torch.manual_seed(3)
    model = nn.Sequential(_FeedForward(), _FeedForward())
    with pytest.raises(RuntimeError):
        install_fused_swiglu(model)                                 # nothing quantized yet
    for ff in model:
        for name in ("gate_proj", "up_proj", "down_proj"):
            shell = _w4(getattr(ff, name))
            shell.reference = True
            setattr(ff, name, shell)
    x = torch.randn(3, 64)
    before = model(x)
    buffers_before = sum(b.numel() * b.element_size() for b in model.buffers())
    assert install_fused_swiglu(model) == 2
    for ff in model:
        ff.fused_gate_up_swiglu.reference = True
        assert ff.gate_proj is None and ff.up_proj is None
    assert sum(b.numel() * b.element_size() for b in model.buffers()) == buffers_before
    after = model(x)
    assert torch.allclose(after, before, atol=1e-5)
    assert uninstall_fused_swiglu(model) == 2
    assert isinstance(model[0].gate_proj, W4A16Linear) and not hasattr(model[0], "fused_gate_up_swiglu")
    assert torch.equal(model(x), before)


def test_argmax_flag_value_matches_the_header():
    header = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "b200q.h")
    value = int(re.search(r"#define\s+B200Q_FLAG_ARGMAX\s+(0x[0-9a-fA-F]+)", open(header).read()).group(1), 16)
    assert value == _lib.FLAG_ARGMAX and value & (_lib.FLAG_SWIGLU_PAIRS | _lib.FLAG_STATIC_WEIGHTS | 0xFF) == 0
