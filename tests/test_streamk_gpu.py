"""The persistent stream-K kernel (token tiles of at most 64 rows) against the oracle.

Every format and activation dtype, ragged M and N, K of one to many groups, bias, gated pairs,
and repeated calls on the one shared workspace (tile counters must come back to zero).  The
shape sweep walks M over every residue of the 16-row token tile and N over residues of the
128-channel weight tile, at K of one to three groups and at K long enough that a tile's units
are spread over several blocks (partials through the workspace).
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from full_inference_engine_b200 import _lib
from full_inference_engine_b200.kernels import swiglu, w4a16_format as w4, w4a16_linear, w8a16_linear
from oracle import wq_oracle as oracle
from tests.helpers import assert_within_bar, to_np

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _status_ok():
    ws = _lib.workspace_for(torch.device("cuda", torch.cuda.current_device()), 256)
    assert _lib.library().b200q_workspace_status(ws.data_ptr(), None) == _lib.OK


def _quantized(fmt, weight):
    """(device tensors for the forward, dequantised fp32 weight of the oracle)."""
    k = weight.shape[1]
    if fmt == "ref":
        p, s = w4.quantize_weight_w4_grouped(weight)
        return (p, s, None), oracle.unpack_w4(to_np(p), to_np(s), k)
    if fmt == "asym":
        p, s, z = w4.quantize_weight_w4_asym(weight)
        return (p, s, z), oracle.unpack_w4_asym(to_np(p), to_np(s), to_np(z), k)
    q, s = w8a16_linear.quantize_weight_per_channel(weight)
    return (q, s), oracle.dequant_w8(to_np(q), to_np(s))


def _forward(fmt, x, qw, bias=None, **kw):
    if fmt == "w8":
        return w8a16_linear.w8a16_linear(x, qw[0], qw[1], bias, kernel="streamk", **kw)
    return w4a16_linear.w4a16_linear(x, qw[0], qw[1], bias, zeros=qw[2], kernel="streamk", **kw)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("fmt", ["ref", "asym", "w8"])
@pytest.mark.parametrize("shape", [(1, 4096, 4096), (16, 4096, 1536), (5, 12288, 1024), (48, 2048, 2176),
                                   (64, 4096, 4096), (33, 1024, 896), (8, 1024, 3072)])
def test_streamk_forward_matches_the_oracle(shape, fmt, dtype):
    m, k, n = shape
    torch.manual_seed(m + k + n)
    qw, deq = _quantized(fmt, torch.randn(n, k, device=DEV) * 0.02)
    bias = torch.randn(n, device=DEV).to(dtype)
    x = torch.randn(m, k, device=DEV).to(dtype)
    truth = oracle.linear_fp32(to_np(x).astype(np.float32), deq, to_np(bias).astype(np.float32))
    y = _forward(fmt, x, qw, bias)
    assert y.shape == (m, n) and y.dtype is dtype
    assert_within_bar(y, truth)
    # the call again, and with static weights: identical bits (fixed summation order, counters reset)
    assert torch.equal(y, _forward(fmt, x, qw, bias))
    assert torch.equal(y, _forward(fmt, x, qw, bias, static_weights=True))
    _status_ok()


@pytest.mark.parametrize("fmt", ["ref", "asym", "w8"])
def test_streamk_shape_sweep(fmt):
    """M over the residues of the token tile, N over residues of the weight tile, K of one to
    three groups and one long K; one quantised matrix per (N, K), sliced inputs per M."""
    rng = np.random.default_rng(7)
    worst = 0.0
    for k in (1024, 2048, 5120) if fmt != "w8" else (128, 256, 384, 5120):
        for n in (1, 8, 127, 128, 129, 200, 257, 1000):
            torch.manual_seed(n * 7 + k)
            qw, deq = _quantized(fmt, torch.randn(n, k, device=DEV) * 0.05)
            x_all = torch.randn(64, k, device=DEV).half()
            xf = to_np(x_all).astype(np.float32)
            for m in sorted({1, 2, 15, 16, 17, 31, 32, 47, 49, 64, int(rng.integers(1, 65))}):
                y = _forward(fmt, x_all[:m], qw)
                truth = oracle.linear_fp32(xf[:m], deq)
                ok, ratio = oracle.within_tolerance(to_np(y).astype(np.float32), truth)
                assert ok, (fmt, m, n, k, ratio)
                worst = max(worst, ratio)
    assert worst < 1e-2
    _status_ok()


@pytest.mark.parametrize("fmt", ["ref", "w8"])
@pytest.mark.parametrize("m", [1, 16, 40])
def test_streamk_gated_pairs(m, fmt):
    k, n = 4096, 1536                      # rows of each projection
    torch.manual_seed(m)
    gate_w = torch.randn(n, k, device=DEV) * 0.02
    up_w = torch.randn(n, k, device=DEV) * 0.02
    (gq, gdeq), (uq, udeq) = _quantized(fmt, gate_w), _quantized(fmt, up_w)
    pairs = tuple(None if a is None else swiglu.interleave_gate_up(a, b) for a, b in zip(gq, uq))
    x = torch.randn(m, k, device=DEV).half()
    xf = to_np(x).astype(np.float32)
    truth = oracle.swiglu_fp32(oracle.linear_fp32(xf, gdeq), oracle.linear_fp32(xf, udeq))
    y = _forward(fmt, x, pairs, swiglu_pairs=True)
    assert y.shape == (m, n)
    assert_within_bar(y, truth)
    _status_ok()


def test_streamk_strided_activations_and_outputs_in_place_of_a_view():
    m, k, n = 7, 1024, 640
    torch.manual_seed(0)
    qw, deq = _quantized("ref", torch.randn(n, k, device=DEV) * 0.02)
    wide = torch.randn(m, 2 * k, device=DEV).half()
    x = wide[:, k:]                        # row pitch 2K, 16-byte aligned
    y = _forward("ref", x, qw)
    assert_within_bar(y, oracle.linear_fp32(to_np(x).astype(np.float32), deq))
    _status_ok()
