"""Largest shapes of the reference's own benchmark table (benchmarks/kernels/w4a16_bench.py:20-29):
the 8B lm_head, K=4096 -> N=151936.  Bit-exact pack at full size against the oracle on a row
sample, forward against torch's fp32 matmul over the dequantised weights (whole output) and the
oracle (sampled columns)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from full_inference_engine_b200.kernels import w4a16_format as w4
from full_inference_engine_b200.kernels import w4a16_linear, w8a16_linear
from oracle import wq_oracle as oracle
from tests.helpers import to_np

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m", [1, 16, 160])
def test_lm_head_shape_int4(m):
    k, n = 4096, 151936
    torch.manual_seed(0)
    weight = torch.randn(n, k, device="cuda", dtype=torch.float16) * 0.02
    packed, scales = w4.quantize_weight_w4_grouped(weight)
    rows = torch.cat([torch.arange(0, 64), torch.arange(75000, 75064), torch.arange(n - 64, n)])
    ref_packed, ref_scales = oracle.quantize_w4_grouped(to_np(weight[rows.cuda()]))
    assert np.array_equal(to_np(packed[rows.cuda()]), ref_packed)
    assert np.array_equal(to_np(scales[rows.cuda()]).view(np.uint16), ref_scales.view(np.uint16))
    del weight
    x = torch.randn(m, k, device="cuda", dtype=torch.float16)
    y = w4a16_linear.w4a16_linear(x, packed, scales)
    assert y.shape == (m, n)
    deq = w4.unpack_w4_reference(packed, scales, k)
    full = x.float() @ deq.float().T
    bound = 1e-2 * float(full.abs().max())
    assert float((y.float() - full).abs().max()) <= bound
    truth = oracle.linear_fp32(to_np(x), oracle.unpack_w4(ref_packed, ref_scales, k))
    assert np.abs(to_np(y[:, rows.cuda()]).astype(np.float32) - truth).max() <= bound


def test_lm_head_shape_w8_and_odd_sizes():
    torch.manual_seed(1)
    k, n = 4096, 151936
    q, s = w8a16_linear.quantize_weight_per_channel(torch.randn(n, k, device="cuda", dtype=torch.float16))
    x = torch.randn(3, k, device="cuda", dtype=torch.bfloat16)
    y = w8a16_linear.w8a16_linear(x, q, s)
    full = x.float() @ (q.float() * s.float()[:, None]).T
    assert float((y.float() - full).abs().max()) <= 1e-2 * float(full.abs().max())
    # K that is a multiple of 32 but not of 64 (CUDA-core kernel), ragged N, every M regime
    for (m, kk, nn) in [(1, 96, 33), (7, 160, 129), (70, 1120, 200), (300, 2144, 77)]:
        qq, ss = w8a16_linear.quantize_weight_per_channel(torch.randn(nn, kk, device="cuda"))
        xx = torch.randn(m, kk, device="cuda", dtype=torch.float16)
        bb = torch.randn(nn, device="cuda", dtype=torch.float16)
        yy = w8a16_linear.w8a16_linear(xx, qq, ss, bb)
        truth = oracle.linear_fp32(to_np(xx), oracle.dequant_w8(to_np(qq), to_np(ss)), to_np(bb))
        err = np.abs(to_np(yy).astype(np.float32) - truth).max()
        assert err <= 1e-2 * np.abs(truth).max(), (m, kk, nn)
