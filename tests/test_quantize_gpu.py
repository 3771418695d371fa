"""Quantize / pack / dequantize kernels against the oracle and the reference's golden vectors.

Integer and byte outputs must be bit-exact (``np.array_equal``); the test matrix follows the
reference's own (tests/kernels/test_w4a16_linear.py:18-118, engine/kernels/w8a16_linear.py:43-47).
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from full_inference_engine_b200.kernels import w4a16_format as w4
from full_inference_engine_b200.kernels import w4a16_linear, w8a16_linear
from oracle import wq_oracle as oracle
from tests.helpers import bits_equal, to_np

pytestmark = pytest.mark.gpu

W4_GOLDEN = ["w4_f32_s0", "w4_f16_s3", "w4_f16_g32", "w4_f32_g64", "w4_bf16_s9",
             "w4_exact_multiples", "w4_halfstep", "w4_degenerate"]


def _weight_from_golden(golden, name):
    w = torch.from_numpy(golden[f"{name}.weight"])
    return w.to(torch.bfloat16) if "bf16" in name else w


@pytest.mark.parametrize("name", W4_GOLDEN)
def test_w4_quantize_matches_the_reference_vectors(golden, name):
    _, n, k, g = (int(v) for v in golden[f"{name}.meta"])
    packed, scales = w4.quantize_weight_w4_grouped(_weight_from_golden(golden, name).cuda(), g)
    assert packed.dtype is torch.uint8 and packed.shape == (n, k // 2)
    assert scales.dtype is torch.float16 and scales.shape == (n, k // g)
    assert bits_equal(packed, golden[f"{name}.packed"])
    assert bits_equal(scales, golden[f"{name}.scales"])
    out = torch.full((n, k), float("nan"), device="cuda", dtype=torch.float16)
    w4a16_linear.w4_dequantize_into(out, packed, scales, group_size=g)
    assert bits_equal(out, golden[f"{name}.dequant"])


@pytest.mark.parametrize("shape", [(6, 512), (8, 1024), (3072, 1024), (12288, 4096), (4096, 12288)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_w4_quantize_is_bit_exact_against_the_oracle(shape, dtype):
    for seed in ((0, 3, 11) if shape[0] * shape[1] < 1 << 22 else (0,)):
        torch.manual_seed(seed)
        weight = (torch.randn(*shape) * (0.02 if seed == 0 else 1.0)).to(dtype)
        packed, scales = w4.quantize_weight_w4_grouped(weight.cuda())
        ref_packed, ref_scales = oracle.quantize_w4_grouped(to_np(weight))
        assert bits_equal(packed, ref_packed)
        assert bits_equal(scales, ref_scales)


def test_w4_split_half_layout_known_answer():
    weight = torch.zeros(1, 256)
    weight[0, 5], weight[0, 5 + 64], weight[0, 0] = 7.0, -7.0, 7.0
    packed, scales = w4.quantize_weight_w4_grouped(weight.cuda(), 128)
    assert float(scales[0, 0]) == pytest.approx(1.0)
    byte = int(packed[0, 5])
    assert byte & 0x0F == 15 and byte >> 4 == 1
    assert int(packed[0, 64]) == 0x88


def test_w4_strided_and_bf16_inputs():
    torch.manual_seed(5)
    big = torch.randn(64, 1024, device="cuda")
    view = big[:, 256:768]                                   # row pitch 1024, width 512
    packed, scales = w4.quantize_weight_w4_grouped(view)
    ref_packed, ref_scales = oracle.quantize_w4_grouped(to_np(view))
    assert bits_equal(packed, ref_packed) and bits_equal(scales, ref_scales)
    wb = (torch.randn(32, 256) * 0.02).to(torch.bfloat16)
    packed, scales = w4.quantize_weight_w4_grouped(wb.cuda())
    ref_packed, ref_scales = oracle.quantize_w4_grouped(to_np(wb))
    assert bits_equal(packed, ref_packed) and bits_equal(scales, ref_scales)


@pytest.mark.parametrize("shape", [(1024, 1024), (3072, 1024), (12288, 4096), (1000, 256)])
def test_w4_dequantize_into_is_bit_identical_to_the_reference_contract(shape):
    torch.manual_seed(3)
    n, k = shape
    weight = torch.randn(n, k, dtype=torch.float16)
    packed, scales = w4.quantize_weight_w4_grouped(weight.cuda())
    out = torch.full((n, k), float("nan"), device="cuda", dtype=torch.float16)
    assert w4a16_linear.w4_dequantize_into(out, packed, scales) is out
    assert bits_equal(out, oracle.unpack_w4(to_np(packed), to_np(scales), k))
    # and the torch reference dequantiser (reference_mode's arithmetic) agrees on the GPU
    assert torch.equal(out, w4.unpack_w4_reference(packed, scales, k))


def test_w4_dequantize_small_groups_and_pitched_output():
    torch.manual_seed(8)
    weight = torch.randn(16, 96)
    for g in (2, 6, 32, 48):
        packed, scales = w4.quantize_weight_w4_grouped(weight.cuda(), g)
        ref_packed, ref_scales = oracle.quantize_w4_grouped(to_np(weight), g)
        assert bits_equal(packed, ref_packed) and bits_equal(scales, ref_scales)
        big = torch.full((16, 128), float("nan"), device="cuda", dtype=torch.float16)
        w4a16_linear.w4_dequantize_into(big[:, :96], packed, scales, group_size=g)
        assert bits_equal(big[:, :96], oracle.unpack_w4(ref_packed, ref_scales, 96, g))
        assert torch.isnan(big[:, 96:]).all()


@pytest.mark.parametrize("name", ["w8_f32_s0", "w8_f16_s1", "w8_bf16_s2", "w8_degenerate"])
def test_w8_quantize_matches_the_reference_vectors(golden, name):
    w = torch.from_numpy(golden[f"{name}.weight"])
    if "bf16" in name:
        w = w.to(torch.bfloat16)
    q, s = w8a16_linear.quantize_weight_per_channel(w.cuda())
    assert q.dtype is torch.int8 and s.dtype is torch.float16
    assert bits_equal(q, golden[f"{name}.q"])
    assert bits_equal(s, golden[f"{name}.scales"])
    if f"{name}.int8linear_q" in golden:
        q, s = w8a16_linear.quantize_weight_per_channel_fp32_scales(w.cuda())
        assert bits_equal(q, golden[f"{name}.int8linear_q"])
        assert bits_equal(s, golden[f"{name}.int8linear_scales"])


@pytest.mark.parametrize("shape,scale,dtype", [
    ((3072, 1024), 0.02, torch.float32),        # config 1
    ((896, 896), 1.0, torch.float16), ((4864, 896), 1.0, torch.float16),
    ((12288, 4096), 0.02, torch.float32),
])
def test_w8_quantize_is_bit_exact_against_the_oracle(shape, scale, dtype):
    torch.manual_seed(0)
    weight = (torch.randn(*shape) * scale).to(dtype)
    q, s = w8a16_linear.quantize_weight_per_channel(weight.cuda())
    rq, rs = oracle.quantize_w8_per_channel(to_np(weight))
    assert bits_equal(q, rq) and bits_equal(s, rs)
    q, s = w8a16_linear.quantize_weight_per_channel_fp32_scales(weight.cuda())
    rq, rs = oracle.quantize_w8_int8linear(to_np(weight))
    assert bits_equal(q, rq) and bits_equal(s, rs)


@pytest.mark.parametrize("shape", [(8, 256), (3072, 1024), (4096, 12288)])
def test_asym_quantize_and_dequantize_match_the_oracle(shape):
    torch.manual_seed(0)
    weight = torch.randn(*shape) * 0.02 + 0.003
    packed, scales, zeros = w4.quantize_weight_w4_asym(weight.cuda())
    rp, rs, rz = oracle.quantize_w4_asym(to_np(weight))
    assert packed.dtype is torch.int32
    assert bits_equal(packed, rp) and bits_equal(scales, rs) and bits_equal(zeros, rz)
    n, k = shape
    out = torch.full((n, k), float("nan"), device="cuda", dtype=torch.float16)
    w4a16_linear.w4_dequantize_into(out, packed, scales, zeros=zeros)
    assert bits_equal(out, oracle.unpack_w4_asym(rp, rs, rz, k))
    assert torch.equal(out, w4.unpack_w4_asym_reference(packed, scales, zeros, k))


def test_shard_then_quantize_equals_quantize_then_shard():
    """Row-wise statistics: an N-shard quantises to the matching slice (any rank count)."""
    torch.manual_seed(1)
    weight = (torch.randn(1024, 512) * 0.02).cuda()
    packed, scales = w4.quantize_weight_w4_grouped(weight)
    q8, s8 = w8a16_linear.quantize_weight_per_channel(weight)
    for parts in (2, 4, 8):
        rows = 1024 // parts
        for r in range(parts):
            p, s = w4.quantize_weight_w4_grouped(weight[r * rows:(r + 1) * rows])
            assert torch.equal(p, packed[r * rows:(r + 1) * rows])
            assert torch.equal(s, scales[r * rows:(r + 1) * rows])
            q, s = w8a16_linear.quantize_weight_per_channel(weight[r * rows:(r + 1) * rows])
            assert torch.equal(q, q8[r * rows:(r + 1) * rows]) and torch.equal(s, s8[r * rows:(r + 1) * rows])
