"""Forward kernels (CUDA-core GEMV and tcgen05 GEMM) against the oracle's fp32 ground truth.

Two bars are checked on every case: the acceptance bar ``max|err| <= 1e-2 * max|ref|`` and
the reference tests' own element-wise tolerances (5e-3 for the INT4 GEMM, rtol 2e-3 / atol
2e-2 for the GEMV, 3e-3 for W8: tests/kernels/test_w4a16_linear.py:73-157,
tests/kernels/test_w8a16_linear.py:13-27), the latter widened only by the half-ulp of the
fp16/bf16 output rounding, which the reference's fp16 comparison target also carries.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from full_inference_engine_b200 import _lib
from full_inference_engine_b200.kernels import w4a16_format as w4
from full_inference_engine_b200.kernels import w4a16_linear, w8a16_linear
from oracle import wq_oracle as oracle
from tests.helpers import assert_close, assert_within_bar, seeded_case, to_np

pytestmark = pytest.mark.gpu

KERNELS = ["auto", "gemv", "dot"]


def _status_ok():
    ws = _lib.workspace_for(torch.device("cuda", torch.cuda.current_device()), 256)
    assert _lib.library().b200q_workspace_status(ws.data_ptr(), None) == _lib.OK


def _out_rounding(dtype):
    return 2.0 ** -11 if dtype is torch.float16 else 2.0 ** -8


def _w4_truth(x, packed, scales, bias, k, g=128):
    return oracle.linear_fp32(to_np(x), oracle.unpack_w4(to_np(packed), to_np(scales), k, g),
                              None if bias is None else to_np(bias))


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("shape", [(16, 1024, 1024), (16, 1024, 3072), (1, 1024, 1024), (5, 2048, 896)])
def test_w4a16_linear_matches_the_dequantised_reference(shape, kernel):
    x, weight, bias = seeded_case(shape)
    packed, scales = w4.quantize_weight_w4_grouped(weight.half().cuda())
    y = w4a16_linear.w4a16_linear(x.cuda(), packed, scales, bias.cuda(), kernel=kernel)
    assert y.shape == (shape[0], shape[2]) and y.dtype is torch.float16
    truth = _w4_truth(x, packed, scales, bias, shape[1])
    assert_within_bar(y, truth)
    assert_close(y, truth, rtol=5e-3 + _out_rounding(torch.float16), atol=5e-3)
    _status_ok()


@pytest.mark.parametrize("kernel", KERNELS)
def test_w4a16_linear_without_bias_and_with_ragged_m_and_n(kernel):
    torch.manual_seed(2)
    x = torch.randn(13, 512).half()
    weight = torch.randn(200, 512).half()
    packed, scales = w4.quantize_weight_w4_grouped(weight.cuda())
    y = w4a16_linear.w4a16_linear(x.cuda(), packed, scales, kernel=kernel)
    truth = _w4_truth(x, packed, scales, None, 512)
    assert_within_bar(y, truth)
    assert_close(y, truth, rtol=5e-3 + 2.0 ** -11, atol=5e-3)
    _status_ok()


@pytest.mark.parametrize("m", [1, 2, 3])
def test_w4a16_gemv_matches_the_dequantised_reference(m):
    torch.manual_seed(m)
    k, n = 1024, 1000
    packed, scales = w4.quantize_weight_w4_grouped(torch.randn(n, k).half().cuda())
    bias = torch.randn(n).half()
    x = torch.randn(m, k).half()
    truth = _w4_truth(x, packed, scales, bias, k)
    for block_n, block_k in [(4, 1024), (8, 1024), (16, 512), (4, 128)]:
        out = w4a16_linear.w4a16_gemv(x.cuda(), packed, scales, bias.cuda(),
                                      block_n=block_n, block_k=block_k)
        assert_close(out, truth, rtol=2e-3, atol=2e-2)
    auto = w4a16_linear.w4a16_linear(x.cuda(), packed, scales, bias.cuda())
    assert_close(auto, truth, rtol=2e-3, atol=2e-2)
    with pytest.raises(ValueError):
        w4a16_linear.w4a16_gemv(torch.zeros(4, k, device="cuda", dtype=torch.float16), packed, scales)


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("shape", [(16, 896, 896), (16, 896, 4864), (1, 896, 896), (8, 1024, 3072)])
def test_w8a16_linear_matches_the_dequantised_reference(shape, kernel):
    config1 = shape == (8, 1024, 3072)          # seed 0, weights ~N(0, 0.02), no bias
    x, weight, bias = seeded_case(shape, seed=0 if config1 else None,
                                  weight_scale=0.02 if config1 else 1.0, bias=not config1)
    q, s = w8a16_linear.quantize_weight_per_channel((weight if config1 else weight.half()).cuda())
    y = w8a16_linear.w8a16_linear(x.cuda(), q, s, None if bias is None else bias.cuda(), kernel=kernel)
    truth = oracle.linear_fp32(to_np(x), oracle.dequant_w8(to_np(q), to_np(s)),
                               None if bias is None else to_np(bias))
    assert_within_bar(y, truth)
    assert_close(y, truth, rtol=3e-3 + 2.0 ** -11, atol=3e-3)
    _status_ok()


@pytest.mark.parametrize("kernel", KERNELS)
def test_int8linear_fp32_scales_and_bf16_activations(kernel):
    torch.manual_seed(4)
    x = torch.randn(7, 512).to(torch.bfloat16)
    weight = torch.randn(300, 512) * 0.02
    q, s = w8a16_linear.quantize_weight_per_channel_fp32_scales(weight.cuda())
    assert s.dtype is torch.float32
    y = w8a16_linear.w8a16_linear(x.cuda(), q, s, kernel=kernel)
    assert y.dtype is torch.bfloat16
    truth = oracle.linear_fp32(to_np(x), oracle.dequant_w8(to_np(q), to_np(s)))
    assert_within_bar(y, truth)
    assert_close(y, truth, rtol=3e-3 + 2.0 ** -8, atol=3e-3)


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("m", [1, 3, 16, 40, 144, 300])
def test_w4a16_bf16_activations(m, kernel):
    torch.manual_seed(m)
    k, n = 1024, 640
    x = torch.randn(m, k).to(torch.bfloat16)
    packed, scales = w4.quantize_weight_w4_grouped((torch.randn(n, k) * 0.02).cuda())
    y = w4a16_linear.w4a16_linear(x.cuda(), packed, scales, kernel=kernel)
    assert y.dtype is torch.bfloat16
    assert_within_bar(y, _w4_truth(x, packed, scales, None, k))
    _status_ok()


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 4, 33])
def test_asym_layout_forward(m, dtype, kernel):
    torch.manual_seed(10 + m)
    k, n = 1024, 384
    x = torch.randn(m, k).to(dtype)
    weight = torch.randn(n, k) * 0.02 + 0.004
    packed, scales, zeros = w4.quantize_weight_w4_asym(weight.cuda())
    bias = torch.randn(n).to(dtype)
    y = w4a16_linear.w4a16_linear(x.cuda(), packed, scales, bias.cuda(), zeros=zeros, kernel=kernel)
    deq = oracle.unpack_w4_asym(to_np(packed), to_np(scales), to_np(zeros), k)
    assert_within_bar(y, oracle.linear_fp32(to_np(x), deq, to_np(bias)))
    _status_ok()


@pytest.mark.parametrize("g", [32, 64, 256])
def test_other_group_sizes_take_the_cuda_core_kernel(g):
    torch.manual_seed(g)
    k, n = 512, 96
    x = torch.randn(6, k).half()
    packed, scales = w4.quantize_weight_w4_grouped(torch.randn(n, k).cuda(), g)
    y = w4a16_linear.w4a16_linear(x.cuda(), packed, scales, group_size=g)
    assert_within_bar(y, _w4_truth(x, packed, scales, None, k, g))


@pytest.mark.parametrize("shape", [(4096, 12288), (12288, 4096)])
def test_config2_int4_m_sweep_at_qwen3_8b_mlp_shapes(shape):
    """benchmark configuration 2: INT4 g128, fp16 activations, M in {1,4,16,64,256}, both layouts."""
    k, n = shape
    torch.manual_seed(0)
    weight = (torch.randn(n, k) * 0.02).cuda()
    packed, scales = w4.quantize_weight_w4_grouped(weight)
    deq = oracle.unpack_w4(to_np(packed), to_np(scales), k)
    apacked, ascales, azeros = w4.quantize_weight_w4_asym(weight)
    adeq = oracle.unpack_w4_asym(to_np(apacked), to_np(ascales), to_np(azeros), k)
    for m in (1, 4, 16, 64, 256):
        x = torch.randn(m, k).half()
        y = w4a16_linear.w4a16_linear(x.cuda(), packed, scales)
        ratio = assert_within_bar(y, oracle.linear_fp32(to_np(x), deq))
        assert ratio < 2e-3, ratio        # well inside the bar: fp16 output rounding dominates
        again = w4a16_linear.w4a16_linear(x.cuda(), packed, scales)
        assert torch.equal(y, again), "split-K must be deterministic"
        ya = w4a16_linear.w4a16_linear(x.cuda(), apacked, ascales, zeros=azeros)
        assert_within_bar(ya, oracle.linear_fp32(to_np(x), adeq))
    _status_ok()


@pytest.mark.parametrize("shape", [(4096, 4096), (4096, 2048), (4096, 12288), (12288, 4096)])
def test_config4_w8_bf16_at_qwen3_8b_shapes(shape):
    """benchmark configuration 4 (one GPU's view): W8 per-channel, bf16 activations."""
    k, n = shape
    torch.manual_seed(0)
    q, s = w8a16_linear.quantize_weight_per_channel((torch.randn(n, k) * 0.02).cuda())
    deq = oracle.dequant_w8(to_np(q), to_np(s))
    for m in (1, 16, 64, 512):
        x = torch.randn(m, k).to(torch.bfloat16)
        y = w8a16_linear.w8a16_linear(x.cuda(), q, s)
        assert_within_bar(y, oracle.linear_fp32(to_np(x), deq))
    _status_ok()


@pytest.mark.parametrize("layout", ["ref", "asym"])
@pytest.mark.parametrize("shape", [(4096, 12288), (12288, 4096)])
def test_config5_prefill_with_outlier_rows(shape, layout):
    """benchmark configuration 5: M=4096 bf16, 1% of rows x20, in both INT4 layouts (the
    asymmetric one is what the benchmark times).  The oracle checks a sample of rows (all
    outlier rows among them); the whole output is checked against torch's fp32 matmul over the
    oracle-identical dequantised weights."""
    k, n = shape
    m = 4096
    torch.manual_seed(0)
    weight = (torch.randn(n, k) * 0.02).cuda()
    x = torch.randn(m, k)
    outliers = torch.randperm(m)[:41]
    x[outliers] *= 20.0
    x = x.to(torch.bfloat16)
    if layout == "ref":
        packed, scales = w4.quantize_weight_w4_grouped(weight)
        y = w4a16_linear.w4a16_linear(x.cuda(), packed, scales)
        deq_gpu = w4.unpack_w4_reference(packed, scales, k)
        deq = oracle.unpack_w4(to_np(packed), to_np(scales), k)
    else:
        packed, scales, zeros = w4.quantize_weight_w4_asym(weight)
        y = w4a16_linear.w4a16_linear(x.cuda(), packed, scales, zeros=zeros)
        deq_gpu = torch.empty(n, k, dtype=torch.float16, device="cuda")
        w4a16_linear.w4_dequantize_into(deq_gpu, packed, scales, zeros=zeros)
        deq = oracle.unpack_w4_asym(to_np(packed), to_np(scales), to_np(zeros), k)
    assert np.array_equal(to_np(deq_gpu).view(np.uint16), deq.view(np.uint16))
    full = x.cuda().float() @ deq_gpu.float().T
    bound = 1e-2 * float(full.abs().max())
    assert float((y.float() - full).abs().max()) <= bound
    rows = torch.cat([outliers, torch.arange(0, m, 97)])
    truth = oracle.linear_fp32(to_np(x[rows]), deq)
    err = np.abs(to_np(y[rows.cuda()]).astype(np.float32) - truth).max()
    assert err <= bound
    _status_ok()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [144, 300, 1000])
def test_asym_layout_wide_token_tiles(m, dtype):
    """The asymmetric layout through the wide-tile instantiations (token tiles above 64 rows,
    sixteen dequantise warps, cluster and workspace split-K), against the oracle."""
    k, n = 4096, 1536
    torch.manual_seed(m)
    packed, scales, zeros = w4.quantize_weight_w4_asym((torch.randn(n, k) * 0.02 + 0.003).cuda())
    deq = oracle.unpack_w4_asym(to_np(packed), to_np(scales), to_np(zeros), k)
    x = torch.randn(m, k).to(dtype)
    bias = torch.randn(n).to(dtype)
    y = w4a16_linear.w4a16_linear(x.cuda(), packed, scales, bias.cuda(), zeros=zeros)
    assert_within_bar(y, oracle.linear_fp32(to_np(x), deq, to_np(bias)))
    _status_ok()
