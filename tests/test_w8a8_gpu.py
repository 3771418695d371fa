"""W8A8 linear (row quantiser + int8 tensor-core GEMM) against the reference's vectors and the oracle.

The integer sums are exact and the scaling follows the reference's operation order, so the
bar is bit equality of the fp16 / bf16 outputs, not a tolerance.  The reference's own test
(tests/kernels/test_w8a8_linear.py:11-27) is repeated with its tolerance as well.
"""

from __future__ import annotations

import os

import numpy as np
import pytest
import torch

from full_inference_engine_b200 import _lib
from full_inference_engine_b200.kernels import w8a8_linear as w8a8
from full_inference_engine_b200.kernels.w8a16_linear import quantize_weight_per_channel
from oracle import wq_oracle as oracle
from tests.helpers import bits_equal, to_np

pytestmark = pytest.mark.gpu

VECTORS = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_w8a8.npz"))
CASES = sorted({key.split(".")[0] for key in VECTORS.files})


def _case(name):
    bf16 = bool(VECTORS[f"{name}.meta"][4])
    dtype = torch.bfloat16 if bf16 else torch.float16
    x = torch.from_numpy(VECTORS[f"{name}.x"]).to(dtype).cuda()
    qweight = torch.from_numpy(VECTORS[f"{name}.qweight"]).cuda()
    scales = torch.from_numpy(VECTORS[f"{name}.scales"]).cuda()
    return x, qweight, scales, VECTORS[f"{name}.y"]


def _rows_where_both_division_rules_agree(x: torch.Tensor) -> np.ndarray:
    """The golden vectors were produced on CPU tensors, where torch divides by 127; on CUDA
    tensors (and in the kernel) it multiplies by the fp32 reciprocal.  Rows whose scale comes
    out the same either way must match the vectors bit for bit."""
    cpu_rule = oracle.quantize_rows_int8(to_np(x), "cpu")[1]
    cuda_rule = oracle.quantize_rows_int8(to_np(x), "cuda")[1]
    return cpu_rule.view(np.uint32) == cuda_rule.view(np.uint32)


@pytest.mark.parametrize("name", CASES)
def test_forward_reproduces_the_reference_outputs_bit_for_bit(name):
    x, qweight, scales, want = _case(name)
    before = _lib.launch_count()
    got = w8a8.w8a8_linear(x, w8a8.pack_w8a8_weight(qweight), scales)
    assert _lib.launch_count() - before == 2            # the row quantiser and the GEMM
    assert got.dtype is x.dtype and got.shape == want.shape
    got32 = to_np(got).astype(np.float32)
    same = _rows_where_both_division_rules_agree(x)
    assert same.any() or len(same) == 1
    assert np.array_equal(got32[same], want.astype(np.float32)[same])
    # every row against the oracle in the reference device's arithmetic
    full = oracle.w8a8_linear(to_np(x), to_np(qweight), to_np(scales), bf16=x.dtype is torch.bfloat16)
    assert np.array_equal(got32, full.astype(np.float32))


@pytest.mark.parametrize("name", ["ragged_rows", "bf16"])
def test_operand_packed_the_reference_way_gives_the_same_result(name):
    """A contiguous [K, N] copy (what the reference's pack_w8a8_weight returns) is accepted too."""
    x, qweight, scales, want = _case(name)
    got = w8a8.w8a8_linear(x, qweight.t().contiguous(), scales)
    assert torch.equal(got, w8a8.w8a8_linear(x, w8a8.pack_w8a8_weight(qweight), scales))
    same = _rows_where_both_division_rules_agree(x)
    assert np.array_equal(to_np(got).astype(np.float32)[same], want.astype(np.float32)[same])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(1, 128), (33, 1000), (7, 4096), (300, 77)])
def test_row_quantiser_is_bit_exact(dtype, shape):
    torch.manual_seed(shape[0] * 131 + shape[1])
    x = (torch.randn(shape) * 2.5).to(dtype)
    x[0, : shape[1] // 2] = 0
    if shape[0] > 4:
        x[4] = 0
    q, scales = w8a8.quantize_activations_per_row(x.cuda())
    want_q, want_scales = oracle.quantize_rows_int8(to_np(x))
    assert q.dtype is torch.int8 and scales.dtype is torch.float32
    assert bits_equal(scales, want_scales)
    assert np.array_equal(q.cpu().numpy(), want_q)
    # and against the very expressions the reference evaluates on its device
    # (engine/kernels/w8a8_linear.py:43-44), which is where tensor / scalar becomes a multiply
    on_device = x.cuda()
    torch_scales = on_device.float().abs().amax(dim=1, keepdim=True).clamp_min(1e-8) / 127.0
    torch_q = torch.round(on_device.float() / torch_scales).clamp(-127, 127).to(torch.int8)
    assert torch.equal(scales.view(torch.int32), torch_scales[:, 0].contiguous().view(torch.int32))
    assert torch.equal(q, torch_q)


def test_the_references_own_test():
    """tests/kernels/test_w8a8_linear.py:11-27: same seed, shapes, construction and tolerance."""
    torch.manual_seed(91)
    inputs = torch.randn((16, 1024), device="cuda", dtype=torch.float16)
    weight = torch.randn((1024, 1024), device="cuda", dtype=torch.float16)
    qweight, weight_scales = quantize_weight_per_channel(weight)
    actual = w8a8.w8a8_linear(inputs, w8a8.pack_w8a8_weight(qweight), weight_scales)
    activation_scales = inputs.float().abs().amax(dim=1, keepdim=True).clamp_min(1e-8) / 127.0
    quantized_inputs = torch.round(inputs.float() / activation_scales).clamp(-127, 127)
    reference = (quantized_inputs.float() @ qweight.t().float()) * activation_scales * weight_scales.float()[None, :]
    assert actual.dtype is inputs.dtype
    torch.testing.assert_close(actual.float(), reference, rtol=4e-3, atol=4e-3)
    # stronger than the reference's tolerance: the same expressions rounded once are the output
    assert torch.equal(actual, reference.to(inputs.dtype))


@pytest.mark.parametrize("shape", [(16, 144, 40), (257, 272, 130), (512, 2048, 384), (100, 16, 8)])
def test_ragged_geometries_against_the_oracle(shape):
    """K that is not a multiple of the 128-byte block, N that is not a multiple of the tile,
    token counts that split into uneven tiles."""
    m, k, n = shape
    rng = np.random.default_rng(m + k + n)
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float16))
    qweight = torch.from_numpy(rng.integers(-127, 128, size=(n, k), dtype=np.int8))
    scales = torch.from_numpy((rng.random(n) * 0.02 + 0.001).astype(np.float16))
    got = w8a8.w8a8_linear(x.cuda(), w8a8.pack_w8a8_weight(qweight.cuda()), scales.cuda())
    want = oracle.w8a8_linear(x.numpy(), qweight.numpy(), scales.numpy())
    assert bits_equal(got, want)


def test_saturated_operands_do_not_overflow_the_accumulator():
    """Every product at its extreme, K = 8192: |sum| = 127 * 127 * 8192 < 2**31, and the int32 ->
    fp32 conversion rounds (the sum is beyond 2**24)."""
    m, k, n = 16, 8192, 128
    x = torch.ones((m, k), dtype=torch.float16)
    x[1::2] = -1
    qweight = torch.full((n, k), 127, dtype=torch.int8)
    qweight[::3] = -127
    scales = torch.full((n,), 0.0001, dtype=torch.float32)
    got = w8a8.w8a8_linear(x.cuda(), w8a8.pack_w8a8_weight(qweight.cuda()), scales.cuda())
    want = oracle.w8a8_linear(x.numpy(), qweight.numpy(), scales.numpy())
    assert bits_equal(got, want)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_prefill_size_sampled_against_the_oracle(dtype):
    """Qwen2.5-3B gate/up at 4096 tokens: M 4096, K 2048, N 22016.  The oracle checks 64 whole
    rows and 256 whole columns (strided through every tile)."""
    m, k, n = 4096, 2048, 22016
    gen = torch.Generator(device="cuda").manual_seed(17)
    x = torch.randn((m, k), device="cuda", dtype=dtype, generator=gen)
    qweight = torch.randint(-127, 128, (n, k), device="cuda", dtype=torch.int8, generator=gen)
    scales = (torch.rand((n,), device="cuda", generator=gen) * 0.01 + 0.001).half()
    got = w8a8.w8a8_linear(x, w8a8.pack_w8a8_weight(qweight), scales)
    bf16 = dtype is torch.bfloat16
    rows = torch.arange(7, m, 64, device="cuda")
    want_rows = oracle.w8a8_linear(to_np(x[rows]), qweight.cpu().numpy(), scales.cpu().numpy(), bf16=bf16)
    assert np.array_equal(to_np(got[rows]).astype(np.float32), want_rows.astype(np.float32))
    cols = torch.arange(3, n, 86, device="cuda")
    want_cols = oracle.w8a8_linear(to_np(x), qweight[cols].cpu().numpy(), scales[cols].cpu().numpy(), bf16=bf16)
    assert np.array_equal(to_np(got[:, cols]).astype(np.float32), want_cols.astype(np.float32))


def test_one_quantised_input_feeds_several_projections():
    torch.manual_seed(3)
    x = torch.randn((24, 512), device="cuda", dtype=torch.float16)
    q, a_scales = w8a8.quantize_activations_per_row(x)
    for n in (64, 200):
        qweight = torch.randint(-127, 128, (n, 512), device="cuda", dtype=torch.int8)
        scales = torch.rand((n,), device="cuda").half() * 0.01
        packed = w8a8.pack_w8a8_weight(qweight)
        once = w8a8.w8a8_linear_prequantized(q, a_scales, packed, scales, torch.float16)
        assert torch.equal(once, w8a8.w8a8_linear(x, packed, scales))


def test_forward_is_capturable_in_a_cuda_graph():
    torch.manual_seed(4)
    x = torch.randn((32, 1024), device="cuda", dtype=torch.float16)
    qweight = torch.randint(-127, 128, (256, 1024), device="cuda", dtype=torch.int8)
    scales = torch.rand((256,), device="cuda").half() * 0.01
    packed = w8a8.pack_w8a8_weight(qweight)
    eager = w8a8.w8a8_linear(x, packed, scales)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        w8a8.w8a8_linear(x, packed, scales)                       # tensor maps and attributes are set up
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            captured = w8a8.w8a8_linear(x, packed, scales)
    torch.cuda.current_stream().wait_stream(stream)
    x.copy_(torch.randn_like(x))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured, w8a8.w8a8_linear(x, packed, scales))
    assert not torch.equal(captured, eager)
