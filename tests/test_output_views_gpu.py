"""Outputs that are views of a larger buffer, through the C ABI: a leading dimension wider than
N, an aligned and an unaligned first column.  The tensor-core kernel writes finished tiles with
one TMA store when rows are 16-byte aligned and with per-thread stores otherwise; both must give
the same values as a dense output and leave every byte outside the view untouched."""

from __future__ import annotations

import pytest
import torch

from full_inference_engine_b200 import _lib
from full_inference_engine_b200.kernels import w4a16_format as w4, w8a16_linear

pytestmark = pytest.mark.gpu

# (M, K, N): direct epilogue with ragged tiles, split-K through the workspace, split-K in a cluster
SHAPES = [(300, 512, 1000), (5, 2048, 328), (200, 4096, 520)]


def _run_w4(x, packed, scales, y_ptr, ldy, m, n, k, flags=0):
    ws = _lib.workspace_for(x.device, _lib.workspace_bytes(4, m, n, k))
    _lib.check(_lib.library().b200q_w4a16_forward(
        x.data_ptr(), x.stride(0), _lib.dtype_enum(x.dtype), packed.data_ptr(), packed.stride(0),
        _lib.W4_REF_SPLIT_HALF_SYM, scales.data_ptr(), None, 128, None, y_ptr, ldy, m, n, k,
        ws.data_ptr(), ws.numel(), _lib.KERNEL_TC | flags, _lib.stream_ptr(x.device)), "b200q_w4a16_forward")


@pytest.mark.parametrize("m,k,n", SHAPES)
@pytest.mark.parametrize("first_column", [0, 8, 3])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_w4_output_view(m, k, n, first_column, dtype):
    torch.manual_seed(m + n + first_column)
    packed, scales = w4.quantize_weight_w4_grouped(torch.randn(n, k, device="cuda") * 0.05)
    x = torch.randn(m, k, device="cuda").to(dtype)
    dense = torch.empty(m, n, device="cuda", dtype=dtype)
    _run_w4(x, packed, scales, dense.data_ptr(), n, m, n, k)
    ld = n + 40                                   # a multiple of 8 for every N above: aligned rows
    sentinel = 1234.0
    wide = torch.full((m + 2, ld), sentinel, device="cuda", dtype=dtype)
    view = wide[1:m + 1, first_column:first_column + n]
    _run_w4(x, packed, scales, view.data_ptr(), ld, m, n, k)
    torch.cuda.synchronize()
    assert torch.equal(view, dense)
    mask = torch.ones_like(wide, dtype=torch.bool)
    mask[1:m + 1, first_column:first_column + n] = False
    assert bool((wide[mask] == sentinel).all()), "bytes outside the output view were written"


@pytest.mark.parametrize("m,k,n", SHAPES)
def test_w4_gated_pairs_output_view(m, k, n):
    n -= n % 2
    torch.manual_seed(m + n)
    packed, scales = w4.quantize_weight_w4_grouped(torch.randn(n, k, device="cuda") * 0.05)
    x = torch.randn(m, k, device="cuda").half()
    dense = torch.empty(m, n // 2, device="cuda", dtype=torch.float16)
    _run_w4(x, packed, scales, dense.data_ptr(), n // 2, m, n, k, _lib.FLAG_SWIGLU_PAIRS)
    for first_column in (0, 16, 5):
        ld = n // 2 + 48 - (n // 2) % 8           # aligned rows
        wide = torch.full((m + 1, ld), -7.0, device="cuda", dtype=torch.float16)
        view = wide[:m, first_column:first_column + n // 2]
        _run_w4(x, packed, scales, view.data_ptr(), ld, m, n, k, _lib.FLAG_SWIGLU_PAIRS)
        torch.cuda.synchronize()
        assert torch.equal(view, dense)
        mask = torch.ones_like(wide, dtype=torch.bool)
        mask[:m, first_column:first_column + n // 2] = False
        assert bool((wide[mask] == -7.0).all())


def test_w8_output_view_with_bias():
    m, k, n = 144, 1024, 776
    torch.manual_seed(1)
    q, s = w8a16_linear.quantize_weight_per_channel(torch.randn(n, k, device="cuda") * 0.05)
    bias = torch.randn(n, device="cuda").bfloat16()
    x = torch.randn(m, k, device="cuda").bfloat16()
    dense = w8a16_linear.w8a16_linear(x, q, s, bias, kernel="dot")
    wide = torch.full((m, n + 16), 3.0, device="cuda", dtype=torch.bfloat16)
    view = wide[:, 8:8 + n]
    ws = _lib.workspace_for(x.device, _lib.workspace_bytes(8, m, n, k))
    _lib.check(_lib.library().b200q_w8a16_forward(
        x.data_ptr(), x.stride(0), _lib.dtype_enum(x.dtype), q.data_ptr(), q.stride(0), s.data_ptr(),
        _lib.dtype_enum(s.dtype), bias.data_ptr(), view.data_ptr(), wide.stride(0), m, n, k,
        ws.data_ptr(), ws.numel(), _lib.KERNEL_TC, _lib.stream_ptr(x.device)), "b200q_w8a16_forward")
    torch.cuda.synchronize()
    assert torch.equal(view, dense)
    assert bool((wide[:, :8] == 3.0).all()) and bool((wide[:, 8 + n:] == 3.0).all())
