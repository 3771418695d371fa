"""Host-side contract of the W8A8 mirror: the reference's argument checks and messages
(engine/kernels/w8a8_linear.py:13-17, 37-44), without a GPU."""

from __future__ import annotations

import pytest
import torch

from full_inference_engine_b200.kernels import w8a8_linear as w8a8


def test_pack_returns_the_references_shape_without_copying():
    qweight = torch.randint(-127, 128, (6, 32), dtype=torch.int8)
    packed = w8a8.pack_w8a8_weight(qweight)
    assert packed.shape == (32, 6) and packed.dtype is torch.int8
    assert packed.data_ptr() == qweight.data_ptr()
    assert torch.equal(packed, qweight.t())


@pytest.mark.parametrize("bad", [torch.zeros(4, dtype=torch.int8), torch.zeros((2, 2), dtype=torch.int32)])
def test_pack_rejects_what_the_reference_rejects(bad):
    with pytest.raises(ValueError, match="qweight must be a 2D INT8 tensor"):
        w8a8.pack_w8a8_weight(bad)


def test_forward_argument_checks_follow_the_reference():
    x = torch.zeros((2, 32), dtype=torch.float16)
    packed = torch.zeros((32, 8), dtype=torch.int8)
    scales = torch.ones(8, dtype=torch.float16)
    with pytest.raises(ValueError, match="inputs must be 2D and packed_weight must be 2D INT8"):
        w8a8.w8a8_linear(x[0], packed, scales)
    with pytest.raises(ValueError, match="inputs must be 2D and packed_weight must be 2D INT8"):
        w8a8.w8a8_linear(x, packed.int(), scales)
    with pytest.raises(ValueError, match="invalid W8A8 geometry"):
        w8a8.w8a8_linear(x, packed[:16], scales)
    with pytest.raises(ValueError, match="invalid W8A8 geometry"):
        w8a8.w8a8_linear(x, packed, scales[:4])
    with pytest.raises(ValueError, match="all W8A8 tensors must be on the same CUDA device"):
        w8a8.w8a8_linear(x, packed, scales)            # CPU tensors: no silent CPU fallback
