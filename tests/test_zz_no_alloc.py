"""The workspace-free INT4 entry point, through the C ABI.

``b200q_w4a16_forward_static_scratch`` serves hosts that cannot allocate device memory when
they call (an engine that has given all free HBM to its KV pool, a binding that only ever
receives input/output pointers): its split-K scratch is a fixed array inside the library.
This checks it against ``b200q_w4a16_forward`` on the same inputs, twice in a row (the array
is shared and keeps the previous call's contents), and that oversized problems are refused.
Collected last so that a failure here cannot mask another test.
"""

from __future__ import annotations

import pytest
import torch

from full_inference_engine_b200 import _lib
from full_inference_engine_b200.kernels import w4a16_format as w4

pytestmark = pytest.mark.gpu


def _call(fn, x, packed, scales, y, m, n, k, *workspace):
    return fn(x.data_ptr(), x.stride(0), _lib.dtype_enum(x.dtype),
              packed.data_ptr(), packed.stride(0), _lib.W4_REF_SPLIT_HALF_SYM,
              scales.data_ptr(), None, 128, None,
              y.data_ptr(), y.stride(0), m, n, k,
              *workspace, _lib.KERNEL_AUTO, _lib.stream_ptr(x.device))


@pytest.mark.parametrize("m", [1, 5, 16, 64])
def test_static_scratch_entry_point_matches_the_workspace_entry_point(m):
    lib = _lib.library()
    torch.manual_seed(m)
    k, n = 4096, 4096                          # 32 N-tiles: the tensor-core path splits K
    packed, scales = w4.quantize_weight_w4_grouped((torch.randn(n, k, device="cuda") * 0.02))
    need = _lib.workspace_bytes(4, m, n, k)
    assert need <= lib.b200q_static_scratch_bytes()
    workspace = torch.zeros(need, dtype=torch.uint8, device="cuda")
    for call in range(2):                      # second call reuses whatever the first left behind
        x = torch.randn(m, k, device="cuda", dtype=torch.float16)
        expected = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float16)
        actual = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float16)
        _lib.check(_call(lib.b200q_w4a16_forward, x, packed, scales, expected, m, n, k,
                         workspace.data_ptr(), workspace.numel()), "b200q_w4a16_forward")
        held = torch.cuda.memory_allocated()
        _lib.check(_call(lib.b200q_w4a16_forward_static_scratch, x, packed, scales, actual, m, n, k),
                   "b200q_w4a16_forward_static_scratch")
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == held
        assert torch.isfinite(actual).all(), f"call {call}"
        err = float((actual.float() - expected.float()).abs().max())
        assert err <= 1e-2 * float(expected.float().abs().max()), f"call {call}: {err}"


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = _lib.library()
    m, k, n = 256, 12288, 6144                 # 48 tiles x 3 K-splits: 18.9 MB of fp32 partials
    assert _lib.workspace_bytes(4, m, n, k) > lib.b200q_static_scratch_bytes()
    packed = torch.zeros(n, k // 2, dtype=torch.uint8, device="cuda")
    scales = torch.ones(n, k // 128, dtype=torch.float16, device="cuda")
    x = torch.zeros(m, k, dtype=torch.float16, device="cuda")
    y = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    before = _lib.launch_count()
    status = _call(lib.b200q_w4a16_forward_static_scratch, x, packed, scales, y, m, n, k)
    assert status == _lib.ERR_WORKSPACE
    assert b"static scratch" in lib.b200q_last_error()
    assert _lib.launch_count() == before
