"""The workspace-free INT4 entry point, through the C ABI.

``b200q_w4a16_forward_static_scratch`` serves hosts that cannot allocate device memory when
they call (an engine that has given all free HBM to its KV pool, a binding that only ever
receives input/output pointers): its split-K scratch is a fixed array inside the library.
This checks it against ``b200q_w4a16_forward`` on the same inputs and against the CPU oracle,
twice in a row (the array is shared and keeps the previous call's contents), that its partial
sums really went through the array inside the library (the caller-owned workspace of the other
entry point is a different buffer, and the geometries are chosen so that partials are needed),
that the fused argmax works on it after such a call, and that oversized problems are refused.
Collected last so that a failure here cannot mask another test.
"""

from __future__ import annotations

import pytest
import torch

import numpy as np

from full_inference_engine_b200 import _lib
from full_inference_engine_b200.kernels import w4a16_format as w4
from oracle import wq_oracle as oracle

pytestmark = pytest.mark.gpu


def _call(fn, x, packed, scales, y, m, n, k, *workspace, flags=0):
    return fn(x.data_ptr(), x.stride(0), _lib.dtype_enum(x.dtype),
              packed.data_ptr(), packed.stride(0), _lib.W4_REF_SPLIT_HALF_SYM,
              scales.data_ptr(), None, 128, None,
              y.data_ptr(), y.stride(0) if y.ndim == 2 else 0, m, n, k,
              *workspace, _lib.KERNEL_AUTO | flags, _lib.stream_ptr(x.device))


@pytest.mark.parametrize("m", [1, 5, 16, 64, 144])
def test_static_scratch_entry_point_matches_the_workspace_entry_point(m):
    lib = _lib.library()
    torch.manual_seed(m)
    # M <= 16: a shape the stream-K kernel takes (75 weight tiles shared among the blocks, partials
    # exchanged through the scratch); M = 64 / 144: the tile kernel with a K split too deep for a
    # cluster (fp32 partials parked in the scratch).
    k, n = (1024, 9600) if m <= 16 else (12288, 1024)
    plan = _lib.describe_plan(4, m, n, k)
    assert ("wq_gemm_sk_kernel" in plan) == (m <= 16), plan
    packed, scales = w4.quantize_weight_w4_grouped((torch.randn(n, k, device="cuda") * 0.02))
    deq = oracle.unpack_w4(packed.cpu().numpy(), scales.cpu().numpy(), k)
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
        truth = oracle.linear_fp32(x.float().cpu().numpy(), deq)
        ok, ratio = oracle.within_tolerance(actual.float().cpu().numpy(), truth)
        assert ok, f"call {call}: {ratio} of max|ref| against the oracle"
        # this geometry exchanges partial sums through the scratch: the tile kernel (M > 64) leaves
        # its fp32 partials behind, the decode kernel hands every exchange word back as zero
        if m > 16:
            assert bool(workspace[128 * 1024 + 5 * 1024 * 1024:].any()), "expected split-K partials"
        else:
            assert not bool(workspace[128 * 1024:].any()), "the exchange region was not left empty"
    # the head's fused argmax on the same array, after calls that left partials in it
    vocab, head_k = 3000, 1024
    hp, hs = w4.quantize_weight_w4_grouped(torch.randn(vocab, head_k, device="cuda") * 0.05)
    hx = torch.randn(m, head_k, device="cuda", dtype=torch.float16)
    logits = torch.empty(m, vocab, device="cuda", dtype=torch.float16)
    _lib.check(_call(lib.b200q_w4a16_forward_static_scratch, hx, hp, hs, logits, m, vocab, head_k),
               "static scratch logits")
    picked = torch.full((m,), -1, device="cuda", dtype=torch.int64)
    _lib.check(_call(lib.b200q_w4a16_forward_static_scratch, hx, hp, hs, picked, m, vocab, head_k,
                     flags=_lib.FLAG_ARGMAX), "static scratch argmax")
    assert torch.equal(picked, logits.argmax(dim=-1))


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
