"""The shared-memory-operand variant of the tensor-core kernel (B200Q_TC_OPERAND=smem; the
default keeps the dequantised operand in tensor memory).  The switch is read once per process,
so the variant runs in a child process; it must meet the same bar against the oracle."""

from __future__ import annotations

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r"""
import sys
sys.path.insert(0, %r)
import numpy as np, torch
from full_inference_engine_b200 import _lib
from full_inference_engine_b200.kernels import w4a16_format as w4, w4a16_linear, w8a16_linear
from oracle import wq_oracle as oracle
torch.manual_seed(0)
k, n = 1024, 640
weight = torch.randn(n, k, device="cuda") * 0.02
packed, scales = w4.quantize_weight_w4_grouped(weight)
ap, asc, az = w4.quantize_weight_w4_asym(weight)
q, s = w8a16_linear.quantize_weight_per_channel(weight)
deq = oracle.unpack_w4(packed.cpu().numpy(), scales.cpu().numpy(), k)
adeq = oracle.unpack_w4_asym(ap.cpu().numpy(), asc.cpu().numpy(), az.cpu().numpy(), k)
qdeq = oracle.dequant_w8(q.cpu().numpy(), s.cpu().numpy())
for dtype in (torch.float16, torch.bfloat16):
    for m in (1, 5, 16, 48, 144, 300):
        x = torch.randn(m, k).to(dtype)
        xf = x.float().numpy()
        for name, y, truth in (
            ("ref", w4a16_linear.w4a16_linear(x.cuda(), packed, scales, kernel="dot"), oracle.linear_fp32(xf, deq)),
            ("asym", w4a16_linear.w4a16_linear(x.cuda(), ap, asc, zeros=az, kernel="dot"), oracle.linear_fp32(xf, adeq)),
            ("w8", w8a16_linear.w8a16_linear(x.cuda(), q, s, kernel="dot"), oracle.linear_fp32(xf, qdeq)),
        ):
            ok, ratio = oracle.within_tolerance(y.float().cpu().numpy(), truth)
            assert ok, (name, dtype, m, ratio)
ws = _lib.workspace_for(torch.device("cuda", 0), 256)
assert _lib.library().b200q_workspace_status(ws.data_ptr(), None) == _lib.OK
print("smem-operand variant ok")
""" % ROOT


def test_shared_memory_operand_variant_meets_the_bar():
    env = dict(os.environ, B200Q_TC_OPERAND="smem")
    done = subprocess.run([sys.executable, "-c", SCRIPT], env=env, capture_output=True, text=True,
                          timeout=300)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]
    assert "smem-operand variant ok" in done.stdout
