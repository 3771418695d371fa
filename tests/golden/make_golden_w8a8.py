"""Generates tests/golden/reference_w8a8.npz by running the REFERENCE's own W8A8 code on CPU.

    python tests/golden/make_golden_w8a8.py /path/to/full-inference-engine

``engine.kernels.w8a8_linear.w8a8_linear`` refuses tensors that are not on a CUDA device, but
every operation in it (including ``torch._int_mm``) also runs on CPU tensors.  This script
takes the function's source text from the reference tree AT GENERATION TIME, drops the two
lines of that device guard, and executes the rest unchanged in the reference module's own
namespace — so the stored outputs are the reference's arithmetic, not a restatement of it.
Weights come from the reference's ``quantize_weight_per_channel`` and ``pack_w8a8_weight``.
bf16 tensors are stored as float32 (exact).
"""

from __future__ import annotations

import inspect
import os
import sys
import textwrap

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name: (seed, rows, in_features, out_features, dtype, input spread)
CASES = {
    "ref_test": (91, 16, 1024, 1024, torch.float16, 1.0),     # tests/kernels/test_w8a8_linear.py:11-27
    "one_row": (92, 1, 256, 384, torch.float16, 1.0),
    "ragged_rows": (93, 33, 512, 200, torch.float16, 3.0),
    "bf16": (94, 48, 1024, 128, torch.bfloat16, 1.0),
    "long_k": (95, 4, 4096, 32,  torch.bfloat16, 0.05),       # sums beyond 2**24: int32 -> fp32 rounds
    "zero_row": (96, 5, 128, 64, torch.float16, 1.0),         # a row of zeros takes the 1e-8 floor
}


def _np(t: torch.Tensor) -> np.ndarray:
    return t.float().numpy() if t.dtype is torch.bfloat16 else t.detach().numpy()


def _cpu_callable(module):
    source = textwrap.dedent(inspect.getsource(module.w8a8_linear))
    lines = source.splitlines()
    guard = [i for i, line in enumerate(lines) if "device.type" in line]
    assert len(guard) == 1 and "raise ValueError" in lines[guard[0] + 1], "the device guard moved"
    del lines[guard[0]:guard[0] + 2]
    namespace = dict(vars(module))
    exec(compile("\n".join(lines), "<reference w8a8_linear without its device guard>", "exec"), namespace)
    return namespace["w8a8_linear"]


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from engine.kernels import w8a8_linear as ref
    from engine.kernels.w8a16_linear import quantize_weight_per_channel

    torch.set_num_threads(1)
    run = _cpu_callable(ref)
    out: dict[str, np.ndarray] = {}
    for name, (seed, m, k, n, dtype, spread) in CASES.items():
        torch.manual_seed(seed)
        x = (torch.randn(m, k) * spread).to(dtype)
        if name == "zero_row":
            x[2] = 0
        weight = torch.randn(n, k, dtype=torch.float16)
        qweight, scales = quantize_weight_per_channel(weight)
        y = run(x, ref.pack_w8a8_weight(qweight), scales)
        out[f"{name}.x"] = _np(x)
        out[f"{name}.qweight"] = _np(qweight)
        out[f"{name}.scales"] = _np(scales)
        out[f"{name}.y"] = _np(y)
        out[f"{name}.meta"] = np.array([seed, m, k, n, int(dtype is torch.bfloat16)], dtype=np.int64)
    path = os.path.join(HERE, "reference_w8a8.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main(sys.argv[1])
