"""Generates tests/golden/*.npz by running the REFERENCE's own CPU code on seeded inputs.

Run it where the reference tree is available::

    python tests/golden/make_golden.py /path/to/full-inference-engine

It imports ``engine.kernels.w4a16_format``, ``engine.kernels.w8a16_linear``,
``engine.quantization.int8`` and ``engine.quantization.w4a16`` from that tree, feeds them
seeded tensors and stores inputs and outputs.  The fixtures pin ``oracle/`` (and through
it the CUDA kernels) to the reference without the reference having to be present when the
tests run.  bf16 tensors are stored as float32 (exact).
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _np(t: torch.Tensor) -> np.ndarray:
    if t.dtype is torch.bfloat16:
        return t.float().numpy()
    return t.detach().cpu().numpy()


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from engine.kernels import w4a16_format as w4
    from engine.kernels.w8a16_linear import quantize_weight_per_channel
    from engine.quantization.int8 import Int8Linear
    from engine.quantization.w4a16 import W4A16Linear

    torch.set_num_threads(1)
    out: dict[str, np.ndarray] = {}

    # ---- W4 quantize / pack / unpack (engine/kernels/w4a16_format.py)
    w4_cases = {
        # name: (seed, n, k, group, dtype, scale)
        "w4_f32_s0": (0, 24, 384, 128, torch.float32, 0.02),
        "w4_f16_s3": (3, 32, 256, 128, torch.float16, 1.0),
        "w4_f16_g32": (5, 16, 128, 32, torch.float16, 1.0),
        "w4_f32_g64": (7, 8, 256, 64, torch.float32, 0.5),
        "w4_bf16_s9": (9, 8, 256, 128, torch.bfloat16, 0.02),
    }
    for name, (seed, n, k, g, dtype, scale) in w4_cases.items():
        torch.manual_seed(seed)
        weight = (torch.randn(n, k) * scale).to(dtype)
        packed, scales = w4.quantize_weight_w4_grouped(weight, g)
        deq = w4.unpack_w4_reference(packed, scales, k, g)
        out[f"{name}.weight"] = _np(weight)
        out[f"{name}.packed"] = _np(packed)
        out[f"{name}.scales"] = _np(scales)
        out[f"{name}.dequant"] = _np(deq)
        out[f"{name}.meta"] = np.array([seed, n, k, g], dtype=np.int64)

    # the reference tests' own constructions (tests/kernels/test_w4a16_linear.py:18-56)
    torch.manual_seed(3)
    n, k, g = 6, 512, 128
    s = torch.rand(n, k // g) + 0.5
    q = torch.randint(-7, 8, (n, k // g, g)).float()
    weight = (q * s[..., None]).reshape(n, k)
    packed, scales = w4.quantize_weight_w4_grouped(weight, g)
    out["w4_exact_multiples.weight"] = _np(weight)
    out["w4_exact_multiples.packed"] = _np(packed)
    out["w4_exact_multiples.scales"] = _np(scales)
    out["w4_exact_multiples.dequant"] = _np(w4.unpack_w4_reference(packed, scales, k, g))
    out["w4_exact_multiples.meta"] = np.array([3, n, k, g], dtype=np.int64)

    torch.manual_seed(11)
    n, k, g = 8, 1024, 128
    weight = torch.randn(n, k) * torch.linspace(0.1, 4.0, n)[:, None]
    packed, scales = w4.quantize_weight_w4_grouped(weight, g)
    out["w4_halfstep.weight"] = _np(weight)
    out["w4_halfstep.packed"] = _np(packed)
    out["w4_halfstep.scales"] = _np(scales)
    out["w4_halfstep.dequant"] = _np(w4.unpack_w4_reference(packed, scales, k, g))
    out["w4_halfstep.meta"] = np.array([11, n, k, g], dtype=np.int64)

    # degenerate groups: all-zero and tiny
    weight = torch.zeros(3, 256)
    weight[1, 3] = 1e-9
    weight[2, 130] = -3.0
    weight[2, 131] = 0.21428572
    packed, scales = w4.quantize_weight_w4_grouped(weight, 128)
    out["w4_degenerate.weight"] = _np(weight)
    out["w4_degenerate.packed"] = _np(packed)
    out["w4_degenerate.scales"] = _np(scales)
    out["w4_degenerate.dequant"] = _np(w4.unpack_w4_reference(packed, scales, 256, 128))
    out["w4_degenerate.meta"] = np.array([0, 3, 256, 128], dtype=np.int64)

    # ---- W8 quantizers
    w8_cases = {
        "w8_f32_s0": (0, 48, 256, torch.float32, 0.02),     # config-1 style weights
        "w8_f16_s1": (1, 16, 896, torch.float16, 1.0),      # reference test style
        "w8_bf16_s2": (2, 16, 128, torch.bfloat16, 0.02),
    }
    for name, (seed, n, k, dtype, scale) in w8_cases.items():
        torch.manual_seed(seed)
        weight = (torch.randn(n, k) * scale).to(dtype)
        qw, sc = quantize_weight_per_channel(weight)
        out[f"{name}.weight"] = _np(weight)
        out[f"{name}.q"] = _np(qw)
        out[f"{name}.scales"] = _np(sc)
        lin = torch.nn.Linear(k, n, bias=False, dtype=dtype)
        with torch.no_grad():
            lin.weight.copy_(weight)
        mod = Int8Linear(lin)
        out[f"{name}.int8linear_q"] = _np(mod.qweight)
        out[f"{name}.int8linear_scales"] = _np(mod.scales)
    weight = torch.zeros(3, 32)
    weight[1, 3] = 1e-9
    weight[1, 4] = -2e-9
    weight[2, 7] = 5.0
    qw, sc = quantize_weight_per_channel(weight)
    out["w8_degenerate.weight"] = _np(weight)
    out["w8_degenerate.q"] = _np(qw)
    out["w8_degenerate.scales"] = _np(sc)

    # ---- forwards through the reference modules on CPU
    torch.manual_seed(0)
    lin = torch.nn.Linear(16, 8, bias=True, dtype=torch.float32)      # tests/quantization/test_int8.py:7-12
    mod = Int8Linear(lin)
    x = torch.randn(4, 16)
    out["int8linear_16x8.weight"] = _np(lin.weight)
    out["int8linear_16x8.bias"] = _np(lin.bias)
    out["int8linear_16x8.x"] = _np(x)
    out["int8linear_16x8.y"] = _np(mod(x))
    out["int8linear_16x8.y_fp32_linear"] = _np(lin(x))

    for tag, dtype in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        torch.manual_seed(21)
        weight = torch.randn(40, 256) * 0.02
        lin = torch.nn.Linear(256, 40, bias=True, dtype=torch.float32)
        with torch.no_grad():
            lin.weight.copy_(weight)
            lin.bias.copy_(torch.randn(40) * 0.1)
        mod = Int8Linear(lin)
        x = torch.randn(5, 256).to(dtype)
        out[f"int8linear_fwd_{tag}.weight"] = _np(weight)
        out[f"int8linear_fwd_{tag}.bias"] = _np(lin.bias)
        out[f"int8linear_fwd_{tag}.x"] = _np(x)
        out[f"int8linear_fwd_{tag}.y"] = _np(mod(x))

        torch.manual_seed(22)
        weight = (torch.randn(40, 256) * 0.02).to(torch.float16)
        layer = W4A16Linear(256, 40, bias=True)
        layer.quantize_from(weight)
        bias = (torch.randn(40) * 0.1).to(torch.float16)
        layer.set_bias(bias)
        x = torch.randn(5, 256).to(dtype)
        out[f"w4a16linear_fwd_{tag}.weight"] = _np(weight)
        out[f"w4a16linear_fwd_{tag}.bias"] = _np(bias)
        out[f"w4a16linear_fwd_{tag}.packed"] = _np(layer.packed)
        out[f"w4a16linear_fwd_{tag}.scales"] = _np(layer.scales)
        out[f"w4a16linear_fwd_{tag}.x"] = _np(x)
        out[f"w4a16linear_fwd_{tag}.y"] = _np(layer(x))

    out["weight_bytes_1024_3072"] = np.array(
        [w4.weight_bytes(1024, 3072)[key] for key in ("fp16", "w8a16", "w4a16")], dtype=np.int64)
    out["weight_bytes_4096_12288_g64"] = np.array(
        [w4.weight_bytes(4096, 12288, 64)[key] for key in ("fp16", "w8a16", "w4a16")], dtype=np.int64)

    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to the reference checkout>")
    main(sys.argv[1])
