"""The reference's CPU forward path, restated with the same torch CPU operators.

TEST / BASELINE INFRASTRUCTURE ONLY: ``bench.py`` times these on the host cores as the
``cpu_baseline`` and ``--impl reference`` legs; the product package never imports them.

The reference (Vaibhav7711/full-inference-engine) runs a quantized linear on CPU as
"dequantise the whole weight to the activation dtype, then ``F.linear``":

* W8A16 — ``Int8Linear.forward`` (engine/quantization/int8.py:30-33):
  ``W = qweight.to(x.dtype) * scales.to(x.dtype)[:, None]; F.linear(x, W, bias)``.
* INT4  — ``W4A16Linear.forward`` on a CPU tensor takes ``_dense`` (engine/quantization/
  w4a16.py:132-146, 158-178): ``unpack_w4_reference`` (engine/kernels/w4a16_format.py:53-69)
  then ``F.linear(rows, W.to(rows.dtype), bias)``, in N slabs of ``dense_slab_bytes`` when
  the fp16 tile exceeds 32 MiB.

Checked against the reference itself by ``tests/golden/make_golden.py`` (run where the
reference tree is present) and ``tests/test_oracle_golden.py``.
"""

from __future__ import annotations

import torch
from torch.nn import functional as F

OFFSET = 8
DENSE_SLAB_BYTES = 32 << 20      # engine/quantization/w4a16.py:151


def int8linear_forward(x: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor,
                       bias: torch.Tensor | None = None) -> torch.Tensor:
    """engine/quantization/int8.py:30-33."""
    weight = qweight.to(dtype=x.dtype) * scales.to(dtype=x.dtype)[:, None]
    b = bias.to(dtype=x.dtype) if bias is not None else None
    return F.linear(x, weight, b)


def unpack_w4(packed: torch.Tensor, scales: torch.Tensor, in_features: int,
              group_size: int = 128) -> torch.Tensor:
    """engine/kernels/w4a16_format.py:53-69 with torch CPU ops (fp16 product)."""
    n = packed.shape[0]
    groups, half = in_features // group_size, group_size // 2
    b = packed.reshape(n, groups, half)
    low = (b & 0x0F).to(torch.int8) - OFFSET
    high = (b >> 4).to(torch.int8) - OFFSET
    q = torch.cat((low, high), dim=-1).to(torch.float16)
    return (q * scales.to(torch.float16)[..., None]).reshape(n, in_features)


def w4a16_dense_forward(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor,
                        bias: torch.Tensor | None = None, group_size: int = 128) -> torch.Tensor:
    """engine/quantization/w4a16.py:158-178, the branches a CPU tensor can reach."""
    out_features, in_features = packed.shape[0], packed.shape[1] * 2
    rows = x.reshape(-1, in_features)
    b = None if bias is None else bias.to(rows.dtype)
    tile_bytes = 2 * out_features * in_features
    if tile_bytes <= DENSE_SLAB_BYTES:
        out = F.linear(rows, unpack_w4(packed, scales, in_features, group_size).to(rows.dtype), b)
    else:
        slab = max(1, DENSE_SLAB_BYTES // (2 * in_features))
        out = torch.empty(rows.shape[0], out_features, dtype=rows.dtype)
        for start in range(0, out_features, slab):
            stop = min(start + slab, out_features)
            weight = unpack_w4(packed[start:stop], scales[start:stop], in_features,
                               group_size).to(rows.dtype)
            out[:, start:stop] = F.linear(rows, weight, None if b is None else b[start:stop])
    return out.reshape(*x.shape[:-1], out_features)


def unpack_w4_asym(packed: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                   in_features: int, group_size: int = 128) -> torch.Tensor:
    """Dequantise the asymmetric int32 layout (no reference counterpart) to fp16."""
    n = packed.shape[0]
    # input i of a word sits at nibble position (i & 1) * 4 + (i >> 1)
    shifts = 4 * torch.tensor([(i & 1) * 4 + (i >> 1) for i in range(8)], dtype=torch.int32)
    nibbles = (packed.reshape(n, in_features // 8, 1) >> shifts) & 0xF
    q = nibbles.reshape(n, in_features // group_size, group_size).to(torch.float32)
    centred = (q - zeros.float()[..., None]).to(torch.float16)
    return (centred * scales.to(torch.float16)[..., None]).reshape(n, in_features)


def w4a16_asym_dense_forward(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor,
                             zeros: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """The same dequantise-then-``F.linear`` shape applied to the asymmetric layout."""
    out_features, in_features = packed.shape[0], packed.shape[1] * 8
    rows = x.reshape(-1, in_features)
    slab = max(1, DENSE_SLAB_BYTES // (2 * in_features))
    out = torch.empty(rows.shape[0], out_features, dtype=rows.dtype)
    for start in range(0, out_features, slab):
        stop = min(start + slab, out_features)
        weight = unpack_w4_asym(packed[start:stop], scales[start:stop], zeros[start:stop],
                                in_features, group_size).to(rows.dtype)
        out[:, start:stop] = F.linear(rows, weight)
    return out.reshape(*x.shape[:-1], out_features)


def gate_up_swiglu_forward(x: torch.Tensor, weights_pairs: torch.Tensor, scales_pairs: torch.Tensor,
                           *, int8: bool = False, group_size: int = 128) -> torch.Tensor:
    """The reference's unfused feed-forward front half on CPU over interleaved (gate, up) rows:
    two dequantise-then-``F.linear`` projections (engine/quantization/w4a16.py:158-178 or
    engine/quantization/int8.py:30-33) and ``silu(gate) * up`` evaluated in fp32 and stored in
    the activation dtype (engine/kernels/swiglu.py:22-26)."""
    halves = []
    for part in (0, 1):
        w, s = weights_pairs[part::2].contiguous(), scales_pairs[part::2].contiguous()
        halves.append(int8linear_forward(x, w, s) if int8 else w4a16_dense_forward(x, w, s, None, group_size))
    g = halves[0].float()
    return (g * torch.sigmoid(g) * halves[1].float()).to(x.dtype)
