"""Gate and up projections of a SwiGLU feed-forward in one quantized kernel.

The reference fuses the two fp16 projections into one matmul (``FusedGateUpProjection``,
engine/kernels/swiglu.py:65-83) and then runs ``silu(gate) * up`` as a second kernel
(``triton_swiglu``, engine/kernels/swiglu.py:43-62); its fusion needs an fp16 ``.weight`` and
cannot wrap a quantized module.  Here both steps are one launch over quantized weights: the
gate and up weight rows are interleaved (row ``2c`` = gate channel ``c``, row ``2c + 1`` = up
channel ``c``), one weight sweep feeds both accumulators of a pair, and the kernel's epilogue
writes ``silu(gate) * up`` directly, evaluated in fp32 and rounded once.

Row interleaving commutes with quantization: every statistic of both formats is taken along
a row, so quantizing the two matrices separately and interleaving the results gives the same
bytes as interleaving first.
"""

from __future__ import annotations

import torch

from . import w4a16_linear as _w4
from . import w8a16_linear as _w8
from .w4a16_format import GROUP_SIZE


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Rows ``gate[0], up[0], gate[1], up[1], ...`` of two equally shaped tensors (dim 0)."""
    if gate.shape != up.shape or gate.dtype != up.dtype or gate.device != up.device:
        raise ValueError("gate and up tensors must have matching shape, dtype, and device")
    if gate.ndim == 0:
        raise ValueError("gate and up must have a row dimension")
    return torch.stack((gate, up), dim=1).reshape(2 * gate.shape[0], *gate.shape[1:]).contiguous()


def w4a16_gate_up_swiglu(inputs: torch.Tensor, packed_pairs: torch.Tensor, scales_pairs: torch.Tensor,
                         bias_pairs: torch.Tensor | None = None, *, group_size: int = GROUP_SIZE,
                         zeros_pairs: torch.Tensor | None = None,
                         static_weights: bool = False) -> torch.Tensor:
    """``silu(x @ Wg.T) * (x @ Wu.T)`` over interleaved 4-bit weights: ``[M, K] -> [M, N]``.

    ``packed_pairs`` / ``scales_pairs`` (/ ``zeros_pairs`` / ``bias_pairs``) hold ``2 N`` rows
    built with ``interleave_gate_up``.  Tensor-core kernel only.
    """
    return _w4.w4a16_linear(inputs, packed_pairs, scales_pairs, bias_pairs, group_size=group_size,
                            kernel="auto", zeros=zeros_pairs, static_weights=static_weights,
                            swiglu_pairs=True)


def w8a16_gate_up_swiglu(inputs: torch.Tensor, qweight_pairs: torch.Tensor, scales_pairs: torch.Tensor,
                         bias_pairs: torch.Tensor | None = None, *,
                         static_weights: bool = False) -> torch.Tensor:
    """The same over interleaved per-channel int8 weights."""
    return _w8.w8a16_linear(inputs, qweight_pairs, scales_pairs, bias_pairs, kernel="auto",
                            static_weights=static_weights, swiglu_pairs=True)


def swiglu_reference(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` the way the reference's kernel evaluates it: fp32 inside, stored in
    the input dtype (engine/kernels/swiglu.py:22-26)."""
    g = gate.float()
    return (g * torch.sigmoid(g) * up.float()).to(gate.dtype)
