"""Greedy token choice over a quantized output head in one kernel.

The reference decodes greedily as ``lm_head(hidden)`` followed by ``torch.argmax`` over the
``[M, vocab]`` logits (two kernels and a ``vocab``-wide round trip through memory).  With
``B200Q_FLAG_ARGMAX`` the projection kernel's epilogue reduces every row to the channel of its
largest output, so the logits are never written.  Values are rounded to the activation dtype
exactly as the plain projection would store them, and among equal values the smallest channel
wins, so the result equals ``w4a16_linear(...).argmax(-1)``.
"""

from __future__ import annotations

import torch

from . import w4a16_linear as _w4
from . import w8a16_linear as _w8
from .w4a16_format import GROUP_SIZE


def w4a16_linear_argmax(inputs: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor,
                        bias: torch.Tensor | None = None, *, group_size: int = GROUP_SIZE,
                        zeros: torch.Tensor | None = None,
                        static_weights: bool = False) -> torch.Tensor:
    """``w4a16_linear(inputs, ...).argmax(-1)`` (int64 ``[M]``) without materialising the outputs."""
    return _w4.w4a16_linear(inputs, packed, scales, bias, group_size=group_size, zeros=zeros,
                            static_weights=static_weights, _argmax=True)


def w8a16_linear_argmax(inputs: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor,
                        bias: torch.Tensor | None = None, *,
                        static_weights: bool = False) -> torch.Tensor:
    """``w8a16_linear(inputs, ...).argmax(-1)`` (int64 ``[M]``) without materialising the outputs."""
    return _w8.w8a16_linear(inputs, qweight, scales, bias, static_weights=static_weights, _argmax=True)
