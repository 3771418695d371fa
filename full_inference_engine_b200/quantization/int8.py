"""Per-output-channel INT8 weight-only ``nn.Linear`` replacement on the B200 kernels.

Same surface as the reference's ``engine/quantization/int8.py`` (``Int8Linear(source)``,
``quantize_linear_modules``, ``model_storage_bytes``; buffers ``qweight`` int8 ``[N, K]``,
``scales`` fp32 ``[N]``, ``bias``), but the forward is one fused kernel instead of
"dequantise the whole weight, then ``F.linear``": the int8 weights enter the multiply as
exact fp16/bf16 integers and the fp32 scale and bias are applied to the fp32 accumulator.

The constructor quantizes on the GPU with the reference's arithmetic (fp32 scale
``max|w|.clamp_min(eps)/127``, ``round(w / scale)``), bit-exact against it.
"""

from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F

from ..kernels import w8a16_linear as _k


class Int8Linear(nn.Module):
    """Drop-in for ``nn.Linear`` holding int8 weights and one fp32 scale per output row."""

    def __init__(self, source: nn.Linear):
        super().__init__()
        self.in_features = source.in_features
        self.out_features = source.out_features
        # True: run the reference's own arithmetic (dequantise to the activation dtype, then
        # F.linear) in torch — the comparison target of the kernels, on any device.
        self.reference = False
        qweight, scales = _quantize(source.weight.detach())
        self.register_buffer("qweight", qweight)
        self.register_buffer("scales", scales)
        self.register_buffer("bias", None if source.bias is None else source.bias.detach().clone())

    def forward(self, inputs: torch.Tensor) -> torch.Tensor:
        if self.reference:
            weight = self.qweight.to(inputs.dtype) * self.scales.to(inputs.dtype)[:, None]
            bias = None if self.bias is None else self.bias.to(inputs.dtype)
            return F.linear(inputs, weight, bias)
        if inputs.device.type != "cuda":
            raise RuntimeError("Int8Linear runs on CUDA tensors; set .reference = True for the "
                               "torch arithmetic on other devices")
        rows = inputs.reshape(-1, self.in_features)
        compute = rows if rows.dtype in (torch.float16, torch.bfloat16) else rows.to(torch.float16)
        out = _k.w8a16_linear(compute, self.qweight, self.scales, self.bias, static_weights=True)
        return out.to(inputs.dtype).reshape(*inputs.shape[:-1], self.out_features)

    def extra_repr(self) -> str:
        return (f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}, "
                f"kernel={'reference' if self.reference else 'b200q'}")


def _quantize(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Int8Linear's quantizer (fp32 scales); a module-level hook so host-side tests can swap it."""
    return _k.quantize_weight_per_channel_fp32_scales(weight)


def quantize_linear_modules(module: nn.Module) -> int:
    """Swap every ``nn.Linear`` below ``module`` for an ``Int8Linear``; returns how many."""
    count = 0
    for name, child in list(module.named_children()):
        if isinstance(child, nn.Linear):
            setattr(module, name, Int8Linear(child))
            count += 1
        else:
            count += quantize_linear_modules(child)
    return count


def model_storage_bytes(module: nn.Module) -> int:
    """Bytes of distinct parameter/buffer storage (tied tensors counted once, meta skipped)."""
    seen: set[tuple[str, int]] = set()
    total = 0
    for tensor in (*module.parameters(), *module.buffers()):
        if tensor.device.type == "meta":
            continue
        key = (str(tensor.device), tensor.data_ptr())
        if key not in seen:
            seen.add(key)
            total += tensor.numel() * tensor.element_size()
    return total
