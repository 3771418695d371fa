"""Quantized gate/up projections and the SwiGLU product as one kernel, installed on a model.

The surface of the reference's ``engine/kernels/swiglu.py`` for quantized feed-forwards:
``FusedGateUpSwiGLU`` plays the part of ``FusedGateUpProjection`` + ``triton_swiglu``
(engine/kernels/swiglu.py:43-83), ``install_fused_swiglu`` / ``uninstall_fused_swiglu`` the
part of ``install_triton_swiglu`` / ``uninstall_triton_swiglu`` (engine/kernels/swiglu.py:
86-140).  The reference can only fuse fp16 ``nn.Linear`` pairs (it concatenates ``.weight``);
this one takes the pair after quantization (``W4A16Linear`` or ``Int8Linear``), interleaves
their rows and lets the kernel's epilogue write ``silu(gate) * up``.

Feed-forwards are found structurally, as in the reference: any module with ``gate_proj``,
``up_proj`` and ``down_proj`` attributes.
"""

from __future__ import annotations

from types import MethodType

import torch
from torch import nn

from ..kernels import swiglu as _k
from .int8 import Int8Linear
from .w4a16 import W4A16Linear


class FusedGateUpSwiGLU(nn.Module):
    """``silu(gate_proj(x)) * up_proj(x)`` over the interleaved quantized weights of the pair."""

    def __init__(self, gate: nn.Module, up: nn.Module):
        super().__init__()
        if type(gate) is not type(up) or not isinstance(gate, (W4A16Linear, Int8Linear)):
            raise ValueError("gate/up projections must both be W4A16Linear or both Int8Linear")
        if (gate.in_features != up.in_features or gate.out_features != up.out_features
                or (gate.bias is None) != (up.bias is None)):
            raise ValueError("gate/up projections must have matching geometry and bias layout")
        self.in_features = gate.in_features
        self.out_features = gate.out_features
        self.kind = "w4a16" if isinstance(gate, W4A16Linear) else "int8"
        # True: run the two projections' reference arithmetic and the reference's SwiGLU in torch
        self.reference = False
        if self.kind == "w4a16":
            if gate.group_size != up.group_size:
                raise ValueError("gate/up projections must share one group size")
            if not (gate.loaded and up.loaded):
                raise ValueError("gate/up projections have no weights yet")
            self.group_size = gate.group_size
            self.register_buffer("packed", _k.interleave_gate_up(gate.packed, up.packed))
            self.register_buffer("scales", _k.interleave_gate_up(gate.scales, up.scales))
        else:
            self.register_buffer("qweight", _k.interleave_gate_up(gate.qweight, up.qweight))
            self.register_buffer("scales", _k.interleave_gate_up(gate.scales, up.scales))
        if gate.bias is None:
            self.register_buffer("bias", None)
        else:
            self.register_buffer("bias", _k.interleave_gate_up(gate.bias.detach(), up.bias.detach()))

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        rows = hidden_states.reshape(-1, self.in_features)
        if self.reference:
            out = self._reference_forward(rows)
        elif rows.device.type != "cuda":
            raise RuntimeError("FusedGateUpSwiGLU runs on CUDA tensors; set .reference = True for "
                               "the torch arithmetic on other devices")
        else:
            compute = rows if rows.dtype in (torch.float16, torch.bfloat16) else rows.to(torch.float16)
            if self.kind == "w4a16":
                out = _k.w4a16_gate_up_swiglu(compute, self.packed, self.scales, self.bias,
                                              group_size=self.group_size, static_weights=True)
            else:
                out = _k.w8a16_gate_up_swiglu(compute, self.qweight, self.scales, self.bias,
                                              static_weights=True)
            out = out.to(hidden_states.dtype)
        return out.reshape(*hidden_states.shape[:-1], self.out_features)

    def _reference_forward(self, rows: torch.Tensor) -> torch.Tensor:
        """Two dequantise-then-``F.linear`` projections (as the unfused reference modules run
        them) followed by the reference's fp32 SwiGLU."""
        from torch.nn import functional as F
        from ..kernels.w4a16_format import unpack_w4_reference

        halves = []
        for part in (0, 1):
            bias = None if self.bias is None else self.bias[part::2].to(rows.dtype)
            if self.kind == "w4a16":
                weight = unpack_w4_reference(self.packed[part::2].contiguous(),
                                             self.scales[part::2].contiguous(),
                                             self.in_features, self.group_size).to(rows.dtype)
            else:
                weight = self.qweight[part::2].to(rows.dtype) * self.scales[part::2].to(rows.dtype)[:, None]
            halves.append(F.linear(rows, weight, bias))
        return _k.swiglu_reference(halves[0], halves[1])

    def extra_repr(self) -> str:
        return (f"in={self.in_features}, out={self.out_features}, weights={self.kind}, "
                f"bias={self.bias is not None}, kernel={'reference' if self.reference else 'b200q'}")


def _fused_mlp_forward(module, hidden_states: torch.Tensor) -> torch.Tensor:
    return module.down_proj(module.fused_gate_up_swiglu(hidden_states))


def _feed_forwards(model: nn.Module):
    for module in model.modules():
        if all(hasattr(module, name) for name in ("gate_proj", "up_proj", "down_proj")):
            yield module


def install_fused_swiglu(model: nn.Module) -> int:
    """Fuse gate/up/SwiGLU of every quantized feed-forward in ``model``; returns how many.

    A feed-forward whose gate/up pair is not (yet) a quantized pair is left alone.  The
    original projections stay reachable for ``uninstall_fused_swiglu`` but leave the module
    tree, so their buffers stop counting as model state.
    """
    installed = 0
    for module in _feed_forwards(model):
        if hasattr(module, "_pre_fused_swiglu_forward"):
            installed += 1
            continue
        gate, up = module.gate_proj, module.up_proj
        if type(gate) is not type(up) or not isinstance(gate, (W4A16Linear, Int8Linear)):
            continue
        fused = FusedGateUpSwiGLU(gate, up)
        module._pre_fused_swiglu_forward = module.forward.__func__
        module.__dict__["_pre_fused_gate_proj"] = gate
        module.__dict__["_pre_fused_up_proj"] = up
        module.gate_proj = None
        module.up_proj = None
        module.fused_gate_up_swiglu = fused
        module.forward = MethodType(_fused_mlp_forward, module)
        installed += 1
    if installed == 0:
        raise RuntimeError("model contains no quantized gate/up/down SwiGLU feed-forward to fuse")
    return installed


def uninstall_fused_swiglu(model: nn.Module) -> int:
    restored = 0
    for module in model.modules():
        original = getattr(module, "_pre_fused_swiglu_forward", None)
        if original is None:
            continue
        module.forward = MethodType(original, module)
        del module._pre_fused_swiglu_forward
        del module.fused_gate_up_swiglu
        module.gate_proj = module.__dict__.pop("_pre_fused_gate_proj")
        module.up_proj = module.__dict__.pop("_pre_fused_up_proj")
        restored += 1
    return restored
