"""Quantized projections that read the same activations, run as ONE launch.

A decoder layer's q/k/v projections (and gate/up when the SwiGLU fusion is not installed) each
read the same hidden states; at decode and mixed-step widths every launch costs microseconds of
fixed latency for a few megabytes of weights.  Quantization is per output row, so concatenating
the projections' quantized rows gives one weight-only linear with N = sum of the parts whose
output columns are the parts' outputs side by side, bit for bit: one launch instead of three.
The reference concatenates fp16 ``.weight``s the same way for its gate/up pair
(engine/kernels/swiglu.py:43-63) and has no quantized counterpart.

``install_fused_qkv`` finds attention blocks structurally (``q_proj``, ``k_proj``, ``v_proj``
attributes, as engine/quantization/w4a16.py:185-210 finds its targets) and replaces the three
projections with views of one ``FusedProjections`` module: the first view called with a tensor
runs the launch, the other two hand out their columns of that result.
"""

from __future__ import annotations

import torch
from torch import nn

from .int8 import Int8Linear
from .w4a16 import W4A16Linear


class FusedProjections(nn.Module):
    """Row-wise concatenation of quantized linears over one input; returns the parts' outputs."""

    def __init__(self, parts: list[nn.Module]):
        super().__init__()
        if not parts:
            raise ValueError("nothing to fuse")
        first = parts[0]
        if not isinstance(first, (W4A16Linear, Int8Linear)) or any(type(p) is not type(first) for p in parts):
            raise ValueError("projections must all be W4A16Linear or all Int8Linear")
        if any(p.in_features != first.in_features for p in parts):
            raise ValueError("projections must read the same input width")
        if any((p.bias is None) != (first.bias is None) for p in parts):
            raise ValueError("projections must all have a bias or none")
        self.splits = [p.out_features for p in parts]
        if isinstance(first, W4A16Linear):
            if any(p.group_size != first.group_size for p in parts) or not all(p.loaded for p in parts):
                raise ValueError("projections must be loaded and share one group size")
            fused = W4A16Linear(first.in_features, sum(self.splits), group_size=first.group_size,
                                bias=False, device="meta")
            fused.packed = torch.cat([p.packed for p in parts], dim=0).contiguous()
            fused.scales = torch.cat([p.scales for p in parts], dim=0).contiguous()
        else:
            fused = Int8Linear.__new__(Int8Linear)
            nn.Module.__init__(fused)
            fused.in_features, fused.out_features = first.in_features, sum(self.splits)
            fused.reference = first.reference
            fused.register_buffer("qweight", torch.cat([p.qweight for p in parts], dim=0).contiguous())
            fused.register_buffer("scales", torch.cat([p.scales for p in parts], dim=0).contiguous())
            fused.register_buffer("bias", None)
        if first.bias is not None:
            fused.bias = torch.cat([p.bias.detach() for p in parts], dim=0).contiguous()
        fused.reference = getattr(first, "reference", False)
        self.fused = fused
        self.in_features, self.out_features = first.in_features, sum(self.splits)
        self._seen = None            # (input tensor, outputs) of the launch the views share

    def forward(self, hidden_states: torch.Tensor) -> tuple[torch.Tensor, ...]:
        return torch.split(self.fused(hidden_states), self.splits, dim=-1)

    def part(self, index: int, hidden_states: torch.Tensor) -> torch.Tensor:
        """Output of projection ``index``; the launch runs once per distinct input tensor."""
        seen = self._seen
        if seen is None or seen[0] is not hidden_states:
            seen = (hidden_states, self.forward(hidden_states))
            self._seen = seen
        out = seen[1][index]
        if index == len(self.splits) - 1:
            self._seen = None        # the last view lets go of the activations
        return out


class _ProjectionView(nn.Module):
    """Stands where one of the fused projections stood."""

    def __init__(self, owner: FusedProjections, index: int, holds_owner: bool):
        super().__init__()
        if holds_owner:
            self.owner = owner                     # registered once, so its buffers count once
        else:
            self.__dict__["owner"] = owner
        self.index = index
        self.in_features, self.out_features = owner.in_features, owner.splits[index]

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return self.owner.part(self.index, hidden_states)


def _attention_blocks(model: nn.Module):
    for module in model.modules():
        if all(hasattr(module, name) for name in ("q_proj", "k_proj", "v_proj")):
            yield module


def install_fused_qkv(model: nn.Module) -> int:
    """Fuse q/k/v of every attention block whose three projections are quantized alike."""
    installed = 0
    for block in _attention_blocks(model):
        if "_pre_fused_qkv" in block.__dict__:
            installed += 1
            continue
        parts = [block.q_proj, block.k_proj, block.v_proj]
        if not isinstance(parts[0], (W4A16Linear, Int8Linear)) or any(type(p) is not type(parts[0]) for p in parts):
            continue
        owner = FusedProjections(parts)
        block.__dict__["_pre_fused_qkv"] = parts
        block.q_proj = _ProjectionView(owner, 0, True)
        block.k_proj = _ProjectionView(owner, 1, False)
        block.v_proj = _ProjectionView(owner, 2, False)
        installed += 1
    if installed == 0:
        raise RuntimeError("model contains no attention block with quantized q/k/v projections")
    return installed


def uninstall_fused_qkv(model: nn.Module) -> int:
    restored = 0
    for block in model.modules():
        parts = block.__dict__.pop("_pre_fused_qkv", None)
        if parts is None:
            continue
        block.q_proj, block.k_proj, block.v_proj = parts
        restored += 1
    return restored
