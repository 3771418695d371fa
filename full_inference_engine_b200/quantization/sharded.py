"""Column-parallel (N-sharded) quantized linears: one process per GPU, outputs all-gathered.

The reference has no multi-GPU path; this is the partitioning its weight-only linear takes
naturally.  Output channels are independent, and both quantizers compute their statistics
per output row, so rank ``r`` of ``P`` simply owns rows ``[r*N/P, (r+1)*N/P)`` of the packed
weights *and* of the scales: quantize-then-shard equals shard-then-quantize bit for bit.
Activations are replicated; after the local kernel the ``[M, N/P]`` shards are joined with
one ``all_gather`` (NCCL over NVLink on GPUs, gloo in the CPU tests).
"""

from __future__ import annotations

import copy

import torch
import torch.distributed as dist
from torch import nn

from .int8 import Int8Linear
from .w4a16 import W4A16Linear


def shard_rows(out_features: int, world: int, rank: int) -> tuple[int, int]:
    """Row range of ``rank``; the output width must divide evenly."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is not in a world of {world}")
    if out_features % world:
        raise ValueError(f"out_features {out_features} does not divide over {world} ranks")
    rows = out_features // world
    return rank * rows, (rank + 1) * rows


def shard_quantized_linear(module: nn.Module, rank: int, world: int) -> nn.Module:
    """A copy of ``module`` (``W4A16Linear`` or ``Int8Linear``) holding only this rank's rows."""
    start, stop = shard_rows(module.out_features, world, rank)
    if isinstance(module, W4A16Linear):
        local = W4A16Linear(module.in_features, stop - start, group_size=module.group_size,
                            bias=False, device="meta")
        local.packed = module.packed[start:stop].contiguous()
        local.scales = module.scales[start:stop].contiguous()
        local.bias = None if module.bias is None else module.bias[start:stop].contiguous()
        local.reference = module.reference
        return local
    if isinstance(module, Int8Linear):
        local = copy.copy(module)                      # shares nothing mutable we keep
        nn.Module.__init__(local)
        local.in_features, local.out_features = module.in_features, stop - start
        local.reference = module.reference
        local.register_buffer("qweight", module.qweight[start:stop].contiguous())
        local.register_buffer("scales", module.scales[start:stop].contiguous())
        local.register_buffer("bias", None if module.bias is None
                              else module.bias[start:stop].contiguous())
        return local
    raise TypeError(f"cannot shard {type(module).__name__}")


class ColumnParallelLinear(nn.Module):
    """This rank's shard plus the all-gather that rebuilds ``[..., N]`` on every rank."""

    def __init__(self, local: nn.Module, *, world: int | None = None, group=None,
                 gather: bool = True):
        super().__init__()
        self.local = local
        self.group = group
        self.world = world if world is not None else dist.get_world_size(group)
        self.gather = gather
        self.in_features = local.in_features
        self.out_features = local.out_features * self.world

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.local(x)
        if not self.gather or self.world == 1:
            return y
        rows = y.reshape(-1, self.local.out_features)
        if not rows.is_contiguous():
            rows = rows.contiguous()
        m, n_local = rows.shape
        joined = torch.empty((self.world * m, n_local), dtype=rows.dtype, device=rows.device)
        dist.all_gather_into_tensor(joined, rows, group=self.group)
        # [P, M, N/P] -> [M, P, N/P] -> [M, N]: rank r's block lands at columns r*N/P..
        out = joined.view(self.world, m, n_local).permute(1, 0, 2).reshape(m, self.out_features)
        return out.reshape(*x.shape[:-1], self.out_features)

    def extra_repr(self) -> str:
        return f"world={self.world}, gather={self.gather}"
