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
import ctypes

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


class SymmetricOutput:
    """A full ``[rows, N]`` output buffer in symmetric memory plus its peer pointers.

    Creating one is a rendezvous: every rank of ``group`` must create the same buffer at the
    same point of its program.  Never create one inside a CUDA-graph capture.
    """

    def __init__(self, rows: int, out_features: int, dtype: torch.dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        from .. import _lib

        group = group if group is not None else dist.group.WORLD
        self.tensor = symm_mem.empty((rows, out_features), dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, group)
        self.desc = _lib.Gather()
        self.desc.rank, self.desc.world = self.handle.rank, self.handle.world_size
        for r in range(self.handle.world_size):
            self.desc.y_peer[r] = self.handle.buffer_ptrs[r]
            self.desc.signal_peer[r] = self.handle.signal_pad_ptrs[r]

    def status(self) -> int:
        """Non-zero if a bounded wait of the fused protocol expired on this rank."""
        pad = self.handle.get_signal_pad(self.handle.rank, (8,), torch.int64)
        return int(pad[2].item())


def fused_forward_gather(rows: torch.Tensor, out: SymmetricOutput, *, qweight=None, packed=None,
                         scales=None, zeros=None, bias=None, group_size: int = 128,
                         form: str = "auto") -> bool:
    """This rank's columns reach every rank's ``out`` through this library's own kernels over
    peer memory (no NCCL); a wait kernel then holds the stream until all ranks' columns have
    arrived here.  ``form``: ``"epilogue"`` — every block of the forward kernel stores its
    finished tile into every rank's buffer; ``"push"`` — a plain forward into this rank's own
    buffer, then a kernel that copies the slab to the peers from hundreds of blocks;
    ``"auto"`` — the library picks by geometry (few large tiles are pushed).  Every rank must
    pass the same ``form``.

    Pass ``qweight`` (int8) for W8A16 or ``packed`` (uint8 reference layout, or int32 with
    ``zeros`` for the asymmetric layout) for INT4; the tensors hold this rank's rows only.
    Returns False (nothing launched) when the tensor-core kernel does not take the geometry.
    """
    from .. import _lib

    lib = _lib.library()
    m, k = rows.shape
    is_w4 = packed is not None
    n_local = (packed if is_w4 else qweight).shape[0]
    tiles = lib.b200q_gather_tiles(4 if is_w4 else 8, m, n_local, k, group_size if is_w4 else 0)
    if tiles <= 0 or m == 0:
        return False
    ws = _lib.workspace_for(rows.device, _lib.workspace_bytes(4 if is_w4 else 8, m, n_local, k))
    stream = _lib.stream_ptr(rows.device)
    bias_ptr = None if bias is None else bias.data_ptr()
    try:
        flags = _lib.FLAG_STATIC_WEIGHTS | {"auto": 0, "epilogue": _lib.FLAG_GATHER_EPILOGUE,
                                            "push": _lib.FLAG_GATHER_PUSH}[form]
    except KeyError:
        raise ValueError(f"form must be auto, epilogue or push; got {form!r}") from None
    with torch.cuda.device(rows.device):
        if is_w4:
            layout = _lib.W4_REF_SPLIT_HALF_SYM if zeros is None else _lib.W4_ASYM_ZP_INT32
            _lib.check(lib.b200q_w4a16_forward_gather(
                rows.data_ptr(), rows.stride(0), _lib.dtype_enum(rows.dtype),
                packed.data_ptr(), packed.stride(0) * packed.element_size(), layout,
                scales.data_ptr(), None if zeros is None else zeros.data_ptr(), group_size, bias_ptr,
                ctypes.byref(out.desc), out.tensor.stride(0), m, n_local, k,
                ws.data_ptr(), ws.numel(), flags, stream),
                "b200q_w4a16_forward_gather")
        else:
            _lib.check(lib.b200q_w8a16_forward_gather(
                rows.data_ptr(), rows.stride(0), _lib.dtype_enum(rows.dtype),
                qweight.data_ptr(), qweight.stride(0), scales.data_ptr(),
                _lib.dtype_enum(scales.dtype), bias_ptr,
                ctypes.byref(out.desc), out.tensor.stride(0), m, n_local, k,
                ws.data_ptr(), ws.numel(), flags, stream),
                "b200q_w8a16_forward_gather")
        _lib.check(lib.b200q_gather_wait(ctypes.byref(out.desc), tiles, stream), "b200q_gather_wait")
    return True


class ColumnParallelLinear(nn.Module):
    """This rank's shard plus the all-gather that rebuilds ``[..., N]`` on every rank.

    ``fused=True`` (CUDA, NVLink peers) replaces "kernel, then NCCL all-gather" by this library's
    own exchange over peer-mapped pointers: the forward writes this rank's columns into its own
    buffer and a push kernel copies them into every peer's, or the forward kernel's epilogue stores
    each finished tile into every rank's buffer (``gather_form``: "auto" picks by geometry, "push",
    "epilogue"); a tiny wait kernel holds the stream until every rank's columns are here.  The
    output is then a persistent
    symmetric-memory buffer per row count (returned as is: copy it if you need it beyond the
    next call with the same row count), allocated on first use by a rendezvous that every rank
    must reach, so all ranks must call with the same sequence of shapes.
    """

    def __init__(self, local: nn.Module, *, world: int | None = None, group=None,
                 gather: bool = True, fused: bool = False, gather_form: str = "auto"):
        super().__init__()
        self.local = local
        self.group = group
        self.world = world if world is not None else dist.get_world_size(group)
        self.gather = gather
        self.fused = fused
        self.gather_form = gather_form
        self.in_features = local.in_features
        self.out_features = local.out_features * self.world
        self._buffers_by_rows: dict = {}

    # ------------------------------------------------------------------ fused path
    def _symmetric_output(self, rows: int, dtype: torch.dtype, device: torch.device) -> SymmetricOutput:
        key = (rows, dtype)
        held = self._buffers_by_rows.get(key)
        if held is None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("first fused call for this row count must happen outside "
                                   "CUDA-graph capture (it allocates symmetric memory)")
            held = SymmetricOutput(rows, self.out_features, dtype, device, self.group)
            self._buffers_by_rows[key] = held
        return held

    def _fused_forward(self, x: torch.Tensor) -> torch.Tensor | None:
        local = self.local
        rows = x.reshape(-1, self.in_features)
        if rows.dtype not in (torch.float16, torch.bfloat16) or rows.device.type != "cuda":
            return None
        if getattr(local, "reference", False) or rows.shape[0] == 0:
            return None
        if rows.stride(1) != 1 or rows.stride(0) % 8 or rows.data_ptr() % 16:
            rows = rows.contiguous()
        out = self._symmetric_output(rows.shape[0], rows.dtype, rows.device)
        bias = None if local.bias is None else local.bias.to(rows.dtype).contiguous()
        if isinstance(local, W4A16Linear):
            done = fused_forward_gather(rows, out, packed=local.packed, scales=local.scales, bias=bias,
                                        group_size=local.group_size, form=self.gather_form)
        else:
            done = fused_forward_gather(rows, out, qweight=local.qweight, scales=local.scales, bias=bias,
                                        form=self.gather_form)
        return out.tensor.reshape(*x.shape[:-1], self.out_features) if done else None

    def gather_status(self) -> int:
        """Non-zero if a bounded wait of the fused protocol ever expired on this rank."""
        status = 0
        for held in self._buffers_by_rows.values():
            status |= held.status()
        return status

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.fused and self.gather and self.world > 1:
            out = self._fused_forward(x)
            if out is not None:
                return out
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


# ---------------------------------------------------------------------------------------
# Row-parallel (K-sharded) linears: the pairing of the column-parallel ones above.
#
# A column-parallel gate/up (or q/k/v) projection leaves rank r with output columns
# [r*N/P, (r+1)*N/P) — which are exactly the INPUT columns a row-parallel down (or o)
# projection needs on rank r.  Each rank then multiplies its activation slice with its K
# slice of the weights and the partial [M, N] results are summed over the ranks: one exchange
# per feed-forward instead of a gather after every layer.  The reference has no such path.

def shard_inputs(in_features: int, world: int, rank: int, group_size: int = 1) -> tuple[int, int]:
    """Input-column range of ``rank``; whole quantization groups, equal shares."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is not in a world of {world}")
    if in_features % (world * group_size):
        raise ValueError(f"in_features {in_features} does not split into {world} shares of whole "
                         f"groups of {group_size}")
    share = in_features // world
    return rank * share, (rank + 1) * share


def shard_quantized_linear_inputs(module: nn.Module, rank: int, world: int) -> nn.Module:
    """A copy of ``module`` holding only this rank's input columns (and their group scales).

    INT4 statistics are per (row, group) and a shard is whole groups, so quantize-then-shard
    equals shard-then-quantize bit for bit.  INT8 scales are per whole row: shard AFTER
    quantizing (every rank keeps the full-row scale).  The bias stays on every shard; the
    row-parallel forward adds it once.
    """
    if isinstance(module, W4A16Linear):
        start, stop = shard_inputs(module.in_features, world, rank, module.group_size)
        local = W4A16Linear(stop - start, module.out_features, group_size=module.group_size,
                            bias=False, device="meta")
        local.packed = module.packed[:, start // 2:stop // 2].contiguous()
        local.scales = module.scales[:, start // module.group_size:stop // module.group_size].contiguous()
        local.bias = None if module.bias is None else module.bias.clone()
        local.reference = module.reference
        return local
    if isinstance(module, Int8Linear):
        start, stop = shard_inputs(module.in_features, world, rank)
        local = copy.copy(module)
        nn.Module.__init__(local)
        local.in_features, local.out_features = stop - start, module.out_features
        local.reference = module.reference
        local.register_buffer("qweight", module.qweight[:, start:stop].contiguous())
        local.register_buffer("scales", module.scales.clone())
        local.register_buffer("bias", None if module.bias is None else module.bias.clone())
        return local
    raise TypeError(f"cannot shard {type(module).__name__}")


class SymmetricReduce:
    """Full ``[rows, N]`` output plus the inbox of partials, both in symmetric memory.

    Creating one is a rendezvous of every rank of ``group``; never inside a graph capture.
    """

    def __init__(self, rows: int, out_features: int, dtype: torch.dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        from .. import _lib

        group = group if group is not None else dist.group.WORLD
        world = dist.get_world_size(group)
        if out_features % world:
            raise ValueError(f"out_features {out_features} does not divide over {world} ranks")
        self.tensor = symm_mem.empty((rows, out_features), dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, group)
        # one 32-bit word per (source rank, row, owned column); zero = "nothing delivered"
        self.inbox = symm_mem.empty((world, rows, out_features // world), dtype=torch.int32, device=device)
        self.inbox.zero_()
        self.inbox_handle = symm_mem.rendezvous(self.inbox, group)
        torch.cuda.synchronize(device)
        dist.barrier(group)                       # every inbox is zero before any rank sends
        self.desc = _lib.Reduce()
        self.desc.rank, self.desc.world = self.handle.rank, self.handle.world_size
        for r in range(self.handle.world_size):
            self.desc.y_peer[r] = self.handle.buffer_ptrs[r]
            self.desc.signal_peer[r] = self.handle.signal_pad_ptrs[r]
            self.desc.inbox_peer[r] = self.inbox_handle.buffer_ptrs[r]

    def status(self) -> int:
        pad = self.handle.get_signal_pad(self.handle.rank, (8,), torch.int64)
        return int(pad[2].item())


def fused_forward_reduce(rows: torch.Tensor, out: SymmetricReduce, *, qweight=None, packed=None,
                         scales=None, zeros=None, bias=None, group_size: int = 128) -> bool:
    """This rank's partial of ``rows_local . W_local^T`` reduced over the ranks inside the kernel's
    epilogue; afterwards ``out.tensor`` holds the full ``[M, N]`` result on every rank.

    ``rows`` is this rank's slice ``[M, K/world]`` of the activations; the weight tensors hold
    this rank's input columns of ALL ``N`` rows.  Returns False (nothing launched) when the
    geometry cannot take the fused path.
    """
    from .. import _lib

    lib = _lib.library()
    m, k_local = rows.shape
    is_w4 = packed is not None
    n = (packed if is_w4 else qweight).shape[0]
    world = out.desc.world
    tiles = lib.b200q_reduce_tiles(4 if is_w4 else 8, m, n, k_local, group_size if is_w4 else 0, world)
    if tiles <= 0 or m == 0:
        return False
    ws = _lib.workspace_for(rows.device, _lib.workspace_bytes(4 if is_w4 else 8, m, n, k_local))
    stream = _lib.stream_ptr(rows.device)
    bias_ptr = None if bias is None else bias.data_ptr()
    with torch.cuda.device(rows.device):
        if is_w4:
            layout = _lib.W4_REF_SPLIT_HALF_SYM if zeros is None else _lib.W4_ASYM_ZP_INT32
            _lib.check(lib.b200q_w4a16_forward_reduce(
                rows.data_ptr(), rows.stride(0), _lib.dtype_enum(rows.dtype),
                packed.data_ptr(), packed.stride(0) * packed.element_size(), layout,
                scales.data_ptr(), None if zeros is None else zeros.data_ptr(), group_size, bias_ptr,
                ctypes.byref(out.desc), out.tensor.stride(0), m, n, k_local,
                ws.data_ptr(), ws.numel(), _lib.FLAG_STATIC_WEIGHTS, stream),
                "b200q_w4a16_forward_reduce")
        else:
            _lib.check(lib.b200q_w8a16_forward_reduce(
                rows.data_ptr(), rows.stride(0), _lib.dtype_enum(rows.dtype),
                qweight.data_ptr(), qweight.stride(0), scales.data_ptr(),
                _lib.dtype_enum(scales.dtype), bias_ptr,
                ctypes.byref(out.desc), out.tensor.stride(0), m, n, k_local,
                ws.data_ptr(), ws.numel(), _lib.FLAG_STATIC_WEIGHTS, stream),
                "b200q_w8a16_forward_reduce")
        _lib.check(lib.b200q_reduce_wait(ctypes.byref(out.desc), tiles, stream), "b200q_reduce_wait")
    return True


class RowParallelLinear(nn.Module):
    """This rank's input-column shard plus the sum over ranks that rebuilds ``[..., N]``.

    ``forward`` takes this rank's SLICE of the activations (``[..., K/world]``).  ``fused=True``
    (CUDA, NVLink peers) does the sum inside the kernel's epilogue through peer memory; otherwise
    the local partial (without bias) goes through one ``all_reduce`` and the bias is added once.
    """

    def __init__(self, local: nn.Module, *, world: int | None = None, group=None, fused: bool = False):
        super().__init__()
        self.local = local
        self.group = group
        self.world = world if world is not None else dist.get_world_size(group)
        self.fused = fused
        self.in_features = local.in_features * self.world
        self.out_features = local.out_features
        self._buffers_by_rows: dict = {}

    def _symmetric(self, rows: int, dtype: torch.dtype, device: torch.device) -> SymmetricReduce:
        key = (rows, dtype)
        held = self._buffers_by_rows.get(key)
        if held is None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("first fused call for this row count must happen outside "
                                   "CUDA-graph capture (it allocates symmetric memory)")
            held = SymmetricReduce(rows, self.out_features, dtype, device, self.group)
            self._buffers_by_rows[key] = held
        return held

    def _fused_forward(self, x: torch.Tensor) -> torch.Tensor | None:
        local = self.local
        rows = x.reshape(-1, local.in_features)
        if rows.dtype not in (torch.float16, torch.bfloat16) or rows.device.type != "cuda":
            return None
        if getattr(local, "reference", False) or rows.shape[0] == 0:
            return None
        if rows.stride(1) != 1 or rows.stride(0) % 8 or rows.data_ptr() % 16:
            rows = rows.contiguous()
        out = self._symmetric(rows.shape[0], rows.dtype, rows.device)
        bias = None if local.bias is None else local.bias.to(rows.dtype).contiguous()
        if isinstance(local, W4A16Linear):
            done = fused_forward_reduce(rows, out, packed=local.packed, scales=local.scales, bias=bias,
                                        group_size=local.group_size)
        else:
            done = fused_forward_reduce(rows, out, qweight=local.qweight, scales=local.scales, bias=bias)
        return out.tensor.reshape(*x.shape[:-1], self.out_features) if done else None

    def reduce_status(self) -> int:
        status = 0
        for held in self._buffers_by_rows.values():
            status |= held.status()
        return status

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.fused and self.world > 1:
            out = self._fused_forward(x)
            if out is not None:
                return out
        bias, self.local.bias = self.local.bias, None     # the partial carries no bias
        try:
            y = self.local(x)
        finally:
            self.local.bias = bias
        if self.world > 1:
            y = y.float()                                  # partials are summed in fp32
            dist.all_reduce(y, group=self.group)
        if bias is not None:
            y = y + bias.to(y.dtype)
        return y.to(x.dtype)

    def extra_repr(self) -> str:
        return f"world={self.world}, fused={self.fused}"
