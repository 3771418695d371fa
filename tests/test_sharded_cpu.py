"""Column-parallel sharding over two gloo ranks on CPU: the gathered output of the N-sharded
module equals the single-process output, and a shard's buffers are slices of the whole."""

from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from full_inference_engine_b200.quantization import W4A16Linear
from full_inference_engine_b200.quantization.sharded import (
    ColumnParallelLinear, shard_quantized_linear, shard_rows,
)
from oracle import wq_oracle as oracle


def _layer(n=96, k=256, bias=True):
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    packed, scales = oracle.quantize_w4_grouped(w, 128)
    layer = W4A16Linear(k, n, bias=bias, device="meta")
    layer.packed, layer.scales = torch.from_numpy(packed), torch.from_numpy(scales)
    if bias:
        layer.bias = torch.from_numpy(rng.standard_normal(n).astype(np.float16))
    layer.reference = True
    return layer, w


def test_shard_rows_and_buffer_slices():
    assert shard_rows(96, 4, 1) == (24, 48)
    with pytest.raises(ValueError):
        shard_rows(100, 8, 0)
    with pytest.raises(ValueError):
        shard_rows(96, 4, 4)
    layer, w = _layer()
    for world in (2, 4, 8):
        for rank in range(world):
            local = shard_quantized_linear(layer, rank, world)
            a, b = shard_rows(96, world, rank)
            assert torch.equal(local.packed, layer.packed[a:b])
            assert torch.equal(local.scales, layer.scales[a:b])
            assert torch.equal(local.bias, layer.bias[a:b])
            # shard-then-quantize gives the same bytes
            p, s = oracle.quantize_w4_grouped(w[a:b], 128)
            assert np.array_equal(local.packed.numpy(), p)
            assert np.array_equal(local.scales.numpy().view(np.uint16), s.view(np.uint16))


def _worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(1)
        layer, _ = _layer()
        x = torch.randn(3, 5, 256)
        full = layer(x)
        parallel = ColumnParallelLinear(shard_quantized_linear(layer, rank, world), world=world)
        out = parallel(x)
        assert out.shape == full.shape
        assert torch.equal(out, full), float((out - full).abs().max())
        local_only = ColumnParallelLinear(shard_quantized_linear(layer, rank, world), world=world,
                                          gather=False)(x)
        a, b = shard_rows(96, world, rank)
        assert torch.equal(local_only, full[..., a:b])
        result[rank] = 1
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_gathered_output_equals_single_process_output(world):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    result = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, port, result), nprocs=world, join=True)
    assert sorted(result.keys()) == list(range(world))


def test_gather_form_is_a_function_of_the_geometry_only():
    """Every rank must pick the same way to deliver its columns (the forms count arrivals alike
    but launch different kernels): few large tiles and single-row int8 calls are pushed."""
    from full_inference_engine_b200 import _lib

    lib = _lib.library()
    form = lambda fmt, m, n_local, k, world, flags=0: lib.b200q_gather_form(fmt, m, n_local, k, 128, world, flags)
    assert form(8, 512, 512, 4096, 8) == 1                 # 16 tiles of 32 KiB x 7 peers
    assert form(4, 256, 1536, 4096, 8) == 1                # 12 tiles of 64 KiB x 7 peers
    assert form(4, 4096, 1536, 4096, 8) == 0               # hundreds of tiles: the epilogue hides the stores
    assert form(4, 16, 1536, 4096, 8) == 0                 # small tiles
    assert form(8, 1, 2048, 4096, 2) == 1                  # the int8 GEMV has no gather epilogue
    assert form(8, 512, 2048, 4096, 2) == 0                # one peer: a tile never reaches 96 KiB
    assert form(8, 512, 512, 4096, 8, _lib.FLAG_GATHER_EPILOGUE) == 0
    assert form(4, 16, 1536, 4096, 8, _lib.FLAG_GATHER_PUSH) == 1
    assert form(4, 16, 1536, 4000, 8) == -1                # the tensor-core kernels do not take this K


def test_column_parallel_module_carries_the_gather_form():
    """The form is part of the module's configuration (every rank must build it alike) and is
    validated where it is used, not silently ignored."""
    from full_inference_engine_b200.quantization.sharded import ColumnParallelLinear, fused_forward_gather

    local = W4A16Linear(256, 128)
    for form in ("auto", "push", "epilogue"):
        assert ColumnParallelLinear(local, world=2, fused=True, gather_form=form).gather_form == form
    assert ColumnParallelLinear(local, world=2).gather_form == "auto"
    import inspect
    assert inspect.signature(fused_forward_gather).parameters["form"].default == "auto"
