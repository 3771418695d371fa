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
