"""Row-parallel (K-sharded) sharding over two gloo ranks on CPU: a shard's buffers are slices of
the whole along K (whole groups), quantize-then-shard equals shard-then-quantize for INT4, and
the all-reduced output of the shards equals the single-process output; together with a
column-parallel first layer a feed-forward needs one exchange."""

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
    ColumnParallelLinear, RowParallelLinear, shard_inputs, shard_quantized_linear,
    shard_quantized_linear_inputs,
)
from oracle import wq_oracle as oracle


def _layer(n, k, seed, bias=True):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    packed, scales = oracle.quantize_w4_grouped(w, 128)
    layer = W4A16Linear(k, n, bias=bias, device="meta")
    layer.packed, layer.scales = torch.from_numpy(packed), torch.from_numpy(scales)
    if bias:
        layer.bias = torch.from_numpy(rng.standard_normal(n).astype(np.float16))
    layer.reference = True
    return layer, w


def test_shard_inputs_and_buffer_slices():
    assert shard_inputs(1024, 4, 1, 128) == (256, 512)
    with pytest.raises(ValueError):
        shard_inputs(1024, 3, 0, 128)          # 1024 / 3 is not whole groups
    with pytest.raises(ValueError):
        shard_inputs(1024, 4, 4, 128)
    layer, w = _layer(96, 1024, 0)
    for world in (2, 4, 8):
        for rank in range(world):
            local = shard_quantized_linear_inputs(layer, rank, world)
            a, b = shard_inputs(1024, world, rank, 128)
            assert local.in_features == b - a and local.out_features == 96
            assert torch.equal(local.packed, layer.packed[:, a // 2:b // 2])
            assert torch.equal(local.scales, layer.scales[:, a // 128:b // 128])
            assert torch.equal(local.bias, layer.bias)
            p, s = oracle.quantize_w4_grouped(np.ascontiguousarray(w[:, a:b]), 128)     # shard, then quantize
            assert np.array_equal(local.packed.numpy(), p)
            assert np.array_equal(local.scales.numpy().view(np.uint16), s.view(np.uint16))


def _worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(1)
        up, _ = _layer(512, 256, 1)            # column-parallel: 256 -> 512
        down, _ = _layer(96, 512, 2)           # row-parallel:    512 -> 96
        x = torch.randn(3, 5, 256)
        hidden = up(x)
        full = down(hidden)
        # the row-parallel layer alone, fed with this rank's slice of the full activations
        a, b = shard_inputs(512, world, rank, 128)
        row = RowParallelLinear(shard_quantized_linear_inputs(down, rank, world), world=world)
        out = row(hidden[..., a:b])
        assert out.shape == full.shape
        tol = 2.0 ** -9 * float(full.float().abs().max())     # fp32 sum of fp16 partials vs one fp16 GEMM
        assert float((out.float() - full.float()).abs().max()) <= tol
        # column-parallel up WITHOUT its gather feeding row-parallel down: one exchange in all
        col = ColumnParallelLinear(shard_quantized_linear(up, rank, world), world=world, gather=False)
        assert col(x).shape[-1] == b - a
        paired = row(col(x))
        assert float((paired.float() - full.float()).abs().max()) <= tol
        result[rank] = 1
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_all_reduced_output_equals_single_process_output(world):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    result = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, port, result), nprocs=world, join=True)
    assert sorted(result.keys()) == list(range(world))
