"""Row-parallel (K-sharded) forward with the all-reduce fused into the kernel epilogue, on two
GPUs: equal (to rounding) to the single-GPU forward, for INT4 and W8, eager, with buffer reuse
and under CUDA-graph replay; and paired with a column-parallel first layer (one exchange per
feed-forward).  Skipped on a single-GPU box (the CPU twin runs the bookkeeping over gloo)."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _close(out, single, what):
    err = float((out.float() - single.float()).abs().max())
    assert err <= 1e-2 * float(single.float().abs().max()), (what, err)


def _worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from full_inference_engine_b200.quantization import Int8Linear, W4A16Linear
        from full_inference_engine_b200.quantization.sharded import (
            ColumnParallelLinear, RowParallelLinear, shard_inputs, shard_quantized_linear,
            shard_quantized_linear_inputs)

        torch.manual_seed(0)
        k, n = 12288, 4096                                  # the Qwen3-8B down projection
        weight = torch.randn(n, k, device="cuda") * 0.02
        w4 = W4A16Linear(k, n, bias=True).cuda()
        w4.quantize_from(weight)
        w4.bias = (torch.randn(n, device="cuda") * 0.1).half()
        w8 = Int8Linear(torch.nn.Linear(k, n, bias=False, device="cuda"))
        a, b = shard_inputs(k, world, rank, 128)
        for full in (w4, w8):
            name = type(full).__name__
            plain = RowParallelLinear(shard_quantized_linear_inputs(full, rank, world), world=world)
            fused = RowParallelLinear(shard_quantized_linear_inputs(full, rank, world), world=world, fused=True)
            for m in (1, 16, 200, 512, 16):
                x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
                dist.broadcast(x, 0)
                single = full(x)
                _close(plain(x[:, a:b]), single, (name, m, "nccl"))
                for _ in range(3):                          # back-to-back reuse of buffers and inbox
                    out = fused(x[:, a:b])
                torch.cuda.synchronize()
                assert out.shape == single.shape
                _close(out, single, (name, m, "fused"))
                again = fused(x[:, a:b]).clone()
                assert torch.equal(again, out), "the sum over ranks has a fixed order"
            assert fused.reduce_status() == 0
            for held in fused._buffers_by_rows.values():    # every inbox word was handed back
                assert not bool(held.inbox.any())
            # under CUDA-graph replay
            x = torch.randn(16, k, device="cuda", dtype=torch.bfloat16)
            dist.broadcast(x, 0)
            xs = x[:, a:b].contiguous()
            fused(xs)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = fused(xs)
            for _ in range(5):
                graph.replay()
            torch.cuda.synchronize()
            _close(out, full(x), (name, "graph"))
            assert fused.reduce_status() == 0
        # a feed-forward with ONE exchange: column-parallel up (no gather) -> row-parallel down
        up = W4A16Linear(4096, k).cuda()
        up.quantize_from(torch.randn(k, 4096, device="cuda") * 0.02)
        col = ColumnParallelLinear(shard_quantized_linear(up, rank, world), world=world, gather=False)
        row = RowParallelLinear(shard_quantized_linear_inputs(w4, rank, world), world=world, fused=True)
        x = torch.randn(64, 4096, device="cuda", dtype=torch.float16)
        dist.broadcast(x, 0)
        _close(row(col(x)), w4(up(x)), "paired feed-forward")
        assert row.reduce_status() == 0
        result[rank] = 1
    finally:
        dist.destroy_process_group()


def test_reduced_output_equals_single_gpu_output():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    result = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(2, port, result), nprocs=2, join=True)
    assert sorted(result.keys()) == [0, 1]
