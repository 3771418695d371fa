"""N-sharded forward over NCCL on two GPUs: the gathered output equals the 1-GPU output.
Skipped when the box has a single GPU (the CPU twin runs the same logic over gloo)."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from full_inference_engine_b200.quantization import Int8Linear, W4A16Linear
        from full_inference_engine_b200.quantization.sharded import (
            ColumnParallelLinear, shard_quantized_linear)

        torch.manual_seed(0)
        weight = torch.randn(4096, 4096, device="cuda") * 0.02
        w4 = W4A16Linear(4096, 4096).cuda()
        w4.quantize_from(weight)
        w8 = Int8Linear(torch.nn.Linear(4096, 4096, bias=False, device="cuda"))
        for full in (w4, w8):
            shard = ColumnParallelLinear(shard_quantized_linear(full, rank, world), world=world)
            for m in (1, 16, 64, 512):
                x = torch.randn(m, 4096, device="cuda", dtype=torch.bfloat16)
                dist.broadcast(x, 0)
                out = shard(x)
                single = full(x)
                assert out.shape == single.shape
                # the same kernel arithmetic per channel; split-K plans may differ with N, so
                # an element may land on the neighbouring bf16 value (one ulp = 2^-8 relative)
                assert float((out.float() - single.float()).abs().max()) <= \
                    2.0 ** -7 * float(single.float().abs().max())
            # the same through this library's own exchange (peer stores + wait kernel, no NCCL
            # call): chosen by geometry, the push kernel, and the epilogue form
            for form in ("auto", "push", "epilogue"):
                fused = ColumnParallelLinear(shard_quantized_linear(full, rank, world), world=world, fused=True,
                                             gather_form=form)
                for m in (1, 16, 64, 512, 16):
                    x = torch.randn(m, 4096, device="cuda", dtype=torch.bfloat16)
                    dist.broadcast(x, 0)
                    single = full(x)
                    for _ in range(3):                      # back-to-back reuse of the same buffer
                        out = fused(x)
                    torch.cuda.synchronize()
                    assert out.shape == single.shape
                    assert float((out.float() - single.float()).abs().max()) <= \
                        2.0 ** -7 * float(single.float().abs().max()), (type(full).__name__, m, form)
                assert fused.gather_status() == 0
                # and under CUDA-graph replay
                x = torch.randn(16, 4096, device="cuda", dtype=torch.bfloat16)
                dist.broadcast(x, 0)
                fused(x)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    out = fused(x)
                for _ in range(5):
                    graph.replay()
                torch.cuda.synchronize()
                single = full(x)
                assert float((out.float() - single.float()).abs().max()) <= \
                    2.0 ** -7 * float(single.float().abs().max())
                assert fused.gather_status() == 0
        result[rank] = 1
    finally:
        dist.destroy_process_group()


def test_gathered_output_equals_single_gpu_output():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    result = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(2, port, result), nprocs=2, join=True)
    assert sorted(result.keys()) == [0, 1]
