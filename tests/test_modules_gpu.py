"""The module layer on a B200: installed models run the kernels and agree with the same
packed weights run through torch (``reference_mode``), CUDA-graph capture and replay of a
mixed step, the streaming loader on the GPU.  Follows the reference's
tests/quantization/test_w4a16_cuda.py with random-init models (no checkpoint is available
offline) and benchmark configuration 3 for the graph test."""

from __future__ import annotations

import pytest
import torch
from torch import nn

from full_inference_engine_b200 import _lib
from full_inference_engine_b200.kernels import w4a16_linear
from full_inference_engine_b200.kernels.w4a16_format import unpack_w4_reference
from full_inference_engine_b200.quantization import (
    Int8Linear, W4A16Linear, describe, install_w4a16, load_w4a16_model, quantize_linear_modules,
    reference_mode, w4a16_modules,
)
from full_inference_engine_b200.quantization.w4a16 import dense_scratch

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")


def _model(hidden, inter, heads, kv, head_dim, vocab, layers=2, dtype=torch.float16, tie=False):
    from transformers import AutoModelForCausalLM, Qwen3Config

    cfg = Qwen3Config(hidden_size=hidden, intermediate_size=inter, num_hidden_layers=layers,
                      num_attention_heads=heads, num_key_value_heads=kv, head_dim=head_dim,
                      vocab_size=vocab, max_position_embeddings=256, tie_word_embeddings=tie)
    torch.manual_seed(0)
    return AutoModelForCausalLM.from_config(cfg, dtype=dtype).eval()


def _logits(model, ids):
    with torch.no_grad():
        return model(input_ids=ids, use_cache=False).logits


@pytest.mark.parametrize("shape,group", [((64, 128, 4, 2, 16, 256), 32), ((256, 512, 4, 2, 64, 512), 128)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_installed_model_kernels_agree_with_reference_mode(shape, group, dtype):
    model = _model(*shape, dtype=dtype).cuda()
    report = install_w4a16(model, group_size=group)
    assert report.replaced == 15 and report.by_kind == {"attention": 8, "mlp": 6, "lm_head": 1}
    assert all(m.packed.is_cuda for m in w4a16_modules(model))
    assert describe(model)["kernel"].startswith("b200q")
    for tokens in (3, 48):                       # decode-width and prefill-width row counts
        ids = torch.randint(0, shape[-1], (1, tokens), device="cuda")
        before = _lib.launch_count()
        actual = _logits(model, ids).float()
        assert _lib.launch_count() - before == 15, "every projection must run one b200q kernel"
        with reference_mode(model):
            expected = _logits(model, ids).float()
        tol = 2e-2 if dtype is torch.float16 else 8e-2
        torch.testing.assert_close(actual, expected, rtol=tol, atol=1e-1)
        top2 = expected.topk(2, dim=-1).values
        decided = (top2[..., 0] - top2[..., 1]) > 0.2
        assert torch.equal(actual.argmax(-1)[decided], expected.argmax(-1)[decided])


def test_layer_equals_linear_over_its_own_dequantised_weight():
    torch.manual_seed(1)
    layer = W4A16Linear(1024, 3072, bias=True).cuda()
    layer.quantize_from(torch.randn(3072, 1024, device="cuda", dtype=torch.float16))
    layer.set_bias(torch.randn(3072, device="cuda"))
    for rows in (1, 2, 7, 64, 200):
        x = torch.randn(2, rows, 1024, device="cuda", dtype=torch.float16)
        weight = unpack_w4_reference(layer.packed, layer.scales, 1024).float()
        expected = x.float() @ weight.T + layer.bias.float()
        out = layer(x)
        assert out.shape == (2, rows, 3072) and out.dtype is torch.float16
        assert float((out.float() - expected).abs().max()) <= 1e-2 * float(expected.abs().max())
    out32 = layer(torch.randn(4, 1024, device="cuda"))          # fp32 in -> fp32 out
    assert out32.dtype is torch.float32


def test_int8_linear_kernel_agrees_with_its_reference_arithmetic():
    torch.manual_seed(2)
    model = nn.Sequential(nn.Linear(1024, 2048), nn.GELU(), nn.Linear(2048, 1024, bias=False))
    model = model.half().cuda()
    assert quantize_linear_modules(model) == 2
    assert all(isinstance(m, Int8Linear) for m in (model[0], model[2]))
    for rows in (1, 16, 144):
        x = torch.randn(rows, 1024, device="cuda", dtype=torch.float16)
        out = model(x)
        for m in (model[0], model[2]):
            m.reference = True
        expected = model(x)
        for m in (model[0], model[2]):
            m.reference = False
        assert float((out.float() - expected.float()).abs().max()) <= 1e-2 * float(expected.abs().max())


def test_dense_scratch_and_dequantize_into_keep_the_reference_contract():
    torch.manual_seed(4)
    a = W4A16Linear(1024, 3072).cuda()
    a.quantize_from(torch.randn(3072, 1024, device="cuda", dtype=torch.float16))
    scratch = dense_scratch(torch.device("cuda", 0), 3072, 1024)
    again = dense_scratch(torch.device("cuda", 0), 1024, 1024)
    assert again.data_ptr() == scratch.data_ptr(), "one buffer per device, grown to the largest tile"
    w4a16_linear.w4_dequantize_into(scratch, a.packed, a.scales)
    assert torch.equal(scratch, a.dequantized())


class _Block(nn.Module):
    """The seven projections of one Qwen3 decoder layer, under their usual attribute names."""

    def __init__(self, hidden, heads, kv, head_dim, inter):
        super().__init__()
        self.q_proj = nn.Linear(hidden, heads * head_dim, bias=False)
        self.k_proj = nn.Linear(hidden, kv * head_dim, bias=False)
        self.v_proj = nn.Linear(hidden, kv * head_dim, bias=False)
        self.o_proj = nn.Linear(heads * head_dim, hidden, bias=False)
        self.gate_proj = nn.Linear(hidden, inter, bias=False)
        self.up_proj = nn.Linear(hidden, inter, bias=False)
        self.down_proj = nn.Linear(inter, hidden, bias=False)

    def forward(self, h):
        """Every projection once; cheap elementwise glue keeps activations O(1)."""
        q, k, v = self.q_proj(h), self.k_proj(h), self.v_proj(h)
        mix = q * torch.cat([k, v], dim=-1).tanh()
        h = torch.nn.functional.normalize(h + self.o_proj(mix), dim=-1) * 32.0
        g, u = self.gate_proj(h), self.up_proj(h)
        return torch.nn.functional.normalize(
            h + self.down_proj(torch.nn.functional.silu(g) * u), dim=-1) * 32.0


def _projection_stack(layers=28, hidden=1024, heads=16, kv=8, head_dim=128, inter=3072):
    """benchmark configuration 3: the seven Qwen3-0.6B projections of every layer, random-init."""
    torch.manual_seed(0)
    stack = nn.Sequential(*[_Block(hidden, heads, kv, head_dim, inter) for _ in range(layers)])
    for p in stack.parameters():
        nn.init.normal_(p, std=0.02)
    return stack.half().cuda()


def _stack_forward(blocks, h):
    return blocks(h)


@pytest.mark.parametrize("quant", ["w8", "w4"])
def test_mixed_step_is_captured_and_replayed_as_a_cuda_graph(quant):
    """M = 144 rows (16 decode tokens + one 128-token chunk) through 28 x 7 projections:
    eager warm-up, capture, replay; replay equals eager bit for bit and allocates nothing."""
    blocks = _projection_stack()
    if quant == "w8":
        assert quantize_linear_modules(blocks) == 28 * 7
    else:
        assert install_w4a16(blocks, targets=("attention", "mlp")).replaced == 28 * 7
    static_in = torch.randn(1, 144, 1024, device="cuda", dtype=torch.float16)
    with torch.inference_mode():
        eager = _stack_forward(blocks, static_in).clone()          # compile and allocate
        torch.cuda.synchronize()
        before = _lib.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_out = _stack_forward(blocks, static_in)
        assert _lib.launch_count() - before == 28 * 7
        torch.cuda.synchronize()
        allocated = torch.cuda.memory_allocated()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == allocated
        assert torch.equal(static_out, eager)
        # new input through the same graph
        fresh = torch.randn_like(static_in)
        static_in.copy_(fresh)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(static_out, _stack_forward(blocks, fresh))
    ws = _lib.workspace_for(torch.device("cuda", 0), 256)
    assert _lib.library().b200q_workspace_status(ws.data_ptr(), None) == _lib.OK


def test_streaming_loader_onto_the_gpu_matches_install(tmp_path):
    model = _model(256, 512, 4, 2, 64, 512, dtype=torch.float16)
    model.save_pretrained(tmp_path, safe_serialization=True)
    ids = torch.randint(0, 512, (1, 7), device="cuda")
    model = model.cuda()
    install_w4a16(model)
    expected = _logits(model, ids)
    loaded, report = load_w4a16_model(str(tmp_path), device="cuda")
    assert report.replaced == 15 and report.skipped == []
    assert not any(t.device.type == "meta" for t in (*loaded.parameters(), *loaded.buffers()))
    assert all(m.packed.is_cuda for m in w4a16_modules(loaded))
    for a, b in zip(w4a16_modules(model), w4a16_modules(loaded)):
        assert torch.equal(a.packed, b.packed) and torch.equal(a.scales, b.scales)
    torch.testing.assert_close(_logits(loaded, ids), expected, rtol=0, atol=0)
    tied = _model(256, 512, 4, 2, 64, 512, tie=True)
    tied.save_pretrained(tmp_path / "tied", safe_serialization=True)
    loaded, report = load_w4a16_model(str(tmp_path / "tied"), device="cuda")
    head = loaded.get_output_embeddings()
    assert isinstance(head, W4A16Linear) and head.loaded and report.by_kind["lm_head"] == 1
    assert torch.isfinite(_logits(loaded, ids)).all()


def test_fused_qkv_runs_one_launch_for_three_projections():
    """q/k/v concatenated into one weight-only linear: two launches fewer per layer, and the
    logits stay within rounding of the unfused model's (same kernel arithmetic per channel)."""
    from full_inference_engine_b200.quantization import install_fused_qkv, uninstall_fused_qkv

    shape = (256, 512, 4, 2, 64, 512)
    model = _model(*shape, dtype=torch.float16).cuda()
    install_w4a16(model, group_size=128)
    ids = torch.randint(0, shape[-1], (1, 24), device="cuda")
    expected = _logits(model, ids).float()
    assert install_fused_qkv(model) == 2
    before = _lib.launch_count()
    actual = _logits(model, ids).float()
    assert _lib.launch_count() - before == 15 - 2 * 2
    torch.testing.assert_close(actual, expected, rtol=2e-2, atol=1e-1)
    with reference_mode(model):
        reference = _logits(model, ids).float()
    torch.testing.assert_close(actual, reference, rtol=2e-2, atol=1e-1)
    assert uninstall_fused_qkv(model) == 2
    torch.testing.assert_close(_logits(model, ids).float(), expected, rtol=0, atol=0)
