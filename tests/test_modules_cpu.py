"""Host-side logic of the module layer on CPU: structural install, reports, reference mode,
the streaming loader, error behaviour.  The CUDA quantizer is swapped for the CPU oracle
(test infrastructure) so that none of this needs a GPU; forwards run in ``reference`` mode,
which is torch arithmetic by design.  Mirrors the reference's
tests/quantization/test_w4a16_install.py and tests/quantization/test_int8.py."""

from __future__ import annotations

import numpy as np
import pytest
import torch
from torch import nn
from torch.nn import functional as F

from full_inference_engine_b200.kernels.w4a16_format import unpack_w4_reference
from full_inference_engine_b200.quantization import int8 as int8_mod
from full_inference_engine_b200.quantization import w4a16 as w4_mod
from full_inference_engine_b200.quantization import (
    Int8Linear, W4A16Linear, describe, install_w4a16, load_w4a16_model, model_storage_bytes,
    quantize_linear_modules, reference_mode, w4a16_modules,
)
from oracle import wq_oracle as oracle

transformers = pytest.importorskip("transformers")
GROUP = 32


@pytest.fixture(autouse=True)
def oracle_quantizers(monkeypatch):
    def w4(weight, group_size):
        w = weight.float().numpy() if weight.dtype is torch.bfloat16 else weight.numpy()
        p, s = oracle.quantize_w4_grouped(w, group_size)
        return torch.from_numpy(p), torch.from_numpy(s)

    def w8(weight):
        q, s = oracle.quantize_w8_int8linear(weight.float().numpy())
        return torch.from_numpy(q), torch.from_numpy(s)

    monkeypatch.setattr(w4_mod, "_quantize", w4)
    monkeypatch.setattr(int8_mod, "_quantize", w8)


def _tiny_config(tie=False):
    from transformers import Qwen3Config

    return Qwen3Config(hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=256,
                       max_position_embeddings=128, tie_word_embeddings=tie)


def _tiny_model(tie=False, dtype=torch.float32):
    from transformers import AutoModelForCausalLM

    torch.manual_seed(0)
    return AutoModelForCausalLM.from_config(_tiny_config(tie), dtype=dtype).eval()


def _logits(model, ids):
    with torch.no_grad():
        return model(input_ids=ids, use_cache=False).logits


def test_install_replaces_every_projection_and_the_head():
    model = _tiny_model()
    report = install_w4a16(model, group_size=GROUP)
    assert report.replaced == 2 * 7 + 1
    assert report.by_kind == {"attention": 8, "mlp": 6, "lm_head": 1}
    assert report.skipped == []
    assert len(w4a16_modules(model)) == 15
    assert 3.0 < report.ratio < 4.0
    assert describe(model)["w4a16_modules"] == 15 and describe(model)["group_size"] == GROUP
    assert report.as_dict()["replaced"] == 15


def test_installed_layer_is_linear_over_its_own_dequantised_weight():
    model = _tiny_model()
    original = model.model.layers[0].mlp.down_proj.weight.detach().clone()
    install_w4a16(model, group_size=GROUP)
    shell = model.model.layers[0].mlp.down_proj
    assert isinstance(shell, W4A16Linear) and shell.loaded
    x = torch.randn(3, 5, shell.in_features)
    dequantised = unpack_w4_reference(shell.packed, shell.scales, shell.in_features, GROUP).float()
    with reference_mode(model):
        torch.testing.assert_close(shell(x), F.linear(x, dequantised), rtol=1e-5, atol=1e-5)
    error = (dequantised - original).abs().reshape(shell.out_features, -1, GROUP).amax(-1)
    assert torch.all(error <= shell.scales.float() / 2 * 1.01 + 1e-3)
    assert torch.equal(shell.dequantized(torch.float32), dequantised)


def test_non_cuda_forward_needs_reference_mode():
    model = _tiny_model()
    install_w4a16(model, group_size=GROUP)
    shell = model.model.layers[0].mlp.down_proj
    with pytest.raises(RuntimeError, match="CUDA"):
        shell(torch.randn(2, shell.in_features))
    empty = W4A16Linear(64, 32, group_size=32, device="meta")
    with pytest.raises(RuntimeError, match="no weights"):
        empty(torch.randn(2, 64))
    with pytest.raises(ValueError):
        W4A16Linear(100, 32)
    with pytest.raises(ValueError):
        shell.quantize_from(torch.zeros(3, 3))


def test_whole_model_runs_in_reference_mode_and_stays_the_same_model():
    model = _tiny_model()
    ids = torch.randint(0, 256, (2, 9))
    before = _logits(model, ids)
    install_w4a16(model, group_size=GROUP)
    with reference_mode(model):
        after = _logits(model, ids)
    assert after.shape == before.shape and torch.isfinite(after).all()
    assert torch.corrcoef(torch.stack([before.flatten(), after.flatten()]))[0, 1] > 0.9


def test_reference_mode_is_a_context_and_restores():
    model = _tiny_model()
    install_w4a16(model, group_size=GROUP)
    modules = w4a16_modules(model)
    modules[3].reference = True
    with reference_mode(model):
        assert all(m.reference for m in modules)
    assert [m.reference for m in modules] == [i == 3 for i in range(len(modules))]


def test_streaming_loader_matches_install_and_leaves_nothing_on_meta(tmp_path):
    model = _tiny_model(dtype=torch.float16)
    model.save_pretrained(tmp_path, safe_serialization=True)
    ids = torch.randint(0, 256, (1, 7))
    install_w4a16(model, group_size=GROUP)
    with reference_mode(model):
        expected = _logits(model.float(), ids)
    loaded, report = load_w4a16_model(str(tmp_path), device="cpu", group_size=GROUP)
    assert report.replaced == 15 and report.skipped == []
    assert not any(t.device.type == "meta" for t in (*loaded.parameters(), *loaded.buffers()))
    rotary = [m for m in loaded.modules() if hasattr(m, "inv_freq")]
    assert rotary and all(m.inv_freq.device.type == "cpu" for m in rotary)
    with reference_mode(loaded):
        torch.testing.assert_close(_logits(loaded.float(), ids), expected, rtol=1e-4, atol=1e-4)


def test_streaming_loader_quantises_a_tied_head_from_the_embedding(tmp_path):
    model = _tiny_model(tie=True)
    model.save_pretrained(tmp_path, safe_serialization=True)
    loaded, report = load_w4a16_model(str(tmp_path), device="cpu", group_size=GROUP)
    head = loaded.get_output_embeddings()
    assert isinstance(head, W4A16Linear) and head.loaded
    assert report.by_kind["lm_head"] == 1
    with reference_mode(loaded):
        assert torch.isfinite(_logits(loaded.float(), torch.randint(0, 256, (1, 5)))).all()


def test_group_size_that_does_not_divide_is_skipped_not_crashed():
    model = _tiny_model()
    report = install_w4a16(model, group_size=48)
    assert report.replaced == 0 and len(report.skipped) == 15


def test_int8_linear_tracks_fp32_linear_in_reference_mode(golden):
    torch.manual_seed(0)
    reference = nn.Linear(16, 8, bias=True, dtype=torch.float32)
    quantized = Int8Linear(reference)
    assert quantized.qweight.dtype is torch.int8 and quantized.scales.dtype is torch.float32
    assert np.array_equal(quantized.qweight.numpy(),
                          oracle.quantize_w8_int8linear(golden["int8linear_16x8.weight"])[0])
    quantized.reference = True
    inputs = torch.from_numpy(golden["int8linear_16x8.x"])
    out = quantized(inputs)
    assert torch.allclose(out, reference(inputs), atol=0.02, rtol=0.02)
    np.testing.assert_allclose(out.detach().numpy(), golden["int8linear_16x8.y"], rtol=1e-6, atol=1e-6)
    quantized.reference = False
    with pytest.raises(RuntimeError, match="CUDA"):
        quantized(inputs)


def test_recursive_int8_replacement_and_storage_accounting():
    model = nn.Sequential(nn.Linear(32, 16), nn.ReLU(), nn.Linear(16, 8)).to(torch.float16)
    before = model_storage_bytes(model)
    assert quantize_linear_modules(model) == 2
    assert not any(isinstance(m, nn.Linear) for m in model.modules())
    assert model_storage_bytes(model) < before
    tied = nn.ModuleList([nn.Linear(8, 8), nn.Linear(8, 8)])
    tied[1].weight = tied[0].weight
    assert model_storage_bytes(tied) == 8 * 8 * 4 + 2 * 8 * 4


def test_dense_scratch_bytes_covers_the_kernel_workspace_of_every_token_count():
    """Engines size their KV pool from this attribute (engine/continuous_batching.py:823-828):
    it must cover the deepest split-K workspace, which is not at the largest token count."""
    from full_inference_engine_b200 import _lib

    module = W4A16Linear(12288, 4096)
    worst = max(_lib.workspace_bytes(4, m, 4096, 12288) for m in (1, 16, 64, 256, 1024, 4096))
    assert module.dense_scratch_bytes >= worst
    assert module.dense_scratch_bytes % _lib.WORKSPACE_GRANULE == 0
    module.dense_scratch_bytes = 1 << 20            # the reference lets callers assign it
    assert module.dense_scratch_bytes == 1 << 20
    assert W4A16Linear(12288, 4096).dense_scratch_bytes >= worst
