"""Fused q/k/v projections on CPU (reference arithmetic; the CUDA quantizer is swapped for the
oracle, test infrastructure): the concatenated module's outputs are the parts' outputs bit for
bit, installing it on a model leaves the logits unchanged and counts every buffer once, and
uninstalling restores the three projections."""

from __future__ import annotations

import pytest
import torch
from torch import nn

from full_inference_engine_b200.quantization import int8 as int8_mod
from full_inference_engine_b200.quantization import w4a16 as w4_mod
from full_inference_engine_b200.quantization import (
    FusedProjections, Int8Linear, W4A16Linear, install_fused_qkv, install_w4a16,
    quantize_linear_modules, reference_mode, uninstall_fused_qkv, w4a16_modules,
)
from oracle import wq_oracle as oracle

transformers = pytest.importorskip("transformers")


@pytest.fixture(autouse=True)
def oracle_quantizers(monkeypatch):
    def w4(weight, group_size):
        p, s = oracle.quantize_w4_grouped(weight.float().numpy(), group_size)
        return torch.from_numpy(p), torch.from_numpy(s)

    def w8(weight):
        q, s = oracle.quantize_w8_int8linear(weight.float().numpy())
        return torch.from_numpy(q), torch.from_numpy(s)

    monkeypatch.setattr(w4_mod, "_quantize", w4)
    monkeypatch.setattr(int8_mod, "_quantize", w8)


def _model():
    from transformers import AutoModelForCausalLM, Qwen3Config

    cfg = Qwen3Config(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16, vocab_size=256, max_position_embeddings=128,
                      tie_word_embeddings=False)
    torch.manual_seed(0)
    return AutoModelForCausalLM.from_config(cfg, dtype=torch.float32).eval()


def _logits(model, ids):
    with torch.no_grad():
        return model(input_ids=ids, use_cache=False).logits


@pytest.mark.parametrize("kind", ["w4", "int8"])
def test_concatenated_rows_give_the_parts_outputs_bit_for_bit(kind):
    torch.manual_seed(1)
    sources = [nn.Linear(64, n, bias=True) for n in (64, 32, 32)]
    if kind == "w4":
        parts = []
        for src in sources:
            layer = W4A16Linear(64, src.out_features, group_size=32, bias=True)
            layer.quantize_from(src.weight.detach())
            layer.set_bias(src.bias.detach())
            layer.reference = True
            parts.append(layer)
    else:
        parts = [Int8Linear(src) for src in sources]
        for p in parts:
            p.reference = True
    fused = FusedProjections(parts)
    x = torch.randn(2, 5, 64)
    outs = fused(x)
    assert [o.shape[-1] for o in outs] == [64, 32, 32]
    for got, part in zip(outs, parts):
        assert torch.equal(got, part(x))
    # the views: one launch per distinct input, then columns of it
    assert torch.equal(fused.part(0, x), parts[0](x)) and fused._seen is not None
    assert torch.equal(fused.part(1, x), parts[1](x))
    assert torch.equal(fused.part(2, x), parts[2](x)) and fused._seen is None
    with pytest.raises(ValueError):
        FusedProjections([parts[0], nn.Linear(64, 8)])


def test_install_on_a_w4a16_model_keeps_the_logits_and_counts_buffers_once():
    model = _model()
    install_w4a16(model, group_size=32)
    ids = torch.randint(0, 256, (1, 7))
    with reference_mode(model):
        before = _logits(model, ids)
        bytes_before = sum(b.numel() * b.element_size() for b in model.buffers())
        assert install_fused_qkv(model) == 2
        assert install_fused_qkv(model) == 2                 # idempotent
    assert len(w4a16_modules(model)) == 15 - 2 * 2           # three projections became one, twice
    with reference_mode(model):
        after = _logits(model, ids)
    assert torch.equal(before, after)
    assert sum(b.numel() * b.element_size() for b in model.buffers()) == bytes_before
    assert uninstall_fused_qkv(model) == 2
    assert len(w4a16_modules(model)) == 15
    with reference_mode(model):
        assert torch.equal(_logits(model, ids), before)


def test_install_on_an_int8_model():
    model = _model()
    quantize_linear_modules(model)
    for m in model.modules():
        if isinstance(m, Int8Linear):
            m.reference = True
    ids = torch.randint(0, 256, (1, 5))
    before = _logits(model, ids)
    assert install_fused_qkv(model) == 2
    for m in model.modules():
        if isinstance(m, Int8Linear):
            m.reference = True
    assert torch.equal(_logits(model, ids), before)


def test_nothing_to_fuse_is_an_error():
    with pytest.raises(RuntimeError):
        install_fused_qkv(_model())
