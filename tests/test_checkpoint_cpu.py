"""Pre-quantized checkpoint round trip on CPU (the CUDA quantizer is swapped for the oracle):
what is written, that a load reproduces every buffer bit for bit without running a quantizer,
tied heads, and the error behaviour."""

from __future__ import annotations

import json
import os

import pytest
import torch

from full_inference_engine_b200.quantization import (
    W4A16Linear, install_w4a16, load_w4a16_checkpoint, reference_mode, save_w4a16_checkpoint,
)
from full_inference_engine_b200.quantization import checkpoint as ckpt
from full_inference_engine_b200.quantization import w4a16 as w4_mod
from oracle import wq_oracle as oracle

transformers = pytest.importorskip("transformers")
pytest.importorskip("safetensors")
GROUP = 32


@pytest.fixture(autouse=True)
def oracle_quantizer(monkeypatch):
    calls = {"n": 0}

    def w4(weight, group_size):
        calls["n"] += 1
        p, s = oracle.quantize_w4_grouped(weight.float().numpy(), group_size)
        return torch.from_numpy(p), torch.from_numpy(s)

    monkeypatch.setattr(w4_mod, "_quantize", w4)
    return calls


def _tiny(tie=False):
    from transformers import AutoModelForCausalLM, Qwen3Config

    torch.manual_seed(0)
    config = Qwen3Config(hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=256,
                         max_position_embeddings=128, tie_word_embeddings=tie)
    return AutoModelForCausalLM.from_config(config, dtype=torch.float32).eval()


def _logits(model, ids):
    with torch.no_grad(), reference_mode(model):
        return model(input_ids=ids, use_cache=False).logits


@pytest.mark.parametrize("tie", [False, True])
def test_round_trip_reproduces_every_buffer_and_runs_no_quantizer(tmp_path, oracle_quantizer, tie):
    model = _tiny(tie)
    install_w4a16(model, group_size=GROUP)
    ids = torch.randint(0, 256, (2, 9))
    expected = _logits(model, ids)
    meta = save_w4a16_checkpoint(model, str(tmp_path))
    assert meta["format"] == ckpt.FORMAT_TAG and meta["group_size"] == GROUP
    assert len(meta["modules"]) == 15
    assert {ckpt.META_FILE, "config.json", ckpt.WEIGHTS_FILE} <= set(os.listdir(tmp_path))
    quantizer_calls = oracle_quantizer["n"]

    loaded, report = load_w4a16_checkpoint(str(tmp_path), device="cpu", dtype=torch.float32)
    assert oracle_quantizer["n"] == quantizer_calls          # nothing was re-quantized
    assert report.replaced == 15 and report.by_kind == {"attention": 8, "mlp": 6, "lm_head": 1}
    ours = dict(model.named_modules())
    for name, module in loaded.named_modules():
        if isinstance(module, W4A16Linear):
            assert module.loaded and module.group_size == GROUP
            assert torch.equal(module.packed, ours[name].packed)
            assert torch.equal(module.scales, ours[name].scales)
    assert torch.equal(_logits(loaded, ids), expected)


def test_file_holds_packed_bytes_not_fp16_weights(tmp_path):
    from safetensors import safe_open

    model = _tiny()
    install_w4a16(model, group_size=GROUP)
    save_w4a16_checkpoint(model, str(tmp_path))
    with safe_open(os.path.join(tmp_path, ckpt.WEIGHTS_FILE), framework="pt") as f:
        keys = set(f.keys())
        assert "model.layers.0.mlp.down_proj.packed" in keys
        assert "model.layers.0.mlp.down_proj.scales" in keys
        assert not any(k.endswith("down_proj.weight") for k in keys)
        assert not any("rotary" in k for k in keys)
        packed = f.get_tensor("model.layers.0.mlp.down_proj.packed")
        assert packed.dtype is torch.uint8 and tuple(packed.shape) == (64, 64)


def test_errors(tmp_path):
    with pytest.raises(ValueError):
        save_w4a16_checkpoint(_tiny(), str(tmp_path / "plain"))          # nothing quantized
    with pytest.raises(FileNotFoundError):
        load_w4a16_checkpoint(str(tmp_path), device="cpu")               # no metadata
    model = _tiny()
    install_w4a16(model, group_size=GROUP)
    folder = str(tmp_path / "ok")
    save_w4a16_checkpoint(model, folder)
    meta_path = os.path.join(folder, ckpt.META_FILE)
    meta = json.load(open(meta_path))

    bad = dict(meta, format="something-else")
    json.dump(bad, open(meta_path, "w"))
    with pytest.raises(ValueError, match="unknown checkpoint format"):
        load_w4a16_checkpoint(folder, device="cpu")

    bad = json.loads(json.dumps(meta))
    bad["modules"]["model.layers.0.mlp.down_proj"]["in_features"] = 256
    json.dump(bad, open(meta_path, "w"))
    with pytest.raises(ValueError, match="down_proj"):
        load_w4a16_checkpoint(folder, device="cpu")

    bad = json.loads(json.dumps(meta))
    bad["modules"]["model.layers.7.mlp.down_proj"] = bad["modules"]["model.layers.0.mlp.down_proj"]
    json.dump(bad, open(meta_path, "w"))
    with pytest.raises(ValueError, match="does not have"):
        load_w4a16_checkpoint(folder, device="cpu")

    bad = json.loads(json.dumps(meta))
    del bad["modules"]["model.layers.0.mlp.down_proj"]                   # its packed tensor is now homeless
    json.dump(bad, open(meta_path, "w"))
    with pytest.raises(ValueError):
        load_w4a16_checkpoint(folder, device="cpu")
