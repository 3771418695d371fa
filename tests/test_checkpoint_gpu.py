"""A pre-quantized checkpoint written from an installed model loads onto the GPU with identical
buffers and gives identical logits through the kernels."""

from __future__ import annotations

import pytest
import torch

from full_inference_engine_b200.quantization import (
    W4A16Linear, install_w4a16, load_w4a16_checkpoint, save_w4a16_checkpoint,
)

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")


def test_saved_model_loads_on_the_gpu_and_matches(tmp_path):
    from transformers import AutoModelForCausalLM, Qwen3Config

    torch.manual_seed(0)
    config = Qwen3Config(hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=512,
                         max_position_embeddings=128, tie_word_embeddings=False)
    model = AutoModelForCausalLM.from_config(config, dtype=torch.float16).eval().cuda()
    install_w4a16(model)
    ids = torch.randint(0, 512, (2, 11), device="cuda")
    with torch.no_grad():
        expected = model(input_ids=ids, use_cache=False).logits
    save_w4a16_checkpoint(model, str(tmp_path))
    held = torch.cuda.memory_allocated()
    loaded, report = load_w4a16_checkpoint(str(tmp_path), device="cuda")
    assert report.replaced == 15
    grown = torch.cuda.memory_allocated() - held
    packed_bytes = sum(b.numel() * b.element_size() for b in loaded.buffers()) \
        + sum(p.numel() * p.element_size() for p in loaded.parameters())
    assert grown <= packed_bytes + (8 << 20)                 # no fp16 copy of any weight was made
    ours = dict(model.named_modules())
    for name, module in loaded.named_modules():
        if isinstance(module, W4A16Linear):
            assert module.packed.is_cuda and torch.equal(module.packed, ours[name].packed)
            assert torch.equal(module.scales, ours[name].scales)
    with torch.no_grad():
        actual = loaded(input_ids=ids, use_cache=False).logits
    assert torch.equal(actual, expected)
