"""Row-wise argmax fused into the projection kernel: identical to torch.max over the plain
projection's own output (same rounding, smallest channel on ties), and its winner is within the
acceptance bar of the oracle's fp32 maximum."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from full_inference_engine_b200 import _lib
from full_inference_engine_b200.kernels import argmax, w4a16_format as w4, w4a16_linear, w8a16_linear
from oracle import wq_oracle as oracle
from tests.helpers import to_np

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _check(channels, dense, truth=None):
    expect_i = dense.argmax(dim=-1)
    assert channels.dtype is torch.int64
    assert torch.equal(channels, expect_i), (channels.tolist(), expect_i.tolist())
    if truth is not None:
        top = truth.max(axis=1)
        picked = truth[np.arange(truth.shape[0]), channels.cpu().numpy()]
        assert np.all(top - picked <= 1e-2 * np.abs(truth).max())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 7, 16, 40, 200])
def test_w4_head_argmax(m, dtype):
    k, n = 1024, 40000 + 8                      # a vocabulary-sized head: hundreds of tiles, ragged last tile
    torch.manual_seed(m)
    packed, scales = w4.quantize_weight_w4_grouped(torch.randn(n, k, device=DEV) * 0.05)
    x = torch.randn(m, k, device=DEV).to(dtype)
    dense = w4a16_linear.w4a16_linear(x, packed, scales)
    channels = argmax.w4a16_linear_argmax(x, packed, scales)
    assert torch.equal(channels, argmax.w4a16_linear_argmax(x, packed, scales))   # keys were reset
    truth = oracle.linear_fp32(to_np(x).astype(np.float32), oracle.unpack_w4(to_np(packed), to_np(scales), k))
    _check(channels, dense, truth)


def test_small_matrix_that_would_otherwise_split_k():
    m, k, n = 5, 4096, 640                      # five tiles: the plain call splits K, the argmax call does not
    torch.manual_seed(0)
    qp = w4.quantize_weight_w4_asym(torch.randn(n, k, device=DEV) * 0.05)
    bias = torch.randn(n, device=DEV).half()
    x = torch.randn(m, k, device=DEV).half()
    channels = argmax.w4a16_linear_argmax(x, qp[0], qp[1], bias, zeros=qp[2])
    truth = oracle.linear_fp32(to_np(x).astype(np.float32),
                               oracle.unpack_w4_asym(*(to_np(t) for t in qp), k), to_np(bias))
    picked = truth[np.arange(m), channels.cpu().numpy()]
    assert np.all(truth.max(axis=1) - picked <= 1e-2 * np.abs(truth).max())
    # the plain (split-K) call afterwards still finds its counters and workspace clean
    dense = w4a16_linear.w4a16_linear(x, qp[0], qp[1], bias, zeros=qp[2])
    assert np.abs(dense.float().cpu().numpy() - truth).max() <= 1e-2 * np.abs(truth).max()


def test_ties_go_to_the_smallest_channel_and_negative_rows_work():
    k, n = 512, 384
    weight = torch.zeros(n, k, device=DEV)
    weight[:, 0] = -1.0                         # every channel gives the same negative output
    weight[200, 0] = weight[37, 0] = weight[300, 0] = -0.5   # three equal maxima
    q, s = w8a16_linear.quantize_weight_per_channel(weight)
    x = torch.zeros(3, k, device=DEV, dtype=torch.float16)
    x[:, 0] = torch.tensor([1.0, 2.0, 0.0])     # the last row is all zeros: a tie over every channel
    dense = w8a16_linear.w8a16_linear(x, q, s, kernel="dot")
    channels = argmax.w8a16_linear_argmax(x, q, s)
    _check(channels, dense)
    assert channels.tolist() == [37, 37, 0]


def test_errors():
    k, n = 512, 256
    p, s = w4.quantize_weight_w4_grouped(torch.randn(n, k, device=DEV) * 0.05)
    x = torch.randn(4, k, device=DEV).half()
    with pytest.raises(RuntimeError, match="unsupported"):
        w4a16_linear.w4a16_linear(x, p, s, kernel="gemv", _argmax=True)
    with pytest.raises(RuntimeError, match="unsupported"):
        w4a16_linear.w4a16_linear(x, p, s, swiglu_pairs=True, _argmax=True)


def test_module_argmax_matches_forward_argmax():
    from full_inference_engine_b200.quantization import W4A16Linear

    torch.manual_seed(3)
    head = W4A16Linear(512, 3000, device=DEV)
    head.quantize_from(torch.randn(3000, 512, device=DEV) * 0.05)
    x = torch.randn(2, 5, 512, device=DEV).half()
    assert torch.equal(head.argmax(x), head(x).argmax(dim=-1))
    head.reference = True
    assert head.argmax(x).shape == (2, 5)


EXCHANGE = slice(128 * 1024, 128 * 1024 + 5 * 1024 * 1024)     # the decode kernel's partial exchange
PARTIALS = slice(128 * 1024 + 5 * 1024 * 1024, None)           # the tile kernel's split-K partials


@pytest.mark.parametrize("m,k,n", [(16, 4096, 12288), (16, 12288, 4096), (144, 12288, 1024)])
def test_argmax_after_a_forward_that_left_partials_in_the_shared_workspace(m, k, n):
    """A decode step runs projections whose K is split (fp32 partials stay behind in the
    workspace) and then the head's argmax on the SAME workspace: the keys have a region of
    their own, so leftovers can never be taken for keys."""
    torch.manual_seed(1)
    device = torch.device("cuda", torch.cuda.current_device())
    packed, scales = w4.quantize_weight_w4_grouped(torch.randn(n, k, device=DEV) * 0.02)
    x = torch.randn(m, k, device=DEV).half()
    w4a16_linear.w4a16_linear(x, packed, scales)
    ws = _lib.workspace_for(device, 256)
    torch.cuda.synchronize()
    assert not bool(ws[EXCHANGE].any()), "the exchange region was not left empty"
    if "wq_gemm_sk_kernel" not in _lib.describe_plan(4, m, n, k):
        # the tile kernel's K split is too deep for a cluster here: fp32 partials stay behind
        assert bool(ws[PARTIALS].any()), "the split path did not go through the workspace"
    head_k, vocab = 1024, 5000
    hp, hs = w4.quantize_weight_w4_grouped(torch.randn(vocab, head_k, device=DEV) * 0.05)
    hx = torch.randn(m, head_k, device=DEV).half()
    dense = w4a16_linear.w4a16_linear(hx, hp, hs)
    channels = argmax.w4a16_linear_argmax(hx, hp, hs)
    truth = oracle.linear_fp32(to_np(hx).astype(np.float32), oracle.unpack_w4(to_np(hp), to_np(hs), head_k))
    _check(channels, dense, truth)
    assert int(channels.max()) < vocab


def test_whole_model_decode_step_then_head_argmax():
    """install_w4a16 on a two-layer Qwen3, one forward (its projections split K and leave
    partials in the shared workspace), then the quantized head's fused argmax over the final
    hidden states: equal to argmax over the model's own logits."""
    from transformers import AutoModelForCausalLM, Qwen3Config

    from full_inference_engine_b200.quantization import W4A16Linear, install_w4a16

    cfg = Qwen3Config(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=64, vocab_size=512, max_position_embeddings=256,
                      tie_word_embeddings=False)
    torch.manual_seed(0)
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float16).eval().cuda()
    install_w4a16(model, group_size=128)
    head = model.lm_head
    assert isinstance(head, W4A16Linear)
    for tokens in (1, 9, 80):
        ids = torch.randint(0, 512, (1, tokens), device=DEV)
        with torch.no_grad():
            hidden = model.model(input_ids=ids, use_cache=False).last_hidden_state
            logits = head(hidden)
            picked = head.argmax(hidden)
        assert torch.equal(picked, logits.argmax(dim=-1))
        assert int(picked.max()) < 512
