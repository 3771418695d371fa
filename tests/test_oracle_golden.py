"""The CPU oracle against the reference: golden vectors and the reference tests' own KATs.

Every array in ``tests/golden/reference_vectors.npz`` was produced by the reference's code
(``tests/golden/make_golden.py``).  Integer and byte outputs must match bit for bit.
"""

from __future__ import annotations

import os

import numpy as np
import pytest
import torch

from oracle import cpu_path, wq_oracle as oracle

W4_CASES = ["w4_f32_s0", "w4_f16_s3", "w4_f16_g32", "w4_f32_g64", "w4_bf16_s9",
            "w4_exact_multiples", "w4_halfstep", "w4_degenerate"]
W8_CASES = ["w8_f32_s0", "w8_f16_s1", "w8_bf16_s2"]


@pytest.mark.parametrize("name", W4_CASES)
def test_w4_quantize_pack_matches_reference_bits(golden, name):
    _, n, k, g = (int(v) for v in golden[f"{name}.meta"])
    packed, scales = oracle.quantize_w4_grouped(golden[f"{name}.weight"], g)
    assert packed.dtype == np.uint8 and packed.shape == (n, k // 2)
    assert scales.dtype == np.float16 and scales.shape == (n, k // g)
    assert np.array_equal(packed, golden[f"{name}.packed"])
    assert np.array_equal(scales.view(np.uint16), golden[f"{name}.scales"].view(np.uint16))


@pytest.mark.parametrize("name", W4_CASES)
def test_w4_unpack_matches_reference_bits(golden, name):
    _, n, k, g = (int(v) for v in golden[f"{name}.meta"])
    deq = oracle.unpack_w4(golden[f"{name}.packed"], golden[f"{name}.scales"], k, g)
    assert deq.dtype == np.float16
    assert np.array_equal(deq.view(np.uint16), golden[f"{name}.dequant"].view(np.uint16))


def test_w4_split_half_known_answer():
    # tests/kernels/test_w4a16_linear.py:32-45 of the reference
    weight = np.zeros((1, 256), dtype=np.float32)
    weight[0, 5], weight[0, 5 + 64], weight[0, 0] = 7.0, -7.0, 7.0
    packed, scales = oracle.quantize_w4_grouped(weight, 128)
    assert float(scales[0, 0]) == pytest.approx(1.0)
    assert int(packed[0, 5]) & 0x0F == 15 and int(packed[0, 5]) >> 4 == 1
    assert int(packed[0, 64]) == 0x88


def test_w4_roundtrip_is_exact_for_in_range_integers(golden):
    # tests/kernels/test_w4a16_linear.py:18-29
    weight = golden["w4_exact_multiples.weight"]
    packed, scales = oracle.quantize_w4_grouped(weight, 128)
    restored = oracle.unpack_w4(packed, scales, 512, 128).astype(np.float32)
    np.testing.assert_allclose(restored, weight.astype(np.float16).astype(np.float32),
                               rtol=2e-3, atol=2e-3)


def test_w4_error_within_half_a_step(golden):
    # tests/kernels/test_w4a16_linear.py:48-56
    weight = golden["w4_halfstep.weight"]
    packed, scales = oracle.quantize_w4_grouped(weight, 128)
    restored = oracle.unpack_w4(packed, scales, 1024, 128).astype(np.float32)
    error = np.abs(restored - weight).reshape(8, 8, 128).max(axis=-1)
    assert np.all(error <= scales.astype(np.float32) / 2 * 1.01 + 1e-3)


def test_w4_rejects_untileable_shapes():
    # tests/kernels/test_w4a16_linear.py:59-63
    with pytest.raises(ValueError):
        oracle.quantize_w4_grouped(np.zeros((4, 100), np.float32), 128)
    with pytest.raises(ValueError):
        oracle.quantize_w4_grouped(np.zeros((4, 128), np.float32), 127)


def test_weight_bytes(golden):
    # tests/kernels/test_w4a16_linear.py:66-70
    b = oracle.weight_bytes(1024, 3072)
    assert [b["fp16"], b["w8a16"], b["w4a16"]] == list(golden["weight_bytes_1024_3072"])
    b = oracle.weight_bytes(4096, 12288, 64)
    assert [b["fp16"], b["w8a16"], b["w4a16"]] == list(golden["weight_bytes_4096_12288_g64"])
    b = oracle.weight_bytes(1024, 3072)
    assert b["fp16"] == 2 * 1024 * 3072 and b["w4a16"] * 3.5 < b["fp16"]


@pytest.mark.parametrize("name", W8_CASES + ["w8_degenerate"])
def test_w8_per_channel_matches_reference_bits(golden, name):
    q, s = oracle.quantize_w8_per_channel(golden[f"{name}.weight"])
    assert np.array_equal(q, golden[f"{name}.q"])
    assert np.array_equal(s.view(np.uint16), golden[f"{name}.scales"].view(np.uint16))


@pytest.mark.parametrize("name", W8_CASES)
def test_w8_int8linear_quantizer_matches_reference_bits(golden, name):
    q, s = oracle.quantize_w8_int8linear(golden[f"{name}.weight"])
    assert np.array_equal(q, golden[f"{name}.int8linear_q"])
    assert np.array_equal(s.view(np.uint32), golden[f"{name}.int8linear_scales"].view(np.uint32))


def test_int8linear_tracks_fp32_linear(golden):
    # tests/quantization/test_int8.py:7-12
    q, s = oracle.quantize_w8_int8linear(golden["int8linear_16x8.weight"])
    y = oracle.linear_fp32(golden["int8linear_16x8.x"], oracle.dequant_w8(q, s),
                           golden["int8linear_16x8.bias"])
    np.testing.assert_allclose(y, golden["int8linear_16x8.y"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(y, golden["int8linear_16x8.y_fp32_linear"], rtol=0.02, atol=0.02)


@pytest.mark.parametrize("tag,dtype", [("f16", torch.float16), ("bf16", torch.bfloat16)])
def test_cpu_path_port_reproduces_reference_modules(golden, tag, dtype):
    """The torch restatement bench.py times equals the reference modules' CPU output."""
    g = lambda key: torch.from_numpy(golden[key])  # noqa: E731
    q, s = oracle.quantize_w8_int8linear(golden[f"int8linear_fwd_{tag}.weight"])
    x = g(f"int8linear_fwd_{tag}.x").to(dtype)
    y = cpu_path.int8linear_forward(x, torch.from_numpy(q), torch.from_numpy(s),
                                    g(f"int8linear_fwd_{tag}.bias"))
    assert torch.equal(y.float(), g(f"int8linear_fwd_{tag}.y").float())
    # and the fp32 ground truth sits within the acceptance bar of it
    truth = oracle.linear_fp32(golden[f"int8linear_fwd_{tag}.x"], oracle.dequant_w8(q, s),
                               golden[f"int8linear_fwd_{tag}.bias"])
    ok, ratio = oracle.within_tolerance(y.float().numpy(), truth)
    assert ok, ratio

    x = g(f"w4a16linear_fwd_{tag}.x").to(dtype)
    y = cpu_path.w4a16_dense_forward(x, g(f"w4a16linear_fwd_{tag}.packed"),
                                     g(f"w4a16linear_fwd_{tag}.scales"),
                                     g(f"w4a16linear_fwd_{tag}.bias"))
    assert torch.equal(y.float(), g(f"w4a16linear_fwd_{tag}.y").float())
    packed, scales = oracle.quantize_w4_grouped(golden[f"w4a16linear_fwd_{tag}.weight"])
    assert np.array_equal(packed, golden[f"w4a16linear_fwd_{tag}.packed"])
    truth = oracle.linear_fp32(golden[f"w4a16linear_fwd_{tag}.x"],
                               oracle.unpack_w4(packed, scales, 256),
                               golden[f"w4a16linear_fwd_{tag}.bias"])
    ok, ratio = oracle.within_tolerance(y.float().numpy(), truth)
    assert ok, ratio


def test_asym_layout_roundtrip_and_nibble_order():
    """The asymmetric layout is this library's own (parity unpinned): self-consistency."""
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((8, 256)) * 0.02).astype(np.float32)
    packed, scales, zeros = oracle.quantize_w4_asym(w, 128)
    assert packed.dtype == np.int32 and packed.shape == (8, 32)
    assert scales.shape == zeros.shape == (8, 2)
    deq = oracle.unpack_w4_asym(packed, scales, zeros, 256, 128).astype(np.float32)
    err = np.abs(deq - w).reshape(8, 2, 128).max(axis=-1)
    assert np.all(err <= scales.astype(np.float32) / 2 * 1.01 + 1e-4)
    # input i of word j sits at nibble position (i & 1) * 4 + (i >> 1): one-hot check
    w = np.zeros((1, 128), np.float32)
    w[0, 9] = 1.5       # positive only -> lo = 0, zp = 0, scale = 0.1, q = 15
    packed, scales, zeros = oracle.quantize_w4_asym(w, 128)
    assert float(zeros[0, 0]) == 0.0
    assert int(packed.view(np.uint32)[0, 1]) == 15 << 16          # input 1 of word 1 -> position 4
    w[0, 9], w[0, 14] = 0.0, 1.5                                   # input 6 -> position 3
    assert int(oracle.quantize_w4_asym(w, 128)[0].view(np.uint32)[0, 1]) == 15 << 12
    t = torch.from_numpy
    assert torch.equal(cpu_path.unpack_w4_asym(t(packed), t(scales), t(zeros), 128),
                       t(oracle.unpack_w4_asym(packed, scales, zeros, 128)))


# --------------------------------------------------------------------------- W8A8
W8A8 = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_w8a8.npz"))
W8A8_CASES = sorted({key.split(".")[0] for key in W8A8.files})


@pytest.mark.parametrize("name", W8A8_CASES)
def test_w8a8_oracle_reproduces_the_reference_bit_for_bit(name):
    """The numpy restatement against outputs of the reference's w8a8_linear run on CPU tensors
    (engine/kernels/w8a8_linear.py:35-50)."""
    x, qweight, scales, y = (W8A8[f"{name}.{part}"] for part in ("x", "qweight", "scales", "y"))
    bf16 = bool(W8A8[f"{name}.meta"][4])
    got = oracle.w8a8_linear(x, qweight, scales, bf16=bf16, scalar_division="cpu")
    assert got.shape == y.shape
    assert np.array_equal(got.astype(np.float32), y.astype(np.float32))


def test_w8a8_row_quantiser_properties():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((7, 96)).astype(np.float16)
    x[3] = 0
    q, scales = oracle.quantize_rows_int8(x, "cpu")
    assert q.dtype == np.int8 and scales.dtype == np.float32
    assert np.abs(q).max() == 127 and not q[3].any()
    assert scales[3] == np.float32(1e-8) / np.float32(127.0)
    rows = np.abs(x.astype(np.float32)).max(axis=1)
    assert np.array_equal(scales[rows > 0], (rows[rows > 0] / np.float32(127.0)).astype(np.float32))
    # the CUDA rule multiplies by the rounded reciprocal: at most one ulp away, same integers almost always
    q_cuda, scales_cuda = oracle.quantize_rows_int8(x, "cuda")
    ulps = np.abs(scales.view(np.int32).astype(np.int64) - scales_cuda.view(np.int32).astype(np.int64))
    assert ulps.max() <= 1
    assert np.abs(q.astype(np.int16) - q_cuda.astype(np.int16)).max() <= 1


def test_bf16_rounding_helper_is_round_to_nearest_even():
    import torch
    values = np.random.default_rng(6).standard_normal(4096).astype(np.float32) * 1e3
    want = torch.from_numpy(values).to(torch.bfloat16).float().numpy()
    assert np.array_equal(oracle.round_to_bf16(values), want)
