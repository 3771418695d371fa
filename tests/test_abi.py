"""The C-ABI library: it loads, exports every symbol the header declares, and validates
arguments on the host before anything is launched (no GPU needed for any of this)."""

from __future__ import annotations

import os
import re

import pytest

from full_inference_engine_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions() -> list[str]:
    text = open(os.path.join(ROOT, "include", "b200q.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_what_the_binding_binds():
    assert _declared_functions() == sorted(_lib.exported_symbols())


def test_library_loads_and_exports_every_declared_symbol():
    lib = _lib.library()
    for name in _declared_functions():
        assert hasattr(lib, name), name
    assert lib.b200q_version() >= 100
    assert lib.b200q_status_string(0) == b"ok"
    assert b"workspace" in lib.b200q_status_string(_lib.ERR_WORKSPACE)


def test_workspace_bytes_is_pure_host_arithmetic():
    assert _lib.workspace_bytes(4, 0, 128, 128) == 0
    small = _lib.workspace_bytes(4, 4096, 12288, 4096)      # enough tiles: no split-K partials
    split = _lib.workspace_bytes(4, 16, 4096, 12288)        # few tiles: partials
    assert 0 < small < 1 << 20
    assert split > 16 * 4096 * 4
    assert _lib.workspace_bytes(7, 16, 128, 128) == 0        # unknown format


@pytest.mark.parametrize("call", ["w8", "w4"])
def test_forward_rejects_bad_arguments_before_launching(call):
    lib = _lib.library()
    before = _lib.launch_count()
    fake = 0x1000   # never dereferenced: validation fails first
    if call == "w8":
        bad_k = lib.b200q_w8a16_forward(fake, 24, _lib.F16, fake, 24, fake, _lib.F16, None,
                                        fake, 64, 4, 64, 24, None, 0, 0, None)
        assert bad_k == _lib.ERR_UNSUPPORTED                  # K % 16
        null = lib.b200q_w8a16_forward(None, 32, _lib.F16, fake, 32, fake, _lib.F16, None,
                                       fake, 64, 4, 64, 32, None, 0, 0, None)
        assert null == _lib.ERR_INVALID
        bad_dtype = lib.b200q_w8a16_forward(fake, 32, _lib.F32, fake, 32, fake, _lib.F16, None,
                                            fake, 64, 4, 64, 32, None, 0, 0, None)
        assert bad_dtype == _lib.ERR_INVALID
        no_ws = lib.b200q_w8a16_forward(fake, 128, _lib.F16, fake, 128, fake, _lib.F16, None,
                                        fake, 128, 64, 128, 128, None, 0, _lib.KERNEL_TC, None)
        assert no_ws == _lib.ERR_WORKSPACE
    else:
        bad_group = lib.b200q_w4a16_forward(fake, 256, _lib.F16, fake, 128, 0, fake, None, 100,
                                            None, fake, 64, 4, 64, 256, None, 0, 0, None)
        assert bad_group == _lib.ERR_INVALID                  # K % group
        odd_group = lib.b200q_w4a16_forward(fake, 240, _lib.F16, fake, 120, 0, fake, None, 48,
                                            None, fake, 64, 4, 64, 240, None, 0, 0, None)
        assert odd_group == _lib.ERR_UNSUPPORTED              # group % 32
        asym_without_zeros = lib.b200q_w4a16_forward(fake, 256, _lib.F16, fake, 128, 1, fake, None,
                                                     128, None, fake, 64, 4, 64, 256, None, 0, 0, None)
        assert asym_without_zeros == _lib.ERR_INVALID
        misaligned = lib.b200q_w4a16_forward(fake + 2, 256, _lib.F16, fake, 128, 0, fake, None, 128,
                                             None, fake, 64, 1, 64, 256, None, 0, _lib.KERNEL_SIMT, None)
        assert misaligned == _lib.ERR_ALIGNMENT
    assert _lib.launch_count() == before
    # empty problems are a no-op, not an error
    assert lib.b200q_w8a16_forward(None, 32, 0, None, 32, None, 0, None, None, 64, 0, 64, 32,
                                   None, 0, 0, None) == _lib.OK


def test_quantizers_reject_bad_geometry():
    lib = _lib.library()
    fake = 0x1000
    assert lib.b200q_quantize_w4_grouped(fake, _lib.F32, 100, 4, 100, 128, 0, fake, fake, None,
                                         None) == _lib.ERR_INVALID
    assert lib.b200q_quantize_w4_grouped(fake, _lib.F32, 128, 4, 128, 127, 0, fake, fake, None,
                                         None) == _lib.ERR_INVALID
    assert lib.b200q_quantize_w4_grouped(fake, _lib.F32, 128, 4, 128, 128, 1, fake, fake, None,
                                         None) == _lib.ERR_INVALID   # asym needs zeros
    assert lib.b200q_quantize_w8_per_channel(fake, _lib.F32, 8, 4, 16, 0, fake, fake,
                                             None) == _lib.ERR_INVALID   # ldw < K
    assert lib.b200q_w4_dequant(fake, fake, None, 1, 4, 128, 128, fake, 128, None) == _lib.ERR_INVALID


def test_cpu_tensors_are_refused_loudly():
    import torch

    from full_inference_engine_b200.kernels import w4a16_format, w4a16_linear, w8a16_linear

    with pytest.raises(RuntimeError, match="CUDA"):
        w4a16_format.quantize_weight_w4_grouped(torch.zeros(4, 128))
    with pytest.raises(RuntimeError, match="CUDA"):
        w8a16_linear.quantize_weight_per_channel(torch.zeros(4, 128))
    with pytest.raises(RuntimeError, match="CUDA"):
        w8a16_linear.w8a16_linear(torch.zeros(2, 32, dtype=torch.float16),
                                  torch.zeros(4, 32, dtype=torch.int8), torch.ones(4))
    with pytest.raises(RuntimeError, match="CUDA"):
        w4a16_linear.w4a16_linear(torch.zeros(2, 128, dtype=torch.float16),
                                  torch.zeros(4, 64, dtype=torch.uint8),
                                  torch.ones(4, 1, dtype=torch.float16))


def test_python_api_raises_the_reference_value_errors():
    import torch

    from full_inference_engine_b200.kernels import w4a16_format as w4
    from full_inference_engine_b200.kernels import w4a16_linear, w8a16_linear

    with pytest.raises(ValueError):
        w4.quantize_weight_w4_grouped(torch.zeros(4, 100), 128)
    with pytest.raises(ValueError):
        w4.quantize_weight_w4_grouped(torch.zeros(4, 128), 127)
    with pytest.raises(ValueError):
        w4.unpack_w4_reference(torch.zeros(4, 64, dtype=torch.int8), torch.ones(4, 1), 128)
    x = torch.zeros(2, 128, dtype=torch.float16)
    p = torch.zeros(4, 64, dtype=torch.uint8)
    s = torch.ones(4, 1, dtype=torch.float16)
    with pytest.raises(ValueError):
        w4a16_linear.w4a16_linear(x, p, s, kernel="bogus")
    with pytest.raises(ValueError):
        w4a16_linear.w4a16_linear(x, p, s, group_size=48)
    with pytest.raises(ValueError):
        w4a16_linear.w4a16_linear(x, p, torch.ones(4, 2, dtype=torch.float16))
    with pytest.raises(ValueError):
        w4a16_linear.w4a16_linear(x, p, s, torch.zeros(5))
    with pytest.raises(ValueError):
        w4a16_linear.w4a16_gemv(torch.zeros(4, 128, dtype=torch.float16), p, s)
    with pytest.raises(ValueError):
        w4a16_linear.w4_dequantize_into(torch.zeros(4, 128), p, s)
    with pytest.raises(ValueError):
        w8a16_linear.w8a16_linear(torch.zeros(2, 24, dtype=torch.float16),
                                  torch.zeros(4, 24, dtype=torch.int8), torch.ones(4))
    with pytest.raises(ValueError):
        w8a16_linear.w8a16_linear(x, torch.zeros(4, 128, dtype=torch.uint8), torch.ones(4))
    b = w4.weight_bytes(1024, 3072)
    assert b["fp16"] == 2 * 1024 * 3072 and b["w4a16"] * 3.5 < b["fp16"]
    assert b["w4a16_asym"] - b["w4a16"] == 2 * 3072 * 8
