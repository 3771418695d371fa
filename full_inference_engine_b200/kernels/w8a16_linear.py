"""INT8 per-channel weights x fp16/bf16 activations; mirrors ``engine/kernels/w8a16_linear.py``."""

from __future__ import annotations

import torch

from .. import _lib

_KERNELS = {"auto": _lib.KERNEL_AUTO, "gemv": _lib.KERNEL_SIMT, "dot": _lib.KERNEL_TC,
            "streamk": _lib.KERNEL_STREAMK}


def _quantize(weight: torch.Tensor, mode: int) -> tuple[torch.Tensor, torch.Tensor]:
    if weight.ndim != 2:
        raise ValueError("weight must be [out_features, in_features]")
    _lib.require_cuda(weight, "weight")
    w = weight.detach()
    if w.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        w = w.float()
    if w.stride(1) != 1:
        w = w.contiguous()
    n, k = w.shape
    q = torch.empty((n, k), dtype=torch.int8, device=w.device)
    scales = torch.empty((n,), device=w.device,
                         dtype=torch.float16 if mode == _lib.W8_SCALE_F16 else torch.float32)
    with torch.cuda.device(w.device):
        _lib.check(_lib.library().b200q_quantize_w8_per_channel(
            w.data_ptr(), _lib.dtype_enum(w.dtype), w.stride(0), n, k, mode,
            q.data_ptr(), scales.data_ptr(), _lib.stream_ptr(w.device)), "quantize_weight_per_channel")
    return q, scales


def quantize_weight_per_channel(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``[N, K]`` weights -> ``(int8 [N, K], fp16 scales [N])``.

    Bit-exact with the reference (engine/kernels/w8a16_linear.py:43-47): the scale is
    rounded to fp16 first and the division that quantises uses that rounded scale.
    """
    return _quantize(weight, _lib.W8_SCALE_F16)


def quantize_weight_per_channel_fp32_scales(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """The ``Int8Linear`` constructor's arithmetic (engine/quantization/int8.py:19-20): fp32 scales."""
    return _quantize(weight, _lib.W8_SCALE_F32)


def w8a16_linear(inputs: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor,
                 bias: torch.Tensor | None = None, *, kernel: str = "auto",
                 static_weights: bool = False, swiglu_pairs: bool = False,
                 _argmax: bool = False) -> torch.Tensor:
    """W8A16 linear for 2-D activations (engine/kernels/w8a16_linear.py:50-69).

    The integer weights enter the multiply unscaled (they are exact in fp16 and bf16);
    the per-channel scale and the bias are applied to the fp32 accumulator.
    ``static_weights`` and ``swiglu_pairs``: see ``w4a16_linear``.
    """
    if inputs.ndim != 2 or qweight.ndim != 2 or qweight.dtype is not torch.int8:
        raise ValueError("inputs must be 2D and qweight must be 2D INT8")
    m, k = inputs.shape
    n, weight_k = qweight.shape
    if weight_k != k or scales.shape != (n,) or (bias is not None and bias.shape != (n,)):
        raise ValueError("incompatible W8A16 linear geometry")
    if k % 32:
        raise ValueError("W8A16 kernel requires input width divisible by 32")
    if kernel not in _KERNELS:
        raise ValueError(f"kernel must be auto, gemv, dot or streamk; got {kernel!r}")
    if inputs.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("inputs must be fp16 or bf16")
    if swiglu_pairs and n % 2:
        raise ValueError("gate/up pairs need an even number of weight rows")
    _lib.require_cuda(inputs, "inputs")
    x = inputs if (inputs.stride(1) == 1 and inputs.stride(0) % 8 == 0
                   and inputs.data_ptr() % 16 == 0) else inputs.contiguous()
    w = qweight if qweight.is_contiguous() else qweight.contiguous()
    if scales.dtype not in (torch.float16, torch.float32):
        scales = scales.float()
    s = scales if scales.is_contiguous() else scales.contiguous()
    b = None
    if bias is not None:
        b = bias if (bias.dtype is inputs.dtype and bias.is_contiguous()) \
            else bias.to(inputs.dtype).contiguous()
    if _argmax:     # one channel index per row instead of the [M, N] outputs
        out = torch.empty((m,), dtype=torch.int64, device=inputs.device)
    else:
        out = torch.empty((m, n // 2 if swiglu_pairs else n), dtype=inputs.dtype, device=inputs.device)
    if m == 0 or n == 0:
        return out
    flags = (_lib.FLAG_STATIC_WEIGHTS if static_weights else 0) \
        | (_lib.FLAG_SWIGLU_PAIRS if swiglu_pairs else 0) | (_lib.FLAG_ARGMAX if _argmax else 0)
    ws = _lib.workspace_for(inputs.device, _lib.workspace_bytes(8, m, n, k))
    with torch.cuda.device(inputs.device):
        _lib.check(_lib.library().b200q_w8a16_forward(
            x.data_ptr(), x.stride(0), _lib.dtype_enum(x.dtype),
            w.data_ptr(), w.stride(0), s.data_ptr(), _lib.dtype_enum(s.dtype),
            None if b is None else b.data_ptr(),
            out.data_ptr(), out.stride(0), m, n, k,
            ws.data_ptr(), ws.numel(),
            _KERNELS[kernel] | flags,
            _lib.stream_ptr(inputs.device)),
            "w8a16_linear")
    return out
