"""True INT8 x INT8 linear on the tensor cores; mirrors ``engine/kernels/w8a8_linear.py``.

The reference quantises each activation row on the fly, multiplies in integers with
``torch._int_mm`` and rescales.  Here the row quantiser is one small kernel and the integer GEMM
is a tcgen05 ``kind::i8`` kernel that streams both int8 operands by TMA; the arithmetic (fp32
row maximum, IEEE division by 127, round-half-even, exact int32 sums, activation scale then
weight scale in fp32, one rounding to the activation dtype) is the reference's, so the result
is a deterministic function of the inputs.
"""

from __future__ import annotations

import torch

from .. import _lib


def pack_w8a8_weight(qweight: torch.Tensor) -> torch.Tensor:
    """``[out_features, in_features]`` INT8 weights -> the ``[in_features, out_features]`` operand
    ``w8a8_linear`` takes (engine/kernels/w8a8_linear.py:13-17).

    The reference copies into a transposed buffer because cuBLAS wants the weights that way.
    The kernel here reads K-major rows, so the packed operand is the transposed VIEW of the
    contiguous ``[N, K]`` matrix: same shape as the reference's, no second copy of the weights.
    """
    if qweight.ndim != 2 or qweight.dtype is not torch.int8:
        raise ValueError("qweight must be a 2D INT8 tensor")
    return qweight.contiguous().t()


def _k_major_rows(packed_weight: torch.Tensor) -> torch.Tensor:
    """The ``[N, K]`` row-major matrix behind a packed operand, 16-byte aligned rows."""
    rows = packed_weight.t()
    if rows.stride(1) != 1 or rows.stride(0) % 16 or rows.data_ptr() % 16:
        # an operand packed by the reference's function (a contiguous [K, N] copy), or a
        # width that is not a multiple of 16 bytes: repack (callers should pack once)
        n, k = rows.shape
        padded = torch.zeros((n, (k + 15) // 16 * 16), dtype=torch.int8, device=rows.device)
        padded[:, :k].copy_(rows)
        rows = padded[:, :k]
    return rows


def quantize_activations_per_row(inputs: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``[M, K]`` activations -> ``(int8 [M, K], fp32 scales [M])``, the reference's dynamic
    quantisation (engine/kernels/w8a8_linear.py:43-44).  The int8 rows are padded to a multiple
    of 16 bytes in memory (the returned tensor is the ``[:, :K]`` view)."""
    if inputs.ndim != 2:
        raise ValueError("inputs must be 2D")
    _lib.require_cuda(inputs, "inputs")
    x = inputs if inputs.dtype in (torch.float16, torch.bfloat16, torch.float32) else inputs.float()
    if x.stride(1) != 1:
        x = x.contiguous()
    m, k = x.shape
    ldq = (k + 15) // 16 * 16
    q = torch.empty((m, ldq), dtype=torch.int8, device=x.device)
    scales = torch.empty((m,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.library().b200q_quantize_rows_int8(
            x.data_ptr(), x.stride(0), _lib.dtype_enum(x.dtype), m, k, q.data_ptr(), ldq,
            scales.data_ptr(), _lib.stream_ptr(x.device)), "quantize_activations_per_row")
    return q[:, :k], scales


def w8a8_linear(inputs: torch.Tensor, packed_weight: torch.Tensor, weight_scales: torch.Tensor) -> torch.Tensor:
    """Dynamically quantise each input row, multiply in int8 on the tensor cores, dequantise
    (engine/kernels/w8a8_linear.py:35-50; same arguments, checks and error messages)."""
    if inputs.ndim != 2 or packed_weight.dtype is not torch.int8 or packed_weight.ndim != 2:
        raise ValueError("inputs must be 2D and packed_weight must be 2D INT8")
    _, width = inputs.shape
    weight_width, output_width = packed_weight.shape
    if weight_width != width or weight_scales.shape != (output_width,):
        raise ValueError("invalid W8A8 geometry")
    if inputs.device.type != "cuda" or packed_weight.device != inputs.device or weight_scales.device != inputs.device:
        raise ValueError("all W8A8 tensors must be on the same CUDA device")
    if inputs.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("inputs must be fp16 or bf16")
    if width % 16:
        raise ValueError("W8A8 kernel requires input width divisible by 16")
    qinputs, activation_scales = quantize_activations_per_row(inputs)
    return w8a8_linear_prequantized(qinputs, activation_scales, packed_weight, weight_scales, inputs.dtype)


def w8a8_linear_prequantized(qinputs: torch.Tensor, activation_scales: torch.Tensor, packed_weight: torch.Tensor,
                             weight_scales: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The integer GEMM and rescale alone, for callers that feed several projections from one
    quantised input (the reference recomputes the quantisation per call)."""
    rows = _k_major_rows(packed_weight)
    n, k = rows.shape
    m = qinputs.shape[0]
    if qinputs.shape != (m, k) or qinputs.dtype is not torch.int8 or activation_scales.shape != (m,):
        raise ValueError("invalid W8A8 geometry")
    if qinputs.stride(1) != 1 or qinputs.stride(0) % 16 or qinputs.data_ptr() % 16:
        raise ValueError("quantised activations must have 16-byte aligned rows")
    scales = weight_scales if weight_scales.dtype in (torch.float16, torch.float32) else weight_scales.float()
    scales = scales.contiguous()
    out = torch.empty((m, n), dtype=dtype, device=qinputs.device)
    with torch.cuda.device(qinputs.device):
        _lib.check(_lib.library().b200q_w8a8_forward(
            qinputs.data_ptr(), qinputs.stride(0), activation_scales.data_ptr(), rows.data_ptr(), rows.stride(0),
            scales.data_ptr(), _lib.dtype_enum(scales.dtype), out.data_ptr(), out.stride(0), _lib.dtype_enum(dtype),
            m, n, k, None, 0, _lib.stream_ptr(qinputs.device)), "w8a8_linear")
    return out
