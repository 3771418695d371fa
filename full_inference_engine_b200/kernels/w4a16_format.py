"""The 4-bit weight formats: quantize + pack on the GPU, the torch reference dequantiser.

Mirrors ``engine/kernels/w4a16_format.py`` of the reference (same names, arguments and
errors).  ``quantize_weight_w4_grouped`` runs a CUDA kernel that is bit-exact against the
reference's torch arithmetic; ``unpack_w4_reference`` stays a plain torch function on
purpose — it is the arithmetic ``reference_mode`` compares the kernels with.

Reference layout ("split-half"): group of G inputs -> G/2 bytes, byte j = input j (low
nibble) | input j+G/2 (high nibble), values in [-7,7] stored +8, one fp16 scale per
(row, group).  A second, asymmetric layout (fp16 scale and zero-point, eight nibbles per
int32, pairs of K-neighbours 16 bits apart) is this library's own: ``quantize_weight_w4_asym``.
"""

from __future__ import annotations

import torch

from .. import _lib

GROUP_SIZE = 128
GEMV_MAX_ROWS = 3      # widest M the reference sends to its GEMV (engine/kernels/w4a16_format.py:27)
Q_MAX = 7.0
OFFSET = 8


def _check_weight(weight: torch.Tensor, group_size: int, divisor: int) -> tuple[int, int]:
    if weight.ndim != 2:
        raise ValueError("weight must be [out_features, in_features]")
    out_features, in_features = weight.shape
    if group_size <= 0 or group_size % divisor or in_features % group_size:
        raise ValueError(f"in_features {in_features} must be a multiple of an even group_size "
                         f"({group_size})")
    return out_features, in_features


def _as_kernel_input(weight: torch.Tensor) -> torch.Tensor:
    _lib.require_cuda(weight, "weight")
    w = weight.detach()
    if w.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        w = w.float()
    if w.stride(1) != 1:
        w = w.contiguous()
    return w


def quantize_weight_w4_grouped(weight: torch.Tensor, group_size: int = GROUP_SIZE,
                               ) -> tuple[torch.Tensor, torch.Tensor]:
    """``[N, K]`` weights -> ``(packed uint8 [N, K//2], scales fp16 [N, K//group])``.

    Bit-exact with the reference's ``quantize_weight_w4_grouped``
    (engine/kernels/w4a16_format.py:32-50) run on CPU.
    """
    n, k = _check_weight(weight, group_size, 2)
    w = _as_kernel_input(weight)
    packed = torch.empty((n, k // 2), dtype=torch.uint8, device=w.device)
    scales = torch.empty((n, k // group_size), dtype=torch.float16, device=w.device)
    with torch.cuda.device(w.device):
        _lib.check(_lib.library().b200q_quantize_w4_grouped(
            w.data_ptr(), _lib.dtype_enum(w.dtype), w.stride(0), n, k, group_size,
            _lib.W4_REF_SPLIT_HALF_SYM, packed.data_ptr(), scales.data_ptr(), None,
            _lib.stream_ptr(w.device)), "quantize_weight_w4_grouped")
    return packed, scales


def quantize_weight_w4_asym(weight: torch.Tensor, group_size: int = GROUP_SIZE,
                            ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``[N, K]`` -> ``(packed int32 [N, K//8], scales fp16, zeros fp16)``, both ``[N, K//group]``.

    Asymmetric 4-bit (no counterpart in the reference): per group ``lo=min(min w,0)``,
    ``hi=max(max w,0)``, ``s=max((hi-lo)/15,1e-8)``, ``zp=clamp(round(-lo/s),0,15)``,
    ``q=clamp(round(w/s)+zp,0,15)``; word ``j`` holds inputs ``8j..8j+7`` with input ``i`` at
    nibble position ``(i & 1) * 4 + (i >> 1)``.
    """
    n, k = _check_weight(weight, group_size, 8)
    w = _as_kernel_input(weight)
    packed = torch.empty((n, k // 8), dtype=torch.int32, device=w.device)
    scales = torch.empty((n, k // group_size), dtype=torch.float16, device=w.device)
    zeros = torch.empty_like(scales)
    with torch.cuda.device(w.device):
        _lib.check(_lib.library().b200q_quantize_w4_grouped(
            w.data_ptr(), _lib.dtype_enum(w.dtype), w.stride(0), n, k, group_size,
            _lib.W4_ASYM_ZP_INT32, packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
            _lib.stream_ptr(w.device)), "quantize_weight_w4_asym")
    return packed, scales, zeros


def unpack_w4_reference(packed: torch.Tensor, scales: torch.Tensor, in_features: int,
                        group_size: int = GROUP_SIZE) -> torch.Tensor:
    """Torch dequantiser: fp16 ``[N, K]`` with ``(nibble - 8) * scale`` taken in fp16.

    The arithmetic contract of the format (engine/kernels/w4a16_format.py:53-69); kept in
    torch so that ``reference_mode`` is independent of the CUDA kernels it checks.
    """
    if packed.dtype is not torch.uint8:
        raise ValueError("packed weights must be uint8")
    rows = packed.shape[0]
    half = group_size // 2
    tile = packed.reshape(rows, in_features // group_size, half)
    first = (tile & 0x0F).to(torch.int8) - OFFSET
    second = (tile >> 4).to(torch.int8) - OFFSET
    values = torch.cat((first, second), dim=-1).to(torch.float16)
    return (values * scales.to(torch.float16)[..., None]).reshape(rows, in_features)


def unpack_w4_asym_reference(packed: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                             in_features: int, group_size: int = GROUP_SIZE) -> torch.Tensor:
    """Torch dequantiser of the asymmetric layout: fp16 ``(nibble - zero) * scale``."""
    if packed.dtype is not torch.int32:
        raise ValueError("packed weights must be int32")
    rows = packed.shape[0]
    positions = [(i & 1) * 4 + (i >> 1) for i in range(8)]      # where input i sits in its word
    shifts = 4 * torch.tensor(positions, dtype=torch.int32, device=packed.device)
    nibbles = (packed.reshape(rows, in_features // 8, 1) >> shifts) & 0xF
    q = nibbles.reshape(rows, in_features // group_size, group_size).to(torch.float16)
    centred = q - zeros.to(torch.float16)[..., None]
    return (centred * scales.to(torch.float16)[..., None]).reshape(rows, in_features)


def weight_bytes(in_features: int, out_features: int, group_size: int = GROUP_SIZE) -> dict[str, int]:
    """Bytes one forward reads per projection, by format (engine/kernels/w4a16_format.py:72-77).

    ``w4a16_asym`` adds the fp16 zero-points of the asymmetric layout.
    """
    groups = in_features // group_size
    return {
        "fp16": 2 * in_features * out_features,
        "w8a16": in_features * out_features + 2 * out_features,
        "w4a16": in_features * out_features // 2 + 2 * out_features * groups,
        "w4a16_asym": in_features * out_features // 2 + 4 * out_features * groups,
    }
