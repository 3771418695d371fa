"""INT4 weights x fp16/bf16 activations on B200; mirrors ``engine/kernels/w4a16_linear.py``.

Same function names, arguments and ``ValueError`` behaviour as the reference's Triton
module.  The Triton tile arguments (``block_m``, ``block_n``, ``block_k``, ``num_warps``)
are accepted and ignored.  ``kernel`` keeps the reference's vocabulary: ``"gemv"`` is the
CUDA-core split-K kernel, ``"dot"`` the tcgen05 tensor-core kernel, ``"auto"`` picks by M.
"""

from __future__ import annotations

import torch

from .. import _lib
from .w4a16_format import (  # noqa: F401  (re-exported like the reference module does)
    GEMV_MAX_ROWS, GROUP_SIZE, OFFSET, quantize_weight_w4_grouped,
)

_KERNELS = {"auto": _lib.KERNEL_AUTO, "gemv": _lib.KERNEL_SIMT, "dot": _lib.KERNEL_TC,
            "streamk": _lib.KERNEL_STREAMK}


def _forward(inputs, packed, scales, zeros, bias, group_size, kernel, where, static_weights=False,
             swiglu_pairs=False, argmax=False):
    _lib.require_cuda(inputs, "inputs")
    m, k = inputs.shape
    n = packed.shape[0]
    if inputs.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("inputs must be fp16 or bf16")
    x = inputs if (inputs.stride(1) == 1 and inputs.stride(0) % 8 == 0
                   and inputs.data_ptr() % 16 == 0) else inputs.contiguous()
    if x.stride(0) % 8 or x.data_ptr() % 16:
        raise ValueError("activation rows must be 16-byte aligned (K a multiple of 8)")
    w = packed if packed.is_contiguous() else packed.contiguous()
    s = scales if (scales.dtype is torch.float16 and scales.is_contiguous()) \
        else scales.to(torch.float16).contiguous()
    z = None
    if zeros is not None:
        z = zeros if (zeros.dtype is torch.float16 and zeros.is_contiguous()) \
            else zeros.to(torch.float16).contiguous()
    b = None
    if bias is not None:
        b = bias if (bias.dtype is inputs.dtype and bias.is_contiguous()) \
            else bias.to(inputs.dtype).contiguous()
    if argmax:      # one channel index per row instead of the [M, N] outputs
        out = torch.empty((m,), dtype=torch.int64, device=inputs.device)
    else:
        out = torch.empty((m, n // 2 if swiglu_pairs else n), dtype=inputs.dtype, device=inputs.device)
    if m == 0 or n == 0:
        return out
    flags = (_lib.FLAG_STATIC_WEIGHTS if static_weights else 0) \
        | (_lib.FLAG_SWIGLU_PAIRS if swiglu_pairs else 0) | (_lib.FLAG_ARGMAX if argmax else 0)
    need = _lib.workspace_bytes(4, m, n, k)
    ws = _lib.workspace_for(inputs.device, need)
    layout = _lib.W4_REF_SPLIT_HALF_SYM if zeros is None else _lib.W4_ASYM_ZP_INT32
    with torch.cuda.device(inputs.device):
        _lib.check(_lib.library().b200q_w4a16_forward(
            x.data_ptr(), x.stride(0), _lib.dtype_enum(x.dtype),
            w.data_ptr(), w.stride(0) * w.element_size(), layout,
            s.data_ptr(), None if z is None else z.data_ptr(), group_size,
            None if b is None else b.data_ptr(),
            out.data_ptr(), out.stride(0), m, n, k,
            ws.data_ptr(), ws.numel(), kernel | flags,
            _lib.stream_ptr(inputs.device)), where)
    return out


def w4a16_linear(inputs: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor,
                 bias: torch.Tensor | None = None, *, group_size: int = GROUP_SIZE,
                 block_m: int = 16, block_n: int = 64, num_warps: int = 4,
                 kernel: str = "auto", zeros: torch.Tensor | None = None,
                 static_weights: bool = False, swiglu_pairs: bool = False,
                 _argmax: bool = False) -> torch.Tensor:
    """``inputs [M, K]`` x dequantised ``packed/scales`` -> ``[M, N]`` in ``inputs.dtype``.

    Reference: ``w4a16_linear`` (engine/kernels/w4a16_linear.py:77-117).  With ``zeros``
    the weights are the asymmetric int32 layout (``packed`` is ``[N, K//8] int32``).
    ``static_weights=True`` promises that packed/scales/zeros/bias were not written by the
    kernel just before this call in the stream (module buffers): the kernel may then read
    them while that kernel is still finishing.  ``swiglu_pairs=True``: the rows are
    interleaved (gate, up) pairs and the result is ``silu(gate) * up``, ``[M, N // 2]``
    (see ``kernels/swiglu.py``).
    """
    asym = zeros is not None
    want = torch.int32 if asym else torch.uint8
    if inputs.ndim != 2 or packed.ndim != 2 or packed.dtype is not want:
        raise ValueError("inputs must be 2D fp16 and packed weights 2D uint8")
    if kernel not in _KERNELS:
        raise ValueError(f"kernel must be auto, gemv, dot or streamk; got {kernel!r}")
    m, k = inputs.shape
    n, packed_k = packed.shape
    if group_size % 32 or group_size < 32:
        raise ValueError("group_size must be a multiple of 32 (each half feeds a tl.dot)")
    if k % group_size or packed_k != (k // 8 if asym else k // 2):
        raise ValueError(f"packed width {packed_k} does not match K={k} with group {group_size}")
    if scales.shape != (n, k // group_size) or (asym and zeros.shape != scales.shape):
        raise ValueError("scales must have shape [N, K // group_size]")
    if bias is not None and bias.shape != (n,):
        raise ValueError("bias must have shape [N]")
    if block_m < 16 or block_n < 16:
        raise ValueError("tl.dot requires tiles of at least 16")
    if swiglu_pairs and n % 2:
        raise ValueError("gate/up pairs need an even number of weight rows")
    return _forward(inputs, packed, scales, zeros, bias, group_size, _KERNELS[kernel], "w4a16_linear",
                    static_weights, swiglu_pairs, _argmax)


def w4a16_gemv(inputs: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor,
               bias: torch.Tensor | None = None, *, group_size: int = GROUP_SIZE,
               block_n: int = 4, block_k: int = 1024, num_warps: int = 4,
               zeros: torch.Tensor | None = None) -> torch.Tensor:
    """The decode-width path, ``M <= GEMV_MAX_ROWS`` (engine/kernels/w4a16_linear.py:180-209)."""
    m, k = inputs.shape
    n = packed.shape[0]
    asym = zeros is not None
    if m > GEMV_MAX_ROWS:
        raise ValueError(f"w4a16_gemv serves M <= {GEMV_MAX_ROWS}; got {m}")
    if k % group_size or packed.shape != (n, k // 8 if asym else k // 2) \
            or scales.shape != (n, k // group_size):
        raise ValueError("packed/scales do not match inputs with this group size")
    block_k = min(block_k, k)
    if block_k % group_size or k % block_k:
        raise ValueError(f"block_k {block_k} must be a multiple of the group and divide K={k}")
    return _forward(inputs, packed, scales, zeros, bias, group_size, _lib.KERNEL_SIMT, "w4a16_gemv")


def w4_dequantize_into(out: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, *,
                       group_size: int = GROUP_SIZE, block_n: int = 32, num_warps: int = 4,
                       zeros: torch.Tensor | None = None) -> torch.Tensor:
    """Dequantise into caller-owned fp16 ``out [N, K]`` with one launch; returns ``out``.

    Bit-identical to ``unpack_w4_reference`` (engine/kernels/w4a16_linear.py:245-274).
    """
    n, k = out.shape
    asym = zeros is not None
    if out.dtype is not torch.float16 or packed.dtype is not (torch.int32 if asym else torch.uint8):
        raise ValueError("out must be fp16 and packed uint8")
    if group_size % 2 or k % group_size or packed.shape != (n, k // 8 if asym else k // 2):
        raise ValueError(f"packed {tuple(packed.shape)} does not match out {tuple(out.shape)} "
                         f"with group {group_size}")
    if scales.shape != (n, k // group_size):
        raise ValueError("scales must have shape [N, K // group_size]")
    _lib.require_cuda(out, "out")
    if out.stride(1) != 1:
        raise ValueError("out rows must be contiguous")
    w = packed if packed.is_contiguous() else packed.contiguous()
    s = scales if (scales.dtype is torch.float16 and scales.is_contiguous()) \
        else scales.to(torch.float16).contiguous()
    z = None if zeros is None else zeros.to(torch.float16).contiguous()
    with torch.cuda.device(out.device):
        _lib.check(_lib.library().b200q_w4_dequant(
            w.data_ptr(), s.data_ptr(), None if z is None else z.data_ptr(),
            _lib.W4_ASYM_ZP_INT32 if asym else _lib.W4_REF_SPLIT_HALF_SYM,
            n, k, group_size, out.data_ptr(), out.stride(0),
            _lib.stream_ptr(out.device)), "w4_dequantize_into")
    return out
