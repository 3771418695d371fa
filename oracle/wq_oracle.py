"""CPU oracle for the weight-only quantized linear path.  TEST INFRASTRUCTURE ONLY.

A numpy restatement of the reference's algorithm (Vaibhav7711/full-inference-engine,
paths below relative to its root).  Only ``tests/``, ``__graft_entry__.smoke()`` and
``bench.py``'s CPU-baseline legs may import this module; the product package never does,
and it fails loudly when its CUDA library is missing rather than coming here.

Parity pin: every function that restates reference code is checked in
``tests/test_oracle_golden.py`` against (a) the known-answer bytes of the reference's own
tests (``tests/kernels/test_w4a16_linear.py:18-70``) and (b) golden vectors produced by
importing the reference itself (``tests/golden/make_golden.py`` holds the generator,
``tests/golden/*.npz`` its output).

The W8A8 functions are pinned by ``tests/golden/reference_w8a8.npz``: outputs of the
reference's own ``w8a8_linear`` executed on CPU tensors (``tests/golden/make_golden_w8a8.py``),
which the oracle reproduces bit for bit in its ``scalar_division="cpu"`` form.  The one step
where torch's CUDA arithmetic differs from its CPU arithmetic (tensor / Python scalar) is
checked on the GPU against the same torch expressions the reference evaluates.

The asymmetric 4-bit layout (``*_asym`` functions) has no counterpart in the reference:
**parity unpinned** for it.  Its definition is frozen here and in ``include/b200q.h``.

All arithmetic is IEEE: fp32 division (numpy ``/`` on float32), round-half-to-even
(``np.rint``), fp16 conversion by round-to-nearest-even (``astype(np.float16)``).
"""

from __future__ import annotations

import numpy as np

GROUP_SIZE = 128      # engine/kernels/w4a16_format.py:24
GEMV_MAX_ROWS = 3     # engine/kernels/w4a16_format.py:27
Q_MAX = 7.0           # engine/kernels/w4a16_format.py:28
OFFSET = 8            # engine/kernels/w4a16_format.py:29


def _nan_to_zero_int(values: np.ndarray, dtype) -> np.ndarray:
    """torch's CPU float->int conversion sends NaN to 0 (an all-zero W8 row is 0/0)."""
    cleaned = np.where(np.isnan(values), np.float32(0.0), values)
    return cleaned.astype(dtype)


# --------------------------------------------------------------------------- W8
def quantize_w8_per_channel(weight: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """engine/kernels/w8a16_linear.py:43-47 — int8 weights + fp16 scale per output row.

    The division that quantises uses the fp16-ROUNDED scale promoted back to fp32.
    """
    w = weight.astype(np.float32)
    s32 = np.maximum(np.abs(w).max(axis=1), np.float32(1e-8)) / np.float32(127.0)
    s16 = s32.astype(np.float16)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.rint(w / s16.astype(np.float32)[:, None])
    q = np.clip(q, -127.0, 127.0)          # clip keeps NaN
    return _nan_to_zero_int(q, np.int8), s16


def quantize_w8_int8linear(weight: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """engine/quantization/int8.py:19-20 — Int8Linear's constructor: fp32 scales."""
    w = weight.astype(np.float32)
    s32 = np.maximum(np.abs(w).max(axis=1), np.finfo(np.float32).eps) / np.float32(127.0)
    q = np.clip(np.rint(w / s32[:, None]), -127.0, 127.0)
    return _nan_to_zero_int(q, np.int8), s32.astype(np.float32)


def dequant_w8(q: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """fp32 dequantised weight used by the ground truth: q * scale."""
    return q.astype(np.float32) * scales.astype(np.float32)[:, None]


# --------------------------------------------------------------------------- W4 (reference layout)
def quantize_w4_grouped(weight: np.ndarray, group_size: int = GROUP_SIZE):
    """engine/kernels/w4a16_format.py:32-50 — symmetric [-7,7]+8, split-half packing."""
    if weight.ndim != 2:
        raise ValueError("weight must be [out_features, in_features]")
    n, k = weight.shape
    if group_size % 2 or k % group_size:
        raise ValueError(f"in_features {k} must be a multiple of an even group_size ({group_size})")
    groups, half = k // group_size, group_size // 2
    values = weight.astype(np.float32).reshape(n, groups, group_size)
    scales = np.maximum(np.abs(values).max(axis=-1), np.float32(1e-8)) / np.float32(Q_MAX)
    q = np.clip(np.rint(values / scales[..., None]), -Q_MAX, Q_MAX) + OFFSET
    q = q.astype(np.uint8)
    low, high = q[..., :half], q[..., half:]
    packed = (low | (high << 4)).reshape(n, groups * half)
    return np.ascontiguousarray(packed), np.ascontiguousarray(scales.astype(np.float16))


def unpack_w4(packed: np.ndarray, scales: np.ndarray, in_features: int,
              group_size: int = GROUP_SIZE) -> np.ndarray:
    """engine/kernels/w4a16_format.py:53-69 — fp16 [N,K]; the product is taken in fp16."""
    if packed.dtype != np.uint8:
        raise ValueError("packed weights must be uint8")
    n = packed.shape[0]
    groups, half = in_features // group_size, group_size // 2
    b = packed.reshape(n, groups, half)
    low = (b & 0x0F).astype(np.int8) - OFFSET
    high = (b >> 4).astype(np.int8) - OFFSET
    q = np.concatenate((low, high), axis=-1).astype(np.float16)
    # numpy multiplies float16 by converting to float32 and rounding the exact product
    # once, which is an fp16 multiply
    return (q * scales.astype(np.float16)[..., None]).reshape(n, in_features)


def weight_bytes(in_features: int, out_features: int, group_size: int = GROUP_SIZE) -> dict:
    """engine/kernels/w4a16_format.py:72-77."""
    return {
        "fp16": 2 * in_features * out_features,
        "w8a16": in_features * out_features + 2 * out_features,
        "w4a16": in_features * out_features // 2 + 2 * out_features * (in_features // group_size),
    }


# --------------------------------------------------------------------------- W4 asymmetric (no reference)
# nibble position of input i inside its int32 word
ASYM_POSITION = np.array([(i & 1) * 4 + (i >> 1) for i in range(8)])


def quantize_w4_asym(weight: np.ndarray, group_size: int = GROUP_SIZE):
    """Asymmetric 4-bit, fp16 scale + fp16 zero-point per group, 8 nibbles per int32.

    PARITY UNPINNED: the reference defines no such layout.  Per (row, group):
    lo=min(min w,0), hi=max(max w,0), s=max((hi-lo)/15,1e-8), zp=clip(rint(-lo/s),0,15),
    q=clip(rint(w/s)+zp,0,15); input i of a word sits at nibble position
    ``(i & 1) * 4 + (i >> 1)`` (positions 0..7 hold inputs 0,2,4,6,1,3,5,7).
    """
    if weight.ndim != 2:
        raise ValueError("weight must be [out_features, in_features]")
    n, k = weight.shape
    if group_size % 8 or k % group_size:
        raise ValueError("in_features must be a multiple of a group_size divisible by 8")
    groups = k // group_size
    v = weight.astype(np.float32).reshape(n, groups, group_size)
    lo = np.minimum(v.min(axis=-1), np.float32(0.0))
    hi = np.maximum(v.max(axis=-1), np.float32(0.0))
    s = np.maximum((hi - lo) / np.float32(15.0), np.float32(1e-8)).astype(np.float32)
    zp = np.clip(np.rint(-lo / s), 0.0, 15.0).astype(np.float32)
    q = np.clip(np.rint(v / s[..., None]) + zp[..., None], 0.0, 15.0).astype(np.uint32)
    q = q.reshape(n, k // 8, 8)
    shifts = (4 * ASYM_POSITION.astype(np.uint32))[None, None, :]
    words = np.bitwise_or.reduce(q << shifts, axis=-1).astype(np.uint32)
    return (np.ascontiguousarray(words.view(np.int32)), s.astype(np.float16), zp.astype(np.float16))


def unpack_w4_asym(packed: np.ndarray, scales: np.ndarray, zeros: np.ndarray, in_features: int,
                   group_size: int = GROUP_SIZE) -> np.ndarray:
    """fp16 [N,K]: fp16(nibble - zero) * fp16(scale), product in fp16."""
    n = packed.shape[0]
    words = packed.view(np.uint32).reshape(n, in_features // 8, 1)
    shifts = (4 * ASYM_POSITION.astype(np.uint32))[None, None, :]
    q = ((words >> shifts) & 0xF).reshape(n, in_features // group_size, group_size)
    centred = (q.astype(np.float32) - zeros.astype(np.float32)[..., None]).astype(np.float16)
    return (centred * scales.astype(np.float16)[..., None]).reshape(n, in_features)


# --------------------------------------------------------------------------- W8A8
def quantize_rows_int8(x: np.ndarray, scalar_division: str = "cuda") -> tuple[np.ndarray, np.ndarray]:
    """engine/kernels/w8a8_linear.py:43-44 — per-row dynamic activation quantisation:
    ``scale = amax(|x.float()|).clamp_min(1e-8) / 127.0`` and
    ``q = round(x.float() / scale).clamp(-127, 127).to(int8)``.  Returns (int8 [M,K], fp32 [M]).

    ``/ 127.0`` divides a tensor by a Python scalar.  torch's CUDA kernel evaluates that as a
    multiplication by the fp32 reciprocal (``scalar_division="cuda"``: the reference's
    arithmetic, since its function only accepts CUDA tensors); torch's CPU kernel divides
    (``"cpu"``: what the CPU-generated golden vectors hold).  The two scales differ by at most
    one ulp.  ``x / scale`` is tensor by tensor, an IEEE division on both devices."""
    if scalar_division not in ("cuda", "cpu"):
        raise ValueError("scalar_division must be 'cuda' or 'cpu'")
    x32 = x.astype(np.float32)
    peak = np.maximum(np.abs(x32).max(axis=1, keepdims=True), np.float32(1e-8)) if x32.shape[1] else \
        np.full((x32.shape[0], 1), 1e-8, np.float32)
    if scalar_division == "cuda":
        scales = (peak * (np.float32(1.0) / np.float32(127.0))).astype(np.float32)
    else:
        scales = (peak / np.float32(127.0)).astype(np.float32)
    q = np.clip(np.rint(x32 / scales), -127, 127).astype(np.int8)
    return q, scales[:, 0]


def round_to_bf16(values: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 by round-to-nearest-even, returned as the exactly representable fp32."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return rounded.view(np.float32)


def w8a8_linear(x: np.ndarray, qweight: np.ndarray, weight_scales: np.ndarray, bf16: bool = False,
                scalar_division: str = "cuda") -> np.ndarray:
    """engine/kernels/w8a8_linear.py:35-50 for ``qweight`` [N,K] int8 (the reference passes its
    transpose): exact integer sums, then ``(acc.float() * act_scale) * weight_scale.float()`` and
    one rounding to the activation dtype (fp16, or bf16 returned as fp32 values)."""
    q, a_scales = quantize_rows_int8(x, scalar_division)
    # float64 carries these sums exactly (every partial sum is an integer below 2**53)
    acc = (q.astype(np.float64) @ qweight.astype(np.float64).T).astype(np.int64)
    assert np.abs(acc).max(initial=0) < 2 ** 31
    y = (acc.astype(np.int32).astype(np.float32) * a_scales[:, None]) * weight_scales.astype(np.float32)[None, :]
    return round_to_bf16(y) if bf16 else y.astype(np.float16)


# --------------------------------------------------------------------------- ground truth
def linear_fp32(x: np.ndarray, w_deq: np.ndarray, bias: np.ndarray | None = None) -> np.ndarray:
    """fp32-accumulated ground truth: x.float() @ W.float().T (+ bias)."""
    y = x.astype(np.float32) @ w_deq.astype(np.float32).T
    if bias is not None:
        y = y + bias.astype(np.float32)[None, :]
    return y


def swiglu_fp32(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """``silu(gate) * up`` in fp32: the arithmetic of the reference's SwiGLU kernel
    (engine/kernels/swiglu.py:22-26, ``gate * sigmoid(gate) * up`` on fp32 promotions)."""
    g = gate.astype(np.float32)
    return g * (np.float32(1.0) / (np.float32(1.0) + np.exp(-g))) * up.astype(np.float32)


def interleave_rows(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """Rows gate[0], up[0], gate[1], up[1], ... (the fused gate/up weight order)."""
    return np.stack((gate, up), axis=1).reshape((2 * gate.shape[0],) + gate.shape[1:])


def within_tolerance(actual: np.ndarray, truth: np.ndarray, rel: float = 1e-2) -> tuple[bool, float]:
    """The acceptance bar: max|actual - truth| <= rel * max|truth|.  Returns (ok, ratio)."""
    denom = float(np.abs(truth).max())
    err = float(np.abs(actual.astype(np.float32) - truth).max())
    ratio = err / denom if denom > 0 else err
    return ratio <= rel, ratio
