"""ctypes binding of libb200q.so — the only bridge between Python and the CUDA kernels.

Nothing but raw pointers, sizes, enums and the current CUDA stream crosses this boundary
(see ``include/b200q.h``).  There is no CPU implementation behind it: if the library is
missing or a call fails, an exception says so.
"""

from __future__ import annotations

import ctypes
import os
import threading

import torch

PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PACKAGE_DIR, "lib", "libb200q.so")

# enums of include/b200q.h
F16, BF16, F32 = 0, 1, 2
W4_REF_SPLIT_HALF_SYM, W4_ASYM_ZP_INT32 = 0, 1
KERNEL_AUTO, KERNEL_SIMT, KERNEL_TC, KERNEL_STREAMK = 0, 1, 2, 3
FLAG_STATIC_WEIGHTS = 0x100
FLAG_SWIGLU_PAIRS = 0x200
FLAG_ARGMAX = 0x400
FLAG_GATHER_EPILOGUE = 0x800
FLAG_GATHER_PUSH = 0x1000
W8_SCALE_F16, W8_SCALE_F32 = 0, 1
OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_WORKSPACE, ERR_CUDA, ERR_DEVICE_WAIT = range(7)

_DTYPES = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}

_c_void_p, _c_int, _c_i64, _c_size = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t

_SIGNATURES = {
    "b200q_version": (_c_int, []),
    "b200q_status_string": (ctypes.c_char_p, [_c_int]),
    "b200q_launch_count": (ctypes.c_uint64, []),
    "b200q_last_error": (ctypes.c_char_p, []),
    "b200q_quantize_w8_per_channel": (_c_int, [_c_void_p, _c_int, _c_i64, _c_int, _c_int, _c_int,
                                               _c_void_p, _c_void_p, _c_void_p]),
    "b200q_quantize_rows_int8": (_c_int, [_c_void_p, _c_i64, _c_int, _c_int, _c_int, _c_void_p, _c_i64,
                                          _c_void_p, _c_void_p]),
    "b200q_w8a8_forward": (_c_int, [_c_void_p, _c_i64, _c_void_p, _c_void_p, _c_i64, _c_void_p, _c_int,
                                    _c_void_p, _c_i64, _c_int, _c_int, _c_int, _c_int,
                                    _c_void_p, _c_size, _c_void_p]),
    "b200q_quantize_w4_grouped": (_c_int, [_c_void_p, _c_int, _c_i64, _c_int, _c_int, _c_int, _c_int,
                                           _c_void_p, _c_void_p, _c_void_p, _c_void_p]),
    "b200q_w4_dequant": (_c_int, [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                                  _c_void_p, _c_i64, _c_void_p]),
    "b200q_workspace_bytes": (_c_size, [_c_int, _c_int, _c_int, _c_int]),
    "b200q_workspace_status": (_c_int, [_c_void_p, _c_void_p]),
    "b200q_describe_plan": (_c_int, [_c_int, _c_int, _c_int, _c_int, _c_int, _c_int, ctypes.c_char_p, _c_size]),
    "b200q_w8a16_forward": (_c_int, [_c_void_p, _c_i64, _c_int, _c_void_p, _c_i64, _c_void_p, _c_int,
                                     _c_void_p, _c_void_p, _c_i64, _c_int, _c_int, _c_int,
                                     _c_void_p, _c_size, _c_int, _c_void_p]),
    "b200q_w4a16_forward": (_c_int, [_c_void_p, _c_i64, _c_int, _c_void_p, _c_i64, _c_int, _c_void_p,
                                     _c_void_p, _c_int, _c_void_p, _c_void_p, _c_i64, _c_int, _c_int,
                                     _c_int, _c_void_p, _c_size, _c_int, _c_void_p]),
    "b200q_static_scratch_bytes": (_c_size, []),
    "b200q_w4a16_forward_static_scratch": (_c_int, [_c_void_p, _c_i64, _c_int, _c_void_p, _c_i64, _c_int,
                                                    _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                                    _c_i64, _c_int, _c_int, _c_int, _c_int, _c_void_p]),
}



class Gather(ctypes.Structure):
    """``b200q_gather`` of include/b200q.h: peer-mapped output and signal pointers of every rank."""

    _fields_ = [("rank", ctypes.c_int), ("world", ctypes.c_int),
                ("y_peer", ctypes.c_void_p * 8), ("signal_peer", ctypes.c_void_p * 8)]


_gather_p = ctypes.POINTER(Gather)
_SIGNATURES.update({
    "b200q_gather_tiles": (_c_int, [_c_int, _c_int, _c_int, _c_int, _c_int]),
    "b200q_gather_form": (_c_int, [_c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int]),
    "b200q_w4a16_forward_gather": (_c_int, [_c_void_p, _c_i64, _c_int, _c_void_p, _c_i64, _c_int, _c_void_p,
                                            _c_void_p, _c_int, _c_void_p, _gather_p, _c_i64, _c_int, _c_int,
                                            _c_int, _c_void_p, _c_size, _c_int, _c_void_p]),
    "b200q_w8a16_forward_gather": (_c_int, [_c_void_p, _c_i64, _c_int, _c_void_p, _c_i64, _c_void_p, _c_int,
                                            _c_void_p, _gather_p, _c_i64, _c_int, _c_int, _c_int,
                                            _c_void_p, _c_size, _c_int, _c_void_p]),
    "b200q_gather_wait": (_c_int, [_gather_p, _c_int, _c_void_p]),
})



class Reduce(ctypes.Structure):
    """``b200q_reduce`` of include/b200q.h: peer-mapped output, signal and inbox pointers."""

    _fields_ = [("rank", ctypes.c_int), ("world", ctypes.c_int), ("y_peer", ctypes.c_void_p * 8),
                ("signal_peer", ctypes.c_void_p * 8), ("inbox_peer", ctypes.c_void_p * 8)]


_reduce_p = ctypes.POINTER(Reduce)
_SIGNATURES.update({
    "b200q_reduce_tiles": (_c_int, [_c_int, _c_int, _c_int, _c_int, _c_int, _c_int]),
    "b200q_w4a16_forward_reduce": (_c_int, [_c_void_p, _c_i64, _c_int, _c_void_p, _c_i64, _c_int, _c_void_p,
                                            _c_void_p, _c_int, _c_void_p, _reduce_p, _c_i64, _c_int, _c_int,
                                            _c_int, _c_void_p, _c_size, _c_int, _c_void_p]),
    "b200q_w8a16_forward_reduce": (_c_int, [_c_void_p, _c_i64, _c_int, _c_void_p, _c_i64, _c_void_p, _c_int,
                                            _c_void_p, _reduce_p, _c_i64, _c_int, _c_int, _c_int,
                                            _c_void_p, _c_size, _c_int, _c_void_p]),
    "b200q_reduce_wait": (_c_int, [_reduce_p, _c_int, _c_void_p]),
})

_lib = None
_lock = threading.Lock()


class B200QError(RuntimeError):
    """A libb200q call returned a non-zero status."""

    def __init__(self, status: int, where: str):
        lib = library()
        text = lib.b200q_status_string(status).decode()
        detail = lib.b200q_last_error().decode()
        super().__init__(f"{where}: {text}" + (f" ({detail})" if detail else ""))
        self.status = status


def exported_symbols() -> list[str]:
    """Every entry point ``include/b200q.h`` declares."""
    return list(_SIGNATURES)


def library() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f"{LIB_PATH} is missing: build it with "
                        "`python -m full_inference_engine_b200.build` (needs nvcc). "
                        "This package has no CPU or PyTorch fallback for its kernels.")
                lib = ctypes.CDLL(LIB_PATH)
                for name, (restype, argtypes) in _SIGNATURES.items():
                    fn = getattr(lib, name)
                    fn.restype = restype
                    fn.argtypes = argtypes
                _lib = lib
    return _lib


def check(status: int, where: str) -> None:
    if status != OK:
        raise B200QError(status, where)


def dtype_enum(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {dtype}") from None


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(tensor: torch.Tensor, what: str) -> None:
    if tensor.device.type != "cuda":
        raise RuntimeError(
            f"{what} must be a CUDA tensor: the B200 kernels have no CPU path "
            "(use reference_mode / unpack_w4_reference for the torch arithmetic)")


# ------------------------------------------------------------------ workspace
# One zero-initialised buffer per device (the reference keeps its dequantise scratch the
# same way, engine/quantization/w4a16.py:59-76): split-K partials, tile counters and the
# status word.  Calls on one device are expected to be stream-ordered with one another, as
# they are under the reference's single worker thread; calls that overlap on the GPU from
# different streams would share the counters.  Grown only by allocating a larger buffer;
# earlier buffers stay alive because captured graphs may hold their addresses.
_WORKSPACES: dict[int, torch.Tensor] = {}
_RETIRED: list[torch.Tensor] = []
_GRANULE = 8 << 20
WORKSPACE_GRANULE = _GRANULE


def workspace_for(device: torch.device, nbytes: int) -> torch.Tensor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    buf = _WORKSPACES.get(key)
    if buf is None or buf.numel() < nbytes:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError(
                "the b200q workspace would have to grow during CUDA-graph capture: run the "
                "same call once eagerly on this device before capturing")
        size = max(_GRANULE, (nbytes + _GRANULE - 1) // _GRANULE * _GRANULE)
        if buf is not None:
            _RETIRED.append(buf)
        buf = torch.zeros(size, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = buf
    return buf


def workspace_bytes(fmt: int, m: int, n: int, k: int) -> int:
    return int(library().b200q_workspace_bytes(fmt, m, n, k))


def max_workspace_bytes(fmt: int, max_rows: int, n: int, k: int) -> int:
    """Largest workspace any token count up to ``max_rows`` needs for an [n, k] projection
    (split-K is deepest at middling token counts, so the largest M is not the worst case)."""
    rows = sorted({m for m in (1, 16, 32, 48, 64, 96, 128, 192, 256, 384, 512, 1024, 2048, 4096, 8192)
                   if m <= max_rows} | {max(1, max_rows)})
    return max(workspace_bytes(fmt, m, n, k) for m in rows)


def describe_plan(fmt: int, m: int, n: int, k: int, layout: int = W4_REF_SPLIT_HALF_SYM,
                  group: int = 128) -> str:
    """Kernel instantiation and tiling a plain forward of this geometry takes (diagnostic)."""
    buf = ctypes.create_string_buffer(256)
    check(library().b200q_describe_plan(fmt, layout, m, n, k, group, buf, len(buf)), "b200q_describe_plan")
    return buf.value.decode()


def launch_count() -> int:
    return int(library().b200q_launch_count())
