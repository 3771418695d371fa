"""Helpers shared by the GPU parity tests: seeded inputs and oracle ground truths."""

from __future__ import annotations

import numpy as np
import torch

from oracle import wq_oracle as oracle


def to_np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu()
    return t.float().numpy() if t.dtype is torch.bfloat16 else t.numpy()


def bits_equal(a: torch.Tensor, b: np.ndarray) -> bool:
    """Bitwise comparison of a device tensor with a numpy array of the same dtype/shape."""
    a = a.detach().cpu().contiguous().numpy()
    if a.shape != b.shape:
        return False
    if a.dtype == np.float16:
        return bool(np.array_equal(a.view(np.uint16), b.view(np.uint16)))
    if a.dtype == np.float32:
        return bool(np.array_equal(a.view(np.uint32), b.view(np.uint32)))
    return bool(np.array_equal(a, b))


def assert_within_bar(actual: torch.Tensor, truth: np.ndarray, rel: float = 1e-2) -> float:
    """max|actual - truth| <= rel * max|truth| (the acceptance bar, fp32 ground truth)."""
    ok, ratio = oracle.within_tolerance(to_np(actual).astype(np.float32), truth, rel)
    assert ok, f"max|err| / max|ref| = {ratio:.3e} exceeds {rel}"
    return ratio


def assert_close(actual: torch.Tensor, truth: np.ndarray, rtol: float, atol: float) -> None:
    a = to_np(actual).astype(np.float32)
    bad = np.abs(a - truth) > atol + rtol * np.abs(truth)
    assert not bad.any(), (f"{int(bad.sum())} of {bad.size} elements outside rtol={rtol} atol={atol}; "
                           f"worst |err|={float(np.abs(a - truth).max()):.4e}")


def seeded_case(shape, seed=None, dtype=torch.float16, weight_scale=1.0, bias=True):
    """(x, weight, bias) as CPU tensors, like the reference's kernel tests build them."""
    rows, width, outputs = shape
    torch.manual_seed(sum(shape) if seed is None else seed)
    x = torch.randn(rows, width).to(dtype)
    weight = (torch.randn(outputs, width) * weight_scale)
    b = torch.randn(outputs).to(dtype) if bias else None
    return x, weight, b
