"""Static checks over the CUDA sources, runnable without a GPU.

The analogue of the reference's tests/kernels/test_kernel_static_checks.py for hand-written
sm_100a code: failure classes that can be found by reading the source, and that would hang or
fault a GPU (or silently break the C-ABI contract) if they shipped.
"""

from __future__ import annotations

import pathlib
import re

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]
CSRC = ROOT / "full_inference_engine_b200" / "csrc"
SOURCES = sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")))
HEADER = ROOT / "include" / "b200q.h"


def _code(path: pathlib.Path) -> str:
    """The file without comments (block and line) and without string literals' contents."""
    text = path.read_text()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    return text


def _device_loops(code: str):
    """Bodies of `for (...)`/`while (...)` headers, as (header, position) pairs."""
    for match in re.finditer(r"\b(for|while)\s*\(([^;{}]*?(?:;[^;{}]*?;[^{}]*?)?)\)\s*\{?", code):
        yield match.group(0), match.start()


def test_sources_were_found():
    names = {p.name for p in SOURCES}
    assert {"gemm_tc.cu", "gemm_sk.cu", "gemm_i8.cu", "gemv_simt.cu", "quantize.cu", "api.cu", "ptx.cuh"} <= names


@pytest.mark.parametrize("path", SOURCES, ids=lambda p: p.name)
def test_no_allocation_synchronisation_or_host_readback_in_the_library(path):
    """The C ABI promises: no device allocation, no device-wide synchronisation, capturable.
    The one documented exception is b200q_workspace_status (a diagnostic)."""
    code = _code(path)
    for banned in ("cudaMalloc", "cudaFree", "cudaMallocAsync", "cudaHostAlloc", "cudaDeviceSynchronize",
                   "cudaDeviceReset"):
        assert banned not in code, f"{path.name} calls {banned}"
    assert not re.search(r"Memcpy\w*Batch", code), f"{path.name} calls a batched memcpy"
    syncs = len(re.findall(r"cudaStreamSynchronize", code))
    assert syncs == (1 if path.name == "api.cu" else 0), f"{path.name}: unexpected stream synchronisation"
    assert "cudaMemset(" not in code, f"{path.name}: a default-stream memset is not ordered with the caller's stream"


@pytest.mark.parametrize("path", SOURCES, ids=lambda p: p.name)
def test_no_multicast_loads_traps_or_device_asserts(path):
    code = _code(path)
    assert "multicast" not in code, f"{path.name}: a multicast copy or commit"
    for banned in ("__trap", "multimem", "wgmma", "nanosleep(0x7fffffff"):
        assert banned not in code, f"{path.name} contains {banned}"
    assert not re.search(r"(?<!static_)\bassert\(", code), f"{path.name} has a device-side assert"


@pytest.mark.parametrize("path", SOURCES, ids=lambda p: p.name)
def test_every_spin_wait_is_bounded(path):
    """Any loop that polls an mbarrier, a flag or a peer's signal must have an iteration
    limit: a `while (true)` / `for (;;)` / `while (!done)` poll can hang the GPU."""
    code = _code(path)
    assert not re.search(r"while\s*\(\s*(true|1)\s*\)", code), f"{path.name}: unbounded while"
    assert not re.search(r"for\s*\(\s*;\s*;\s*\)", code), f"{path.name}: unbounded for"
    # every try_wait / test_wait / acquire-load poll sits in a loop with an explicit bound, or
    # in a helper that does
    for name in ("mbar_try_wait", "ld_acquire_sys"):
        for use in re.finditer(rf"\b{name}\s*\(", code):
            before = code[:use.start()]
            # walk back to the enclosing function's start
            start = max(before.rfind("__device__"), before.rfind("__global__"))
            window = code[start:use.end()]
            if f"{name}(" in window.split("{")[0]:
                continue                      # this is the helper's own definition
            loops = re.findall(r"for\s*\(\s*(?:uint32_t|int|unsigned)\s+\w+\s*=\s*0\s*;\s*\w+\s*<\s*[^;]+;", window)
            assert loops, f"{path.name}: {name} outside a counted loop near offset {use.start()}"


def test_wait_helpers_have_the_documented_bounds():
    ptx = _code(CSRC / "ptx.cuh")
    assert re.search(r"kMaxPolls\s*=\s*1u\s*<<\s*22", ptx)
    assert re.search(r"for\s*\(uint32_t i = 0; i < kMaxPolls; \+\+i\)", ptx)
    common = _code(CSRC / "tc_common.cuh")
    assert re.search(r"for\s*\(uint32_t i = 0; i < kMaxPolls; \+\+i\)", common), "wait_or_abort lost its bound"
    assert re.search(r"for\s*\(uint32_t i = 0; i < \(1u << 22\); \+\+i\)", common), "poll_at_least lost its bound"


@pytest.mark.parametrize("name", ["gemm_tc.cu", "gemm_sk.cu", "gemm_i8.cu"])
def test_tensor_memory_is_always_released(name):
    """Every kernel that allocates TMEM frees it on its single exit path, after a block-wide
    barrier that every role reaches (no early `return` inside the kernel body)."""
    code = _code(CSRC / name)
    assert code.count("tmem_alloc(") == code.count("tmem_dealloc("), f"{name}: alloc/dealloc mismatch"
    for kernel in re.finditer(r"__global__ void[^{]*?(?:wq_gemm_\w+|w8a8_gemm)_kernel\([^)]*\)\s*\{", code, flags=re.S):
        depth, i = 1, kernel.end()
        while depth and i < len(code):
            depth += {"{": 1, "}": -1}.get(code[i], 0)
            i += 1
        body = code[kernel.end():i]
        assert "return;" not in body, f"{name}: early return inside a kernel that owns TMEM"
        tail = body[body.rfind("__syncthreads()"):]
        assert "tmem_dealloc(" in tail, f"{name}: TMEM is not freed after the final barrier"


@pytest.mark.parametrize("name", ["gemm_tc.cu", "gemm_sk.cu", "gemm_i8.cu"])
def test_tma_loads_start_on_16_byte_boundaries(name):
    """The innermost coordinate of every tiled load is the literal 0 (whole 64-byte / 128-byte
    rows) or a multiple of eight 2-byte elements (the scale chunks), and tile stores use a
    coordinate that is a multiple of the tile width."""
    code = _code(CSRC / name)
    loads = re.findall(r"tma_load_3d\(([^;]*?)\);", code, flags=re.S)
    assert loads, f"{name}: no TMA loads found"
    for args in loads:
        parts = [a.strip() for a in re.split(r",(?![^()]*\))", args)]
        assert parts[3] == "0" or re.fullmatch(r"\(\w+ >> 3\) \* 8|kb \* 128", parts[3]), \
            f"{name}: TMA load with inner coordinate {parts[3]!r}"
    for args in re.findall(r"tma_store_3d\(([^;]*?)\);", code, flags=re.S):
        parts = [a.strip() for a in re.split(r",(?![^()]*\))", args)]
        assert re.fullmatch(r"n_tile \* (tile_out|kBlockN)", parts[2]), f"{name}: TMA store inner coordinate {parts[2]!r}"


def test_header_symbols_match_the_binding_table():
    from full_inference_engine_b200 import _lib

    declared = set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", _code(HEADER)))
    bound = set(_lib.exported_symbols())
    assert declared == bound, f"header only: {sorted(declared - bound)}; binding only: {sorted(bound - declared)}"


def test_workspace_layout_constants_are_consistent():
    common = _code(CSRC / "tc_common.cuh")
    keys = int(re.search(r"kWsKeysOffset\s*=\s*(\d+)\s*\*\s*1024", common).group(1)) * 1024
    exchange = int(re.search(r"kWsExchangeOffset\s*=\s*(\d+)\s*\*\s*1024", common).group(1)) * 1024
    exchange_mib = int(re.search(r"kWsExchangeBytes\s*=\s*(\d+)\s*\*\s*1024\s*\*\s*1024", common).group(1))
    assert 256 < keys < exchange
    assert re.search(r"kWsPartialOffset\s*=\s*kWsExchangeOffset\s*\+\s*kWsExchangeBytes", common)
    # counters, keys, exchange words and partials never share an address: the layout the header documents
    header = HEADER.read_text()
    assert f"[256, {keys // 1024} KiB)" in header and f"[{keys // 1024} KiB, {exchange // 1024} KiB)" in header
    assert f"[{exchange // 1024} KiB, {exchange // 1024} KiB + {exchange_mib} MiB)" in header
    tile, stream = _code(CSRC / "gemm_tc.cu"), _code(CSRC / "gemm_sk.cu")
    assert "ws + kWsPartialOffset" in tile and "ws + kWsCountersOffset" in tile and "ws + kWsKeysOffset" in tile
    assert "ws + kWsExchangeOffset" in stream and "kWsPartialOffset" not in stream
