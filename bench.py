"""Benchmark of the weight-only quantized linear forward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload all|c1|c2|c3|c3fused|c4|c5|mlp|head|w8a8] [--layout asym|ref]

A *step* is one pass of the hot path over every case of the workload (one forward per
(format, shape, M) case) on synthetic seeded tensors.  The default workload ``all`` is the
union of the benchmark configurations 1, 2, 4 and 5: the single W8A16 case the reference runs
on CPU, the INT4 group-128 M-sweep at the Qwen3-8B MLP shapes (fp16), the W8A16 bf16 sweep
over the Qwen3-8B attention and MLP shapes, and the M=4096 INT4 prefill GEMM with outlier rows
(bf16) — 33 cases, M from 1 to 4096.  ``c1`` … ``c5`` select one configuration (``c3`` is the
graph-captured mixed step of 196 Qwen3-0.6B projections).

``value`` is algorithmic GB/s over the whole step with inputs resident in HBM (CUDA-graph
replay; every launch reads its own weight buffer and step variants alternate, so that every
weight byte comes from HBM, not L2).  ``e2e`` is the same metric through the Python module API
with activations in pinned host memory: host->device copy, forward, device->host copy of the
result, every step.  ``per_case`` lists every case with its own latency, GB/s, TFLOP/s, the
kernel instantiation that served it and its fraction of the roofline that bounds it;
``roofline`` aggregates the cases of the instantiation with the largest share of the step;
``roofline_by_regime`` aggregates the HBM-bound decode cases (M <= 16) and the tensor-bound
prefill cases (M >= 2048).  ``cpu_baseline`` times the reference's CPU path (dequantise to the
activation dtype + ``F.linear``) on the host cores in the same run, whole and split into its
dequantise and matmul halves.

At ``--gpus N`` (N > 1, under torchrun) every matrix is sharded along its output channels; the
line's ``phases`` give the sharded GEMMs alone, GEMM + all-gather fused into the kernel
epilogue, and GEMM + NCCL all-gather, per step and per case, and ``gather_parity`` compares
every case's gathered output with this rank's own single-GPU forward of the whole matrix.

With ``--impl reference`` only the CPU path runs (rank 0 only under torchrun).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC = "W8A16/INT4 GEMM TFLOP/s and HBM GB/s vs M (1-4096), Qwen3-8B shapes"
L2_BYTES = 126 << 20

# Qwen3-8B projections: name -> (K, N)
SHAPES_8B = {"q": (4096, 4096), "kv": (4096, 2048), "o": (4096, 4096),
             "gate_up": (4096, 12288), "down": (12288, 4096)}

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures
# summarised under profiles/; keyed like Case.key.  Absent = not captured.
NCU_TRAFFIC_BYTES: dict[str, float] = {
    "w4_asym:gate_up:M256": 28.91e6,     # profiles/wq_gemm_tc_int4_M256.md
    "w4_asym:down:M256": 33.11e6,        # profiles/wq_gemm_tc_int4_M256.md
    "w4_asym:gate_up:M4096": 139.2e6,    # profiles/wq_gemm_tc_int4_gate_up_M4096.md
}

WORKLOAD_TEXT = {
    "all": "configs 1,2,4,5: W8A16 M=8 1024->3072 fp16; INT4 g128 M in {1,4,16,64,256} at Qwen3-8B "
           "gate/up (4096->12288) and down (12288->4096), fp16; W8A16 bf16 at Qwen3-8B q/kv/o/gate_up/down, "
           "M in {1,16,64,512}; INT4 g128 prefill M=4096 bf16 with 1% outlier rows, gate/up and down",
    "c2": "config 2: INT4 g128 M-sweep {1,4,16,64,256} at Qwen3-8B gate/up (4096->12288) and down "
          "(12288->4096), fp16 activations",
    "c5": "config 5: INT4 g128 prefill M=4096 bf16 with 1% outlier rows, gate/up and down",
    "c4": "config 4: W8A16 bf16 at Qwen3-8B q/kv/o/gate_up/down, M in {1,16,64,512}",
    "c1": "config 1: W8A16 M=8 K=1024 N=3072 fp16",
    "head": "the Qwen3-8B output head, INT4 g128 4096 -> 151936 (the reference's largest matrix, "
            "benchmarks/kernels/w4a16_bench.py), M in {1,16,256}, fp16",
    "mlp": "beyond the reference: INT4 g128 gate_proj + up_proj + silu(gate) * up of a Qwen3-8B "
           "feed-forward (K=4096, 2 x 12288 interleaved rows) in one launch, M in {1,16,64,256,1024}, "
           "fp16; per_case carries the two-projections-plus-elementwise time beside it",
    "c3": "config 3: 28 x 7 random-init Qwen3-0.6B W8A16 projections, one mixed step of M=144 rows "
          "(16 decode + 128 prefill), fp16, one CUDA graph",
    "c3fused": "config 3 with q/k/v and gate/up of every layer concatenated along their output rows "
               "(FusedProjections): 28 x 4 W8A16 launches over the same weights, M=144, fp16, one CUDA graph",
}


class Case:
    def __init__(self, name, fmt, m, k, n, dtype, outliers=False, swiglu=False, cfg=""):
        self.name, self.fmt, self.m, self.k, self.n = name, fmt, m, k, n
        self.dtype, self.outliers = dtype, outliers
        # n rows are interleaved (gate, up) pairs and the output is silu(gate) * up, n / 2 wide
        self.swiglu = swiglu
        self.cfg = cfg

    @property
    def key(self):
        return f"{self.fmt}:{self.name}:M{self.m}"

    @property
    def wkey(self):
        return (self.fmt, self.name)

    @property
    def flops(self):
        return 2.0 * self.m * self.n * self.k

    def weight_bytes(self, fmt=None):
        fmt = fmt or self.fmt
        groups = self.k // 128
        if fmt == "w8":
            return self.n * self.k + 2 * self.n
        if fmt == "w4_ref":
            return self.n * self.k // 2 + 2 * self.n * groups
        return self.n * self.k // 2 + 4 * self.n * groups

    def algorithmic_bytes(self, fmt=None):
        """Every weight byte once, activations in, outputs out."""
        n_out = self.n // 2 if self.swiglu else self.n
        return float(self.weight_bytes(fmt) + 2 * self.m * self.k + 2 * self.m * n_out)

    @property
    def bytes(self):
        return self.algorithmic_bytes()

    def shard(self, world):
        return Case(self.name, self.fmt, self.m, self.k, self.n // world, self.dtype, self.outliers,
                    self.swiglu, self.cfg)


def build_cases(workload: str, layout: str) -> list[Case]:
    w4 = "w4_asym" if layout == "asym" else "w4_ref"
    if workload == "all":
        return [c for part in ("c1", "c2", "c4", "c5") for c in build_cases(part, layout)]
    if workload == "c2":
        return [Case(name, w4, m, *SHAPES_8B[name], torch.float16, cfg="c2")
                for name in ("gate_up", "down") for m in (1, 4, 16, 64, 256)]
    if workload == "c5":
        return [Case(name, w4, 4096, *SHAPES_8B[name], torch.bfloat16, outliers=True, cfg="c5")
                for name in ("gate_up", "down")]
    if workload == "c4":
        return [Case(name, "w8", m, *SHAPES_8B[name], torch.bfloat16, cfg="c4")
                for name in ("q", "kv", "o", "gate_up", "down") for m in (1, 16, 64, 512)]
    if workload == "c1":
        return [Case("gate_0p6b", "w8", 8, 1024, 3072, torch.float16, cfg="c1")]
    if workload == "head":
        # the reference's largest single matrix: the Qwen3-8B output head (4096 -> 151936)
        return [Case("lm_head", w4, m, 4096, 151936, torch.float16, cfg="head") for m in (1, 16, 256)]
    if workload == "mlp":
        # beyond the reference: gate_proj + up_proj + silu(gate) * up of a Qwen3-8B feed-forward
        # as ONE launch over interleaved quantized rows (2 x 12288 rows of K = 4096)
        k, n = SHAPES_8B["gate_up"]
        return [Case("gate_up_swiglu", w4, m, k, 2 * n, torch.float16, swiglu=True, cfg="mlp")
                for m in (1, 16, 64, 256, 1024)]
    if workload == "c3":
        # one mixed step of a Qwen3-0.6B-shaped model: 16 decode rows + one 128-token chunk
        shapes = {"q": (1024, 2048), "k": (1024, 1024), "v": (1024, 1024), "o": (2048, 1024),
                  "gate": (1024, 3072), "up": (1024, 3072), "down": (3072, 1024)}
        return [Case(f"L{layer:02d}.{name}", "w8", 144, k, n, torch.float16, cfg="c3")
                for layer in range(28) for name, (k, n) in shapes.items()]
    if workload == "c3fused":
        # the same step with the projections that read the same activations concatenated along
        # their output rows (q/k/v, gate/up): 4 launches per layer instead of 7, same weight bytes
        shapes = {"qkv": (1024, 4096), "o": (2048, 1024), "gate_up": (1024, 6144), "down": (3072, 1024)}
        return [Case(f"L{layer:02d}.{name}", "w8", 144, k, n, torch.float16, cfg="c3")
                for layer in range(28) for name, (k, n) in shapes.items()]
    raise SystemExit(f"unknown workload {workload}")


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            data = json.load(fh)
        return {"hbm_gbs": float(data["hbm_gbs"]), "tflops": float(data["bf16_tflops"]),
                "tflops_sustained": float(data.get("bf16_tflops_sustained", data["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


def roofline_of(total_bytes: float, total_flops: float, seconds: float, pk: dict) -> dict:
    """Roofline entry of one launch or of a group of launches (sums in, aggregate out)."""
    t_hbm = total_bytes / (pk["hbm_gbs"] * 1e9)
    t_tc = total_flops / (pk["tflops"] * 1e12)
    if t_hbm >= t_tc:
        achieved, peak, unit, bound = total_bytes / seconds / 1e9, pk["hbm_gbs"], "GB/s", "hbm"
    else:
        achieved, peak, unit, bound = total_flops / seconds / 1e12, pk["tflops"], "TFLOP/s", "tensor"
    return {"bound": bound, "achieved": round(achieved, 2), "peak": peak, "unit": unit,
            "frac": round(achieved / peak, 4), "peak_source": pk["source"]}


# --------------------------------------------------------------------------- clocks
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the GPU is under load."""

    def __init__(self, index: int, period: float = 0.005):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_flag = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.nv = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop_flag.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self) -> dict:
        self._stop_flag.set()
        if self.is_alive():
            self.join(timeout=1.0)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# --------------------------------------------------------------------------- inputs
def make_activation(case: Case, seed: int, device) -> torch.Tensor:
    gen = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(case.m, case.k, generator=gen)
    if case.outliers:      # 1% of rows scaled x20
        rows = torch.randperm(case.m, generator=gen)[: max(1, -(-case.m // 100))]
        x[rows] *= 20.0
    return x.to(case.dtype).to(device)


def quantize_for(case: Case, weight: torch.Tensor) -> tuple:
    from full_inference_engine_b200.kernels import w4a16_format as w4
    from full_inference_engine_b200.kernels import w8a16_linear

    if case.fmt == "w8":
        return w8a16_linear.quantize_weight_per_channel(weight)
    if case.fmt == "w4_ref":
        return w4.quantize_weight_w4_grouped(weight)
    return w4.quantize_weight_w4_asym(weight)


def make_weight_sets(cases: list[Case], copies_of: dict, device, rank: int = 0, world: int = 1,
                     keep_full: bool = False):
    """Quantized weights per (fmt, name): ``copies_of[key]`` distinct buffers each (L2 rotation).

    With world > 1 each rank keeps rows [rank*N/world, (rank+1)*N/world) of every matrix;
    ``keep_full`` also returns the whole quantized matrix per key (for the gather parity check).
    """
    sets: dict[tuple, list] = {}
    full: dict[tuple, tuple] = {}
    for case in cases:
        key = case.wkey
        if key in sets:
            continue
        gen = torch.Generator(device=device).manual_seed(1000 + len(sets))
        weight = torch.randn(case.n, case.k, generator=gen, device=device) * 0.02
        if keep_full and world > 1:
            full[key] = quantize_for(case, weight)
        rows = case.n // world
        first = quantize_for(case, weight[rank * rows:(rank + 1) * rows])
        del weight
        sets[key] = [first] + [tuple(t.clone() for t in first) for _ in range(copies_of[key] - 1)]
    return sets, full


def forward(case: Case, x: torch.Tensor, weights: tuple) -> torch.Tensor:
    from full_inference_engine_b200.kernels import w4a16_linear, w8a16_linear

    pairs = case.swiglu
    if case.fmt == "w8":
        return w8a16_linear.w8a16_linear(x, weights[0], weights[1], static_weights=True, swiglu_pairs=pairs)
    if case.fmt == "w4_ref":
        return w4a16_linear.w4a16_linear(x, weights[0], weights[1], static_weights=True, swiglu_pairs=pairs)
    return w4a16_linear.w4a16_linear(x, weights[0], weights[1], zeros=weights[2], static_weights=True,
                                     swiglu_pairs=pairs)


def unfused_forward(case: Case, x: torch.Tensor, halves: tuple) -> torch.Tensor:
    """What the fused gate/up + SwiGLU launch replaces: two projections and an elementwise
    kernel (the reference's route, engine/kernels/swiglu.py:65-83 without its fp16 fusion)."""
    from full_inference_engine_b200.kernels import swiglu

    plain = Case(case.name, case.fmt, case.m, case.k, case.n // 2, case.dtype)
    return swiglu.swiglu_reference(forward(plain, x, halves[0]), forward(plain, x, halves[1]))


def kernel_of(case: Case) -> str:
    """The kernel instantiation (and tiling) that serves this case on the current device."""
    from full_inference_engine_b200 import _lib

    layout = _lib.W4_ASYM_ZP_INT32 if case.fmt == "w4_asym" else _lib.W4_REF_SPLIT_HALF_SYM
    return _lib.describe_plan(8 if case.fmt == "w8" else 4, case.m, case.n, case.k, layout)


def time_graph(graph, reps: int, rounds: int = 7) -> float:
    """Median seconds per launch of a graph holding `reps` launches."""
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(rounds):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e) / reps)
    return statistics.median(times) * 1e-3


# --------------------------------------------------------------------------- CPU path
def cpu_fmt(case: Case) -> str:
    """The layout the reference's CPU path reads: its own split-half INT4, or int8."""
    return "w8" if case.fmt == "w8" else "w4_ref"


def cpu_inputs(cases: list[Case]):
    """Host tensors for the reference's CPU path (quantized with the CPU oracle)."""
    import numpy as np

    from oracle import wq_oracle as oracle

    weights, acts = {}, {}
    for i, case in enumerate(cases):
        key = case.wkey
        if key not in weights:
            gen = torch.Generator().manual_seed(1000 + len(weights))
            w = (torch.randn(case.n, case.k, generator=gen) * 0.02).numpy()
            if case.fmt == "w8":
                q, s = oracle.quantize_w8_per_channel(w)
                weights[key] = (torch.from_numpy(q), torch.from_numpy(s))
            else:     # the only INT4 layout the reference implements
                p, s = oracle.quantize_w4_grouped(w)
                weights[key] = (torch.from_numpy(np.ascontiguousarray(p)), torch.from_numpy(s))
        acts[i] = make_activation(case, 5000 + i, "cpu")
    return weights, acts


def cpu_step(cases, weights, acts):
    from oracle import cpu_path

    for i, case in enumerate(cases):
        w = weights[case.wkey]
        if case.swiglu:
            cpu_path.gate_up_swiglu_forward(acts[i], w[0], w[1], int8=case.fmt == "w8")
        elif case.fmt == "w8":
            cpu_path.int8linear_forward(acts[i], w[0], w[1])
        else:
            cpu_path.w4a16_dense_forward(acts[i], w[0], w[1])


def cpu_split(cases, weights, acts) -> dict:
    """Dequantise-only and matmul-only times of the CPU path, one representative case per
    format (the reference's own split, benchmarks/kernels/w4a16_bench.py:82-90)."""
    from torch.nn import functional as F

    from oracle import cpu_path

    out = {}
    for fmt in ("w4", "w8"):
        pick = [i for i, c in enumerate(cases) if (c.fmt == "w8") == (fmt == "w8") and not c.swiglu]
        if not pick:
            continue
        # the case closest to M = 16 of the widest matrix
        i = min(pick, key=lambda j: (-cases[j].n * cases[j].k, abs(cases[j].m - 16)))
        case, w, x = cases[i], weights[cases[i].wkey], acts[i]

        def dequant():
            if fmt == "w8":
                return w[0].to(dtype=x.dtype) * w[1].to(dtype=x.dtype)[:, None]
            return cpu_path.unpack_w4(w[0], w[1], case.k).to(x.dtype)

        dense = dequant()
        td, tm = [], []
        for _ in range(3):
            t0 = time.perf_counter()
            dequant()
            td.append(time.perf_counter() - t0)
            t0 = time.perf_counter()
            F.linear(x, dense)
            tm.append(time.perf_counter() - t0)
        out[fmt] = {"case": f"{cpu_fmt(case)}:{case.name}:M{case.m}",
                    "dequant_only_ms": round(statistics.median(td) * 1e3, 2),
                    "matmul_only_ms": round(statistics.median(tm) * 1e3, 2)}
    return out


def time_cpu(cases, budget_s: float = 20.0, min_steps: int = 2):
    """(seconds per step, steps timed, cores, sample description, split) on a bounded sample."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    weights, acts = cpu_inputs(cases)
    t0 = time.perf_counter()
    cpu_step(cases, weights, acts)                       # warm-up pass
    warm = time.perf_counter() - t0
    steps = max(min_steps, min(10, int(budget_s / max(warm, 1e-3))))
    if warm > budget_s:
        steps = 1
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_step(cases, weights, acts)
        times.append(time.perf_counter() - t0)
    sample = (f"all {len(cases)} cases of the workload, {steps} timed passes after 1 warm-up, "
              f"torch CPU ops on {cores} threads; INT4 cases use the reference's own "
              f"split-half layout (bytes counted for that layout)")
    return statistics.median(times), steps, cores, sample, cpu_split(cases, weights, acts)


def cpu_bytes(cases) -> float:
    return sum(c.algorithmic_bytes(cpu_fmt(c)) for c in cases)


# --------------------------------------------------------------------------- reference arm
def run_reference(args, cases):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    weights, acts = cpu_inputs(cases)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_step(cases, weights, acts)
    # bounded: never spend more than a few minutes however large --steps is
    t_budget, times = 150.0, []
    start = time.perf_counter()
    for _ in range(args.steps):
        t0 = time.perf_counter()
        cpu_step(cases, weights, acts)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - start > t_budget:
            break
    sec = sum(times) / len(times)
    total_bytes = cpu_bytes(cases)
    total_flops = sum(c.flops for c in cases)
    value = total_bytes / sec / 1e9
    sample = (f"{len(times)} of {args.steps} requested passes over all {len(cases)} cases "
              f"(bounded to {t_budget:.0f} s), torch CPU dequantise + F.linear on {cores} threads; "
              "the oracle's port of the reference CPU path (the reference tree is not on this box); "
              "INT4 in the reference's split-half layout, bytes counted for that layout")
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": "GB/s",
        "tflops": round(total_flops / sec / 1e12, 5), "n_gpus": args.gpus, "steps": len(times),
        "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16/bf16 activations, fp32 accumulate",
        "data": "synthetic", "config": config_dict(args, cases),
        "cpu_baseline": {"value": round(value, 4), "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": sample, "split": cpu_split(cases, weights, acts)},
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def config_dict(args, cases):
    """The same dictionary on both arms: it names the work, not how an arm ran it."""
    int4 = any(c.fmt != "w8" for c in cases)
    return {
        "workload": WORKLOAD_TEXT[args.workload],
        "layout": ("INT4: the B200 arm reads "
                   + ("the asymmetric layout (int32 x8 nibbles + fp16 scale and zero-point)"
                      if args.layout == "asym" else "the reference's split-half uint8 + fp16 scale layout")
                   + "; the reference arm always reads the reference's split-half layout (its only one)"
                   if int4 else "") + ("; " if int4 and any(c.fmt == "w8" for c in cases) else "")
        + ("W8: int8 per-channel, fp16 scale" if any(c.fmt == "w8" for c in cases) else ""),
        "cases": len(cases),
        "parallelism": (f"N-sharded x{args.gpus}, all-gather "
                        + {"fused": "by this library's own kernels (peer stores over NVLink, no NCCL): from the "
                                    "GEMM kernel's epilogue, or by a push kernel where a rank has few large tiles",
                           "epilogue": "fused into the GEMM kernel's epilogue (peer stores over NVLink)",
                           "push": "by this library's push kernel after the GEMM (peer stores over NVLink)",
                           "nccl": "by NCCL"}[args.gather]) if args.gpus > 1 else "single GPU",
        "l2": "inputs larger than L2: every launch reads its own weight buffer and step variants "
              "alternate, so that at least 2 x 126 MiB of distinct weights pass between two uses of a buffer",
    }


# --------------------------------------------------------------------------- B200 arm
def run_b200(args, cases):
    import torch.distributed as dist

    from full_inference_engine_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    cpu_group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        # barriers and the max-over-ranks of the timings go over a gloo side group, so that
        # the only NCCL work in the run is the all-gather being measured
        cpu_group = dist.new_group(backend="gloo")

    def max_over_ranks(value: float) -> float:
        if world == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=cpu_group)
        return float(t.item())

    def barrier():
        if world > 1:
            torch.cuda.synchronize()
            dist.barrier(group=cpu_group)

    def note(msg):
        if args.verbose:
            print(f"# rank {rank}: {msg}", file=sys.stderr, flush=True)

    pk = peaks()
    local_cases = [c.shard(world) for c in cases]
    # Every case of a step reads its own buffer of its matrix; `variants` step variants use
    # disjoint buffers, enough of them that >= 2 x L2 of distinct weights pass between two uses
    # of the same buffer.
    uses: dict[tuple, int] = {}
    use_index = []
    for c in local_cases:
        use_index.append(uses.get(c.wkey, 0))
        uses[c.wkey] = use_index[-1] + 1
    step_weight_bytes = sum(c.weight_bytes() for c in local_cases)
    variants = max(2, min(96, -(-2 * L2_BYTES // step_weight_bytes)))
    if args.workload in ("c3", "c3fused"):
        variants = 1          # 196 distinct matrices, 600 MB per step
    copies_of = {key: n * variants for key, n in uses.items()}
    weight_sets, full_sets = make_weight_sets(cases, copies_of, device, rank, world, keep_full=True)
    acts = [make_activation(c, 5000 + i, device) for i, c in enumerate(cases)]

    def weights_of(i, variant):
        case = local_cases[i]
        return weight_sets[case.wkey][use_index[i] + variant * uses[case.wkey]]

    gathered = [torch.empty(world, c.m, c.n // world, dtype=c.dtype, device=device) if world > 1 else None
                for c in cases]
    # fused all-gather: full [M, N] outputs in symmetric memory, written by every rank's epilogue
    fused_out = None
    if world > 1:
        from full_inference_engine_b200.quantization.sharded import SymmetricOutput

        fused_out = [SymmetricOutput(c.m, c.n, c.dtype, device) for c in cases]

    def forward_gather(i, case, x, w, how):
        """This rank's columns of case i delivered to every rank; returns the full [M, N] view."""
        if how in ("fused", "epilogue", "push"):
            from full_inference_engine_b200.quantization.sharded import fused_forward_gather

            form = "auto" if how == "fused" else how
            if case.fmt == "w8":
                ok = fused_forward_gather(x, fused_out[i], qweight=w[0], scales=w[1], form=form)
            elif case.fmt == "w4_ref":
                ok = fused_forward_gather(x, fused_out[i], packed=w[0], scales=w[1], form=form)
            else:
                ok = fused_forward_gather(x, fused_out[i], packed=w[0], scales=w[1], zeros=w[2], form=form)
            if ok:
                return fused_out[i].tensor
        y = forward(case, x, w)
        dist.all_gather_into_tensor(gathered[i], y)
        return gathered[i].permute(1, 0, 2).reshape(case.m, -1)

    def one_step(variant: int, how: str):
        """how: "local" (this rank's GEMMs only); GEMM + all-gather: "fused" (this library's own
        exchange over peer memory, form picked per geometry), "epilogue" (always from the GEMM's
        epilogue), "push" (always forward + push kernel) or "nccl"."""
        outs = []
        for i, case in enumerate(local_cases):
            w = weights_of(i, variant)
            if world > 1 and how != "local":
                outs.append(forward_gather(i, case, acts[i], w, how))
            else:
                outs.append(forward(case, acts[i], w))
        return outs

    default_how = "local" if world == 1 else args.gather

    # eager warm-up (also sizes the workspace)
    note("inputs ready")
    for v in range(variants):
        one_step(v, default_how)
    torch.cuda.synchronize()
    note("eager warm-up done")

    # ---- multi-rank only: every case's gathered output against this rank's own single-GPU
    # forward of the whole matrix, once, outside every timed region
    gather_parity = None
    if world > 1:
        worst, bad = 0.0, []
        for how in ("fused", "epilogue", "push", "nccl"):
            for i, case in enumerate(local_cases):
                got = forward_gather(i, case, acts[i], weights_of(i, 0), how).float()
                want = forward(cases[i], acts[i], full_sets[cases[i].wkey]).float()
                rel = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
                worst = max(worst, rel)
                if not rel <= 1e-2:
                    bad.append(f"{how}:{cases[i].key}:{rel:.3e}")
                torch.cuda.synchronize()
        flag = torch.tensor([worst, float(len(bad))], dtype=torch.float64)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=cpu_group)
        gather_parity = {"max_rel_err": float(flag[0]), "ok": float(flag[1]) == 0.0,
                         "cases": 4 * len(cases), "bar": 1e-2,
                         "against": "this rank's single-GPU forward of the whole matrix",
                         "failed_on_rank0": bad}
        del full_sets
        note(f"gather parity: {gather_parity}")

    # ---- end to end (measured before any graph holds NCCL work): pinned host activations in,
    # host results out, through the public API
    host_x = [torch.empty(c.m, c.k, dtype=c.dtype).pin_memory().copy_(acts[i].cpu()) for i, c in enumerate(cases)]
    host_y = [torch.empty(c.m, c.n // (2 if c.swiglu else 1), dtype=c.dtype).pin_memory() for c in cases]
    dev_x = [torch.empty_like(a) for a in acts]

    # Three streams per step: activations in, projections, results out.  A projection waits only
    # for its own activations and its result starts back as soon as it exists, so the two copy
    # directions (PCIe is full duplex) and the kernels overlap.  Order: outputs-heavy cases first,
    # inputs-heavy ones last, so that late uploads overlap early downloads.
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    e2e_order = sorted(range(len(local_cases)),
                       key=lambda i: (local_cases[i].k - local_cases[i].n) * local_cases[i].m)

    def e2e_enqueue(variant):
        main = torch.cuda.current_stream()
        copy_in.wait_stream(main)
        copy_out.wait_stream(main)
        for i in e2e_order:
            case = local_cases[i]
            with torch.cuda.stream(copy_in):
                dev_x[i].copy_(host_x[i], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(copy_in)
            main.wait_event(arrived)
            w = weights_of(i, variant)
            y = forward_gather(i, case, dev_x[i], w, args.gather) if world > 1 else forward(case, dev_x[i], w)
            computed = torch.cuda.Event()
            computed.record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(computed)
                host_y[i].copy_(y, non_blocking=True)
            y.record_stream(copy_out)
        main.wait_stream(copy_in)
        main.wait_stream(copy_out)

    # The user-level call pattern of the reference engine: the step (staging copy in, every
    # projection, copy out) is captured once per variant and replayed; each timed step is
    # replay + synchronise + a host read of the result.
    e2e_variants = min(variants, 4)
    for v in range(e2e_variants):
        e2e_enqueue(v)
    torch.cuda.synchronize()
    e2e_graphs = []
    try:
        for v in range(e2e_variants):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                e2e_enqueue(v)
            e2e_graphs.append(g)
    except Exception as exc:
        e2e_graphs = []
        torch.cuda.synchronize()
        note(f"e2e graph capture failed ({exc}); eager")

    def e2e_step(variant):
        if e2e_graphs:
            e2e_graphs[variant].replay()
        else:
            e2e_enqueue(variant)
        torch.cuda.synchronize()          # the step's results are on the host
        return float(host_y[-1][0, 0])

    for j in range(3):
        e2e_step(j % e2e_variants)
    barrier()
    e2e_steps = max(3, min(args.steps, 50))
    t0 = time.perf_counter()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for j in range(e2e_steps):
        e2e_step(j % e2e_variants)
    e.record()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks(max(s.elapsed_time(e), (time.perf_counter() - t0) * 1e3) / e2e_steps)
    note(f"e2e done: {e2e_ms:.4f} ms/step")
    del e2e_graphs

    def capture_steps(how):
        graphs = []
        for v in range(variants):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                one_step(v, how)
            graphs.append(g)
        return graphs

    launches_before = _lib.launch_count()
    use_graph = True
    try:
        graphs = capture_steps(default_how)
    except Exception as exc:      # NCCL capture unsupported etc.: time eager launches instead
        use_graph = False
        graphs = []
        torch.cuda.synchronize()
        if rank == 0:
            print(f"# graph capture failed ({exc}); timing eager launches", file=sys.stderr)
    launches_per_step = (_lib.launch_count() - launches_before) // variants if use_graph else len(cases)
    note(f"capture done (graph={use_graph})")

    def run_step(i):
        if use_graph:
            graphs[i % variants].replay()
        else:
            one_step(i % variants, default_how)

    sampler = ClockSampler(local)
    sampler.start()
    # bring the clocks up, then the requested warm-up steps.  A FIXED count: with more than
    # one rank every rank must issue the same number of collectives.
    for i in range(64):
        run_step(i)
        if i % 16 == 15:
            torch.cuda.synchronize()
    for j in range(max(3, args.warmup)):
        run_step(j)
    torch.cuda.synchronize()
    note("warm-up replays done")
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for j in range(args.steps):
        run_step(j)
    end.record()
    torch.cuda.synchronize()
    barrier()
    ms_total = max_over_ranks(start.elapsed_time(end))
    ms_step = ms_total / args.steps
    note(f"timed region done: {ms_step:.4f} ms/step")

    # ---- multi-rank only: the other phases with the same protocol, so the line can show how
    # the compute phase and each kind of gather scale
    phase_ms = {}
    if world > 1:
        phase_ms[args.gather] = ms_step
        for how in ("local", "fused", "epilogue", "push", "nccl"):
            if how in phase_ms:
                continue
            torch.cuda.synchronize()
            barrier()
            try:
                solo = capture_steps(how)
            except Exception as exc:
                torch.cuda.synchronize()
                note(f"phase {how}: capture failed ({exc})")
                continue
            for j in range(16):
                solo[j % variants].replay()
            torch.cuda.synchronize()
            barrier()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for j in range(args.steps):
                solo[j % variants].replay()
            s1.record()
            torch.cuda.synchronize()
            phase_ms[how] = max_over_ranks(s0.elapsed_time(s1) / args.steps)
            note(f"phase {how}: {phase_ms[how]:.4f} ms/step")
            del solo

    # ---- per-case latency (roofline): back-to-back launches over enough distinct weight
    # buffers that none is still in L2 when it comes round again
    per_case = []
    for i, case in enumerate(local_cases):
        if args.workload in ("c3", "c3fused"):
            if not case.name.startswith("L00."):
                continue
            # the same projection of all 28 layers: 28 distinct weight buffers in rotation
            suffix = case.name.split(".", 1)[1]
            sets = [weight_sets[c.wkey][0] for c in local_cases if c.name.endswith("." + suffix)]
        else:
            sets = list(weight_sets[case.wkey])
            want = max(2, -(-2 * L2_BYTES // max(1, case.weight_bytes())) + 1)
            want = min(want, 64)
            while len(sets) < want:
                sets.append(tuple(t.clone() for t in sets[0]))
        reps = len(sets)
        entry = {"case": cases[i].key, "config": case.cfg, "M": case.m, "K": case.k, "N": cases[i].n,
                 "dtype": "fp16" if case.dtype is torch.float16 else "bf16", "kernel": kernel_of(case)}
        hows = ("local",) if world == 1 else ("local", "fused", "epilogue", "push", "nccl")
        for how in hows:
            def launch(w, how=how):
                if how == "local":
                    return forward(case, acts[i], w)
                return forward_gather(i, case, acts[i], w, how)

            for w in sets[:2]:
                launch(w)
            torch.cuda.synchronize()
            barrier()
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    for w in sets:
                        launch(w)
            except Exception as exc:
                torch.cuda.synchronize()
                note(f"per-case capture failed for {case.key} {how}: {exc}")
                continue
            sec = max_over_ranks(time_graph(g, reps))
            del g
            if how == "local":
                entry.update({"us": round(sec * 1e6, 2), "GBps": round(case.bytes / sec / 1e9, 1),
                              "TFLOPs": round(case.flops / sec / 1e12, 2)})
                entry.update(roofline_of(case.bytes, case.flops, sec, pk))
                entry["traffic"] = NCU_TRAFFIC_BYTES.get(case.key) if world == 1 else None
                entry["frac_of_nominal"] = round(max(case.bytes / 8e12, case.flops / 2.25e15) / sec, 4)
                entry["_sec"] = sec
            else:
                entry[f"{how}_gather_us"] = round(sec * 1e6, 2)
        if world == 1 and args.workload == "head" and case.fmt != "w8":
            # greedy decoding over the head: projection + torch.argmax against the fused epilogue
            from full_inference_engine_b200.kernels import argmax as fused_argmax

            def pick(w, fused):
                z = w[2] if len(w) > 2 else None
                if fused:
                    return fused_argmax.w4a16_linear_argmax(acts[i], w[0], w[1], zeros=z, static_weights=True)
                return forward(case, acts[i], w).argmax(dim=-1)

            for label, fused in (("argmax_after_us", False), ("argmax_fused_us", True)):
                assert torch.equal(pick(sets[0], True), pick(sets[0], False))
                torch.cuda.synchronize()
                g3 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g3):
                    for w in sets:
                        pick(w, fused)
                entry[label] = round(time_graph(g3, reps) * 1e6, 2)
                del g3
        if world == 1 and case.swiglu:
            # the same work as two projections + an elementwise kernel, same protocol
            halves = [tuple(tuple(t[part::2].contiguous() for t in w) for part in (0, 1)) for w in sets]
            unfused_forward(case, acts[i], halves[0])
            torch.cuda.synchronize()
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2):
                for h in halves:
                    unfused_forward(case, acts[i], h)
            entry["unfused_us"] = round(time_graph(g2, reps) * 1e6, 2)
            del g2, halves
        per_case.append(entry)
        del sets
    clocks = sampler.stop()
    note("per-case timing done")

    # ---- multi-rank only: a feed-forward's two projections (INT4 gate/up 4096 -> 12288, down
    # 12288 -> 4096) joined two ways: column-parallel + all-gather after each, against
    # column-parallel without a gather feeding a row-parallel down with the all-reduce fused
    # into its epilogue (one exchange).  Outside the timed region; device time, max over ranks.
    ffn_pairing = None
    if world > 1 and args.workload in ("all", "c2", "c5"):
        ffn_pairing = measure_ffn_pairing(args, device, rank, world, barrier, max_over_ranks, note)

    status = _lib.library().b200q_workspace_status(_lib.workspace_for(device, 256).data_ptr(), None)
    if fused_out is not None:      # a bounded wait of the fused gather protocol expired somewhere
        status = status or (7 if any(o.status() for o in fused_out) else 0)

    exit_code = 0
    if rank == 0:
        total_bytes = sum(c.bytes for c in cases)          # whole job, all ranks
        total_flops = sum(c.flops for c in cases)
        scale = 28 if args.workload in ("c3", "c3fused") else 1
        timed = [r for r in per_case if "_sec" in r]
        step_sec = sum(r["_sec"] for r in timed) * scale

        def aggregate(rows):
            """Roofline of a group of launches: per-rank bytes and flops over their summed time."""
            if not rows:
                return None
            by_key = {c.key: lc for c, lc in zip(cases, local_cases)}
            b = sum(by_key[r["case"]].bytes for r in rows)
            f = sum(by_key[r["case"]].flops for r in rows)
            t = sum(r["_sec"] for r in rows)
            out = roofline_of(b, f, t, pk)
            out.update({"cases": [r["case"] for r in rows], "us": round(t * 1e6, 2),
                        "share_of_step": round(t * scale / step_sec, 3) if step_sec else None})
            return out

        groups: dict[str, list] = {}
        for r in timed:
            groups.setdefault(r["kernel"].split(" ")[0], []).append(r)
        dominant_name = max(groups, key=lambda k: sum(r["_sec"] for r in groups[k])) if groups else None
        roofline = None
        if dominant_name:
            roofline = aggregate(groups[dominant_name])
            roofline["kernel"] = dominant_name
            captured = [r for r in groups[dominant_name] if r.get("traffic")]
            # per launch, like `achieved`: the ncu DRAM byte count of one captured case of this
            # instantiation (named beside it), or null when none has been captured
            roofline["traffic"] = captured[0]["traffic"] if captured else None
            roofline["traffic_case"] = captured[0]["case"] if captured else None
        by_instantiation = {name: {k: v for k, v in aggregate(rows).items() if k != "cases"} | {"launches": len(rows)}
                            for name, rows in groups.items()}
        regimes = {
            "hbm_M<=16": aggregate([r for r in timed if r["M"] <= 16]),
            "mid_16<M<2048": aggregate([r for r in timed if 16 < r["M"] < 2048]),
            "tensor_M>=2048": aggregate([r for r in timed if r["M"] >= 2048]),
        }
        for r in per_case:
            r.pop("_sec", None)
        line = {
            "metric": METRIC, "value": round(total_bytes / (ms_step * 1e-3) / 1e9, 2), "unit": "GB/s",
            "tflops": round(total_flops / (ms_step * 1e-3) / 1e12, 3),
            "n_gpus": args.gpus, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": round(ms_step, 5), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16/bf16 activations, fp32 accumulate", "data": "synthetic",
            "config": config_dict(args, cases),
            "l2_rotation": f"{variants} step variants, {variants * step_weight_bytes / 2**20:.0f} MiB of "
                           f"distinct weights per rank between two uses of a buffer (L2 = 126 MiB)",
            "roofline": roofline,
            "roofline_by_regime": regimes,
            "roofline_by_instantiation": by_instantiation,
            "per_case": per_case,
            "clocks": clocks,
            "e2e": {"value": round(total_bytes / (e2e_ms * 1e-3) / 1e9, 2), "unit": "GB/s",
                    "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": int(sum(2 * c.m * c.k for c in cases)),
                    "d2h_bytes_per_step": int(sum(hy.numel() * hy.element_size() for hy in host_y)),
                    "note": "weights stay resident on the device (module state); every step copies the "
                            "activations from pinned host memory, runs every forward and copies the "
                            "results back to pinned host memory (copy-in, compute and copy-out "
                            "streams overlapped inside one captured graph per step), then "
                            "synchronises and reads a result on the host"},
            "gpu_launches": int(launches_per_step * args.steps),
            "timing": "cuda-graph replay" if use_graph else "eager launches",
            "phases": None if world == 1 else {
                "sharded_gemm_only_ms_per_step": round(phase_ms["local"], 5) if "local" in phase_ms else None,
                "with_fused_all_gather_ms_per_step": round(phase_ms["fused"], 5) if "fused" in phase_ms else None,
                "with_epilogue_all_gather_ms_per_step": round(phase_ms["epilogue"], 5) if "epilogue" in phase_ms else None,
                "with_push_all_gather_ms_per_step": round(phase_ms["push"], 5) if "push" in phase_ms else None,
                "with_nccl_all_gather_ms_per_step": round(phase_ms["nccl"], 5) if "nccl" in phase_ms else None,
                "timed_value_is": args.gather,
                "per_case": "per_case[*].us is the sharded GEMM alone, fused_gather_us / epilogue_gather_us / "
                            "push_gather_us / nccl_gather_us the GEMM with that all-gather"},
            "gather_parity": gather_parity,
            "ffn_pairing": ffn_pairing,
            "device_status": status,
        }
        if world == 1:
            sec, steps, cores, sample, split = time_cpu(cases)
            line["cpu_baseline"] = {"value": round(cpu_bytes(cases) / sec / 1e9, 4), "unit": "GB/s",
                                    "cores": cores, "kind": "port", "sample": sample,
                                    "ms_per_step": round(sec * 1e3, 2), "split": split}
        print(json.dumps(line), flush=True)
        if gather_parity is not None and not gather_parity["ok"]:
            exit_code = 3
        if status:
            exit_code = exit_code or 4
    if world > 1:
        # leave without further collectives: tear the communicator down from a helper thread
        # and exit even if that blocks (every rank has synchronised its device by now)
        code = torch.tensor([float(exit_code)], dtype=torch.float64)
        dist.all_reduce(code, op=dist.ReduceOp.MAX, group=cpu_group)
        torch.cuda.synchronize()
        sys.stdout.flush()
        closer = threading.Thread(target=dist.destroy_process_group, daemon=True)
        closer.start()
        closer.join(timeout=10.0)
        os._exit(int(code.item()))
    if exit_code:
        sys.exit(exit_code)


def measure_ffn_pairing(args, device, rank, world, barrier, max_over_ranks, note):
    import torch.distributed as dist

    from full_inference_engine_b200.kernels import w4a16_format as w4
    from full_inference_engine_b200.kernels import w4a16_linear
    from full_inference_engine_b200.quantization.sharded import (
        SymmetricOutput, SymmetricReduce, fused_forward_gather, fused_forward_reduce)

    hidden, inter = 4096, 12288
    gen = torch.Generator(device=device).manual_seed(77)
    up_w = torch.randn(inter, hidden, generator=gen, device=device) * 0.02
    down_w = torch.randn(hidden, inter, generator=gen, device=device) * 0.02
    rows_up, rows_down, k_share = inter // world, hidden // world, inter // world
    copies = 6
    up_col = [w4.quantize_weight_w4_grouped(up_w[rank * rows_up:(rank + 1) * rows_up])]
    down_col = [w4.quantize_weight_w4_grouped(down_w[rank * rows_down:(rank + 1) * rows_down])]
    down_row = [w4.quantize_weight_w4_grouped(down_w[:, rank * k_share:(rank + 1) * k_share].contiguous())]
    down_full = w4.quantize_weight_w4_grouped(down_w)
    up_full = w4.quantize_weight_w4_grouped(up_w)
    del up_w, down_w
    for sets in (up_col, down_col, down_row):
        sets += [tuple(t.clone() for t in sets[0]) for _ in range(copies - 1)]
    out = []
    for m in (16, 512, 4096):
        x = torch.randn(m, hidden, generator=gen, device=device).half()
        dist.broadcast(x, 0)
        mid_buf = SymmetricOutput(m, inter, torch.float16, device)
        y_buf = SymmetricOutput(m, hidden, torch.float16, device)
        red_buf = SymmetricReduce(m, hidden, torch.float16, device)

        def two_gathers(i):
            fused_forward_gather(x, mid_buf, packed=up_col[i][0], scales=up_col[i][1])
            fused_forward_gather(mid_buf.tensor, y_buf, packed=down_col[i][0], scales=down_col[i][1])
            return y_buf.tensor

        def paired(i):
            mid = w4a16_linear.w4a16_linear(x, up_col[i][0], up_col[i][1], static_weights=True)
            fused_forward_reduce(mid, red_buf, packed=down_row[i][0], scales=down_row[i][1])
            return red_buf.tensor

        want = w4a16_linear.w4a16_linear(w4a16_linear.w4a16_linear(x, up_full[0], up_full[1]),
                                         down_full[0], down_full[1]).float()
        entry = {"M": m}
        for label, fn in (("two_gathers_us", two_gathers), ("paired_one_exchange_us", paired)):
            got = fn(0).float()
            entry[label.replace("_us", "_max_rel_err")] = round(
                float((got - want).abs().max() / want.abs().max()), 5)
            fn(1)
            torch.cuda.synchronize()
            barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(copies):
                    fn(i)
            entry[label] = round(max_over_ranks(time_graph(g, copies)) * 1e6, 2)
            del g
        out.append(entry)
        note(f"ffn pairing: {entry}")
        del mid_buf, y_buf, red_buf
    return {"shapes": "INT4 g128 4096 -> 12288 -> 4096, fp16", "cases": out}


# --------------------------------------------------------------------------- W8A8 prefill
W8A8_SHAPES = [("gate_up", 2048, 22016), ("down", 11008, 2048), ("qkv", 2048, 2560), ("o", 2048, 2048)]
W8A8_TOKENS = 4096


def run_w8a8(args):
    """The W8A8 linear (row quantiser + int8 tensor-core GEMM) on the four projection shapes of a
    Qwen2.5-3B layer at 4096 tokens.  One step = quantise + GEMM for each shape.  The roofline
    entry is compute-bound; its peak is cuBLAS's int8 GEMM (torch._int_mm) on the same shapes,
    timed in this run, because the measured-peaks file has no int8 figure."""
    m = W8A8_TOKENS
    ops = sum(2.0 * m * k * n for _, k, n in W8A8_SHAPES)
    config = {"workload": f"w8a8 prefill: {m} tokens x Qwen2.5-3B layer projections "
                          + ", ".join(f"{name} {n}x{k}" for name, k, n in W8A8_SHAPES),
              "activations": "fp16, per-row dynamic int8", "weights": "int8 per-channel, fp16 scales",
              "l2": "operands and outputs of one step exceed L2 (360 MB)"}
    base = {"metric": "w8a8_linear_int8_throughput", "unit": "TOP/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "s8", "data": "synthetic", "config": config}
    gen = np.random.default_rng(8)
    if args.impl == "reference":
        from oracle import wq_oracle as oracle
        rows = 64                                           # bounded sample: 64 of the 4096 tokens
        xs = {name: gen.standard_normal((rows, k)).astype(np.float16) for name, k, n in W8A8_SHAPES}
        ws = {name: gen.integers(-127, 128, size=(n, k), dtype=np.int8) for name, k, n in W8A8_SHAPES}
        sc = {name: (gen.random(n) * 0.01).astype(np.float16) for name, k, n in W8A8_SHAPES}
        def step():
            for name, _, _ in W8A8_SHAPES:
                oracle.w8a8_linear(xs[name], ws[name], sc[name])
        for _ in range(max(1, min(args.warmup, 2))):
            step()
        steps = max(1, min(args.steps, 5))
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        seconds = (time.perf_counter() - t0) / steps
        value = ops * rows / m / seconds / 1e12
        cores = os.cpu_count() or 1
        line = dict(base, impl="reference", value=round(value, 5), ms_per_step=round(seconds * 1e3 * m / rows, 2),
                    cpu_baseline={"value": round(value, 5), "unit": "TOP/s", "cores": cores, "kind": "port",
                                  "sample": f"{rows} of {m} tokens per shape, {steps} timed passes, numpy/BLAS threads"},
                    e2e={"value": round(value, 5), "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
        line["steps"] = steps
        print(json.dumps(line))
        return
    from full_inference_engine_b200 import _lib
    from full_inference_engine_b200.kernels import w8a8_linear as w8a8
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    tensors = {}
    for name, k, n in W8A8_SHAPES:
        x_host = torch.from_numpy(gen.standard_normal((m, k)).astype(np.float16)).pin_memory()
        qw = torch.from_numpy(gen.integers(-127, 128, size=(n, k), dtype=np.int8)).to(device)
        sc = torch.from_numpy((gen.random(n) * 0.01).astype(np.float16)).to(device)
        tensors[name] = (x_host, x_host.to(device), w8a8.pack_w8a8_weight(qw), sc, qw.t().contiguous())
    def step():
        return [w8a8.w8a8_linear(x, packed, sc) for _, x, packed, sc, _ in tensors.values()]
    def timed(fn, steps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / steps / 1e3
    for _ in range(max(3, args.warmup)):
        step()
    sampler = ClockSampler(0)
    sampler.start()
    launches_before = _lib.launch_count()
    seconds = timed(step, args.steps)
    launches = _lib.launch_count() - launches_before
    clocks = sampler.stop()
    # the integer GEMM alone, and cuBLAS's on the same operands (the measured int8 peak)
    quantised = {name: w8a8.quantize_activations_per_row(t[1]) for name, t in tensors.items()}
    def gemm_only():
        for name, (_, _, packed, sc, _) in tensors.items():
            w8a8.w8a8_linear_prequantized(*quantised[name], packed, sc, torch.float16)
    def cublas_only():
        for name, (_, _, _, _, ref_packed) in tensors.items():
            torch._int_mm(quantised[name][0], ref_packed)
    def quantise_only():
        for _, x, _, _, _ in tensors.values():
            w8a8.quantize_activations_per_row(x)
    def reference_pipeline():
        out = []
        for name, (_, x, _, sc, ref_packed) in tensors.items():
            a = x.float().abs().amax(dim=1, keepdim=True).clamp_min(1e-8) / 127.0
            q = torch.round(x.float() / a).clamp(-127, 127).to(torch.int8).contiguous()
            out.append((torch._int_mm(q, ref_packed).float() * a * sc.float()[None, :]).to(x.dtype))
        return out
    for fn in (gemm_only, cublas_only, quantise_only, reference_pipeline):
        for _ in range(3):
            fn()
    t_gemm, t_cublas = timed(gemm_only, args.steps), timed(cublas_only, args.steps)
    t_quant, t_ref = timed(quantise_only, args.steps), timed(reference_pipeline, max(3, args.steps // 5))
    # end to end: activations from pinned host memory, results back to the host
    outs_host = [torch.empty((m, n), dtype=torch.float16).pin_memory() for _, _, n in W8A8_SHAPES]
    def e2e_step():
        for (x_host, x_dev, packed, sc, _), out in zip(tensors.values(), outs_host):
            x_dev.copy_(x_host, non_blocking=True)
            out.copy_(w8a8.w8a8_linear(x_dev, packed, sc), non_blocking=True)
    for _ in range(2):
        e2e_step()
    t_e2e = timed(e2e_step, max(3, args.steps // 5))
    h2d = sum(t[0].numel() * 2 for t in tensors.values())
    d2h = sum(o.numel() * 2 for o in outs_host)
    peak = ops / t_cublas / 1e12
    line = dict(base, value=round(ops / seconds / 1e12, 2), ms_per_step=round(seconds * 1e3, 4),
                e2e={"value": round(ops / t_e2e / 1e12, 2), "unit": "TOP/s", "h2d_bytes_per_step": h2d,
                     "d2h_bytes_per_step": d2h},
                gpu_launches=int(launches), clocks=clocks,
                roofline={"bound": "tensor", "kernel": "w8a8_gemm_kernel", "achieved": round(ops / t_gemm / 1e12, 2),
                          "peak": round(peak, 2), "unit": "TOP/s", "frac": round(t_cublas / t_gemm, 4),
                          "peak_source": "cuBLAS int8 GEMM (torch._int_mm) on the same operands, timed in this run",
                          "traffic": None},
                phases={"quantise_ms": round(t_quant * 1e3, 4), "gemm_ms": round(t_gemm * 1e3, 4),
                        "cublas_int_mm_ms": round(t_cublas * 1e3, 4),
                        "torch_reference_pipeline_ms": round(t_ref * 1e3, 4)})
    print(json.dumps(line))


def run_profile(args, cases):
    """Plain eager launches, one weight buffer per launch: the command ncu wraps."""
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    copies_of = {c.wkey: 6 for c in cases}
    weight_sets, _ = make_weight_sets(cases, copies_of, device)
    acts = [make_activation(c, 5000 + i, device) for i, c in enumerate(cases)]
    n = 0
    for step in range(max(1, args.warmup) + args.steps):
        for i, case in enumerate(cases):
            sets = weight_sets[case.wkey]
            forward(case, acts[i], sets[(step + i) % len(sets)])
            n += 1
    torch.cuda.synchronize()
    print(json.dumps({"profile_launches": n, "cases": [c.key for c in cases],
                      "kernels": sorted({kernel_of(c) for c in cases})}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="all", choices=["all", "c1", "c2", "c3", "c3fused", "c4", "c5", "mlp", "head", "w8a8"])
    ap.add_argument("--layout", default="asym", choices=["asym", "ref"])
    ap.add_argument("--cases", default="", help="comma list of substrings; keep only matching case keys")
    ap.add_argument("--gather", default="fused", choices=["fused", "epilogue", "push", "nccl"],
                    help="at --gpus > 1: the all-gather that `value` times (both are reported in `phases`)")
    ap.add_argument("--verbose", action="store_true", help="progress notes on stderr")
    ap.add_argument("--profile", action="store_true",
                    help="eager launches of the selected cases only (for ncu): no graphs, no e2e, no CPU leg")
    args = ap.parse_args()
    if args.workload == "w8a8":
        if args.gpus > 1:
            raise SystemExit("the w8a8 workload is single-GPU")
        run_w8a8(args)
        return
    cases = build_cases(args.workload, args.layout)
    if args.cases:
        wanted = [w for w in args.cases.split(",") if w]
        cases = [c for c in cases if any(c.key.endswith(w) or w in c.key for w in wanted)]
        if not cases:
            raise SystemExit("--cases matched nothing")
    if args.workload == "mlp" and args.gpus > 1:
        raise SystemExit("the mlp workload is single-GPU (the gather entry points do not take gate/up pairs)")
    if args.profile:
        run_profile(args, cases)
        return
    if args.impl == "reference":
        run_reference(args, cases)
    else:
        run_b200(args, cases)


if __name__ == "__main__":
    main()
