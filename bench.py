"""Benchmark of the weight-only quantized linear forward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload c2|c5|c4|c1] [--layout asym|ref]

A *step* is one pass of the hot path over every case of the workload (one forward per
(shape, M) pair) on synthetic seeded tensors.  The default workload ``c2`` is the INT4
group-128 M-sweep at the Qwen3-8B MLP shapes; ``c5`` the M=4096 prefill GEMM; ``c4`` the
W8A16 bf16 sweep; ``c1`` the single W8A16 case the reference runs on CPU.

``value`` is algorithmic GB/s over the whole step with inputs resident in HBM (CUDA-graph
replay, two weight sets alternated so every weight byte comes from HBM, not L2).  ``e2e`` is
the same metric through the Python module API with activations in pinned host memory:
host->device copy, forward, device->host copy of the result, every step.  ``per_case``
lists every (shape, M) with its own latency, GB/s, TFLOP/s and fraction of roofline, and
``roofline`` repeats the entry of the kernel that takes the largest share of the step.
``cpu_baseline`` times the reference's CPU path (dequantise to the activation dtype +
``F.linear``) on the host cores in the same run.

With ``--impl reference`` only that CPU path runs (rank 0 only under torchrun).
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

import torch  # noqa: E402

METRIC = "W8A16/INT4 GEMM TFLOP/s and HBM GB/s vs M (1-4096), Qwen3-8B shapes"
L2_BYTES = 126 << 20

# Qwen3-8B projections: name -> (K, N)
SHAPES_8B = {"q": (4096, 4096), "kv": (4096, 2048), "o": (4096, 4096),
             "gate_up": (4096, 12288), "down": (12288, 4096)}

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures
# summarised under profiles/; keyed like Case.key.  None = not captured.
NCU_TRAFFIC_BYTES: dict[str, float] = {
    "w4_asym:gate_up:M16": 26.97e6,      # profiles/wq_gemm_tc_int4_gate_up_M16.md
    "w4_asym:gate_up:M256": 28.91e6,     # profiles/wq_gemm_tc_int4_M256.md
    "w4_asym:down:M256": 33.11e6,        # profiles/wq_gemm_tc_int4_M256.md
    "w4_asym:gate_up:M4096": 139.2e6,    # profiles/wq_gemm_tc_int4_gate_up_M4096.md
}


class Case:
    def __init__(self, name, fmt, m, k, n, dtype, outliers=False, swiglu=False):
        self.name, self.fmt, self.m, self.k, self.n = name, fmt, m, k, n
        self.dtype, self.outliers = dtype, outliers
        # n rows are interleaved (gate, up) pairs and the output is silu(gate) * up, n / 2 wide
        self.swiglu = swiglu

    @property
    def key(self):
        return f"{self.fmt}:{self.name}:M{self.m}"

    @property
    def flops(self):
        return 2.0 * self.m * self.n * self.k

    def weight_bytes(self):
        groups = self.k // 128
        if self.fmt == "w8":
            return self.n * self.k + 2 * self.n
        if self.fmt == "w4_ref":
            return self.n * self.k // 2 + 2 * self.n * groups
        return self.n * self.k // 2 + 4 * self.n * groups

    @property
    def bytes(self):
        """Algorithmic bytes: every weight byte once, activations in, outputs out."""
        n_out = self.n // 2 if self.swiglu else self.n
        return float(self.weight_bytes() + 2 * self.m * self.k + 2 * self.m * n_out)


def build_cases(workload: str, layout: str) -> list[Case]:
    w4 = "w4_asym" if layout == "asym" else "w4_ref"
    if workload == "c2":
        return [Case(name, w4, m, *SHAPES_8B[name], torch.float16)
                for name in ("gate_up", "down") for m in (1, 4, 16, 64, 256)]
    if workload == "c5":
        return [Case(name, w4, 4096, *SHAPES_8B[name], torch.bfloat16, outliers=True)
                for name in ("gate_up", "down")]
    if workload == "c4":
        return [Case(name, "w8", m, *SHAPES_8B[name], torch.bfloat16)
                for name in ("q", "kv", "o", "gate_up", "down") for m in (1, 16, 64, 512)]
    if workload == "c1":
        return [Case("gate_0p6b", "w8", 8, 1024, 3072, torch.float16)]
    if workload == "head":
        # the reference's largest single matrix: the Qwen3-8B output head (4096 -> 151936)
        return [Case("lm_head", w4, m, 4096, 151936, torch.float16) for m in (1, 16, 256)]
    if workload == "mlp":
        # beyond the reference: gate_proj + up_proj + silu(gate) * up of a Qwen3-8B feed-forward
        # as ONE launch over interleaved quantized rows (2 x 12288 rows of K = 4096)
        k, n = SHAPES_8B["gate_up"]
        return [Case("gate_up_swiglu", w4, m, k, 2 * n, torch.float16, swiglu=True)
                for m in (1, 16, 64, 256, 1024)]
    if workload == "c3":
        # one mixed step of a Qwen3-0.6B-shaped model: 16 decode rows + one 128-token chunk
        shapes = {"q": (1024, 2048), "k": (1024, 1024), "v": (1024, 1024), "o": (2048, 1024),
                  "gate": (1024, 3072), "up": (1024, 3072), "down": (3072, 1024)}
        return [Case(f"L{layer:02d}.{name}", "w8", 144, k, n, torch.float16)
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


def roofline_entry(case: Case, seconds: float, pk: dict) -> dict:
    t_hbm = case.bytes / (pk["hbm_gbs"] * 1e9)
    t_tc = case.flops / (pk["tflops"] * 1e12)
    if t_hbm >= t_tc:
        achieved, peak, unit, bound = case.bytes / seconds / 1e9, pk["hbm_gbs"], "GB/s", "hbm"
    else:
        achieved, peak, unit, bound = case.flops / seconds / 1e12, pk["tflops"], "TFLOP/s", "tensor"
    return {"bound": bound, "achieved": round(achieved, 2), "peak": peak, "unit": unit,
            "frac": round(achieved / peak, 4), "peak_source": pk["source"],
            "traffic": NCU_TRAFFIC_BYTES.get(case.key)}


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


def make_weight_sets(cases: list[Case], copies: int, device, rank: int = 0, world: int = 1):
    """Quantized weights per (fmt, shape): `copies` distinct buffers each (L2 rotation).

    With world > 1 each rank keeps rows [rank*N/world, (rank+1)*N/world) of every matrix.
    """
    from full_inference_engine_b200.kernels import w4a16_format as w4
    from full_inference_engine_b200.kernels import w8a16_linear

    sets: dict[tuple, list] = {}
    for case in cases:
        key = (case.fmt, case.name)
        if key in sets:
            continue
        gen = torch.Generator(device=device).manual_seed(1000 + len(sets))
        weight = torch.randn(case.n, case.k, generator=gen, device=device) * 0.02
        rows = case.n // world
        weight = weight[rank * rows:(rank + 1) * rows]
        if case.fmt == "w8":
            first = w8a16_linear.quantize_weight_per_channel(weight)
        elif case.fmt == "w4_ref":
            first = w4.quantize_weight_w4_grouped(weight)
        else:
            first = w4.quantize_weight_w4_asym(weight)
        del weight
        sets[key] = [first] + [tuple(t.clone() for t in first) for _ in range(copies - 1)]
    return sets


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


# --------------------------------------------------------------------------- CPU path
def cpu_inputs(cases: list[Case]):
    """Host tensors for the reference's CPU path (quantized with the CPU oracle)."""
    import numpy as np

    from oracle import wq_oracle as oracle

    weights, acts = {}, {}
    for i, case in enumerate(cases):
        key = (case.fmt, case.name)
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


def cpu_step(cases, weights, acts, limit=None):
    from oracle import cpu_path

    done = 0
    for i, case in enumerate(cases):
        if limit is not None and i not in limit:
            continue
        w = weights[(case.fmt, case.name)]
        if case.swiglu:
            cpu_path.gate_up_swiglu_forward(acts[i], w[0], w[1], int8=case.fmt == "w8")
        elif case.fmt == "w8":
            cpu_path.int8linear_forward(acts[i], w[0], w[1])
        else:
            cpu_path.w4a16_dense_forward(acts[i], w[0], w[1])
        done += 1
    return done


def time_cpu(cases, budget_s: float = 20.0, min_steps: int = 2):
    """(seconds per step, steps timed, cores, sample description) on a bounded sample."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    # keep the sample bounded: the M=4096 cases are sampled as they are, but only one pass
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
              f"split-half layout")
    return statistics.median(times), steps, cores, sample


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
    total_bytes = sum(c.bytes for c in cases)
    total_flops = sum(c.flops for c in cases)
    value = total_bytes / sec / 1e9
    sample = (f"{len(times)} of {args.steps} requested passes over all {len(cases)} cases "
              f"(bounded to {t_budget:.0f} s), torch CPU dequantise + F.linear on {cores} threads; "
              "the oracle's port of the reference CPU path (the reference tree is not on this box)")
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": "GB/s",
        "tflops": round(total_flops / sec / 1e12, 5), "n_gpus": args.gpus, "steps": len(times),
        "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16/bf16 activations, fp32 accumulate",
        "data": "synthetic", "config": config_dict(args, cases, rotation=None),
        "cpu_baseline": {"value": round(value, 4), "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def config_dict(args, cases, rotation):
    return {
        "workload": {"c2": "config 2: INT4 g128 M-sweep {1,4,16,64,256} at Qwen3-8B gate/up "
                           "(4096->12288) and down (12288->4096), fp16 activations",
                     "c5": "config 5: INT4 g128 prefill M=4096 bf16 with 1% outlier rows, "
                           "gate/up and down",
                     "c4": "config 4: W8A16 bf16 at Qwen3-8B q/kv/o/gate_up/down, M in {1,16,64,512}",
                     "c1": "config 1: W8A16 M=8 K=1024 N=3072 fp16",
                     "head": "the Qwen3-8B output head, INT4 g128 4096 -> 151936 (the reference's largest "
                             "matrix, benchmarks/kernels/w4a16_bench.py), M in {1,16,256}, fp16",
                     "mlp": "beyond the reference: INT4 g128 gate_proj + up_proj + silu(gate) * up of a "
                            "Qwen3-8B feed-forward (K=4096, 2 x 12288 interleaved rows) in one launch, "
                            "M in {1,16,64,256,1024}, fp16; per_case carries the two-projections-plus-"
                            "elementwise time beside it",
                     "c3": "config 3: 28 x 7 random-init Qwen3-0.6B W8A16 projections, one mixed "
                           "step of M=144 rows (16 decode + 128 prefill), fp16, one CUDA graph"}[args.workload],
        "layout": {"asym": "asymmetric int32 x8 nibbles + fp16 scale and zero-point",
                   "ref": "reference split-half uint8 + fp16 scale"}[args.layout]
        if cases[0].fmt != "w8" else "int8 per-channel fp16 scale",
        "cases": len(cases),
        "parallelism": (f"N-sharded x{args.gpus}, all-gather "
                        + ("fused into the kernel epilogue (peer stores over NVLink)"
                           if args.gather == "fused" else "by NCCL")) if args.gpus > 1 else "single GPU",
        "l2": rotation,
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
    copies = {"c1": 48, "c2": 10, "c3": 1, "c4": 4, "c5": 6, "mlp": 6, "head": 2}[args.workload]
    weight_sets = make_weight_sets(cases, copies, device, rank, world)
    acts = [make_activation(c, 5000 + i, device) for i, c in enumerate(cases)]
    # per-rank view of each case
    local_cases = [Case(c.name, c.fmt, c.m, c.k, c.n // world, c.dtype, c.outliers, c.swiglu) for c in cases]
    gathered = [torch.empty(world, c.m, c.n // world, dtype=c.dtype, device=device) if world > 1 else None
                for c in cases]
    # fused all-gather: full [M, N] outputs in symmetric memory, written by every rank's epilogue
    fused_out = None
    if world > 1 and args.gather == "fused":
        from full_inference_engine_b200.quantization.sharded import SymmetricOutput

        fused_out = [SymmetricOutput(c.m, c.n, c.dtype, device) for c in cases]

    def forward_gather(i, case, x, w):
        """This rank's columns of case i delivered to every rank; returns the local view."""
        if fused_out is not None:
            from full_inference_engine_b200.quantization.sharded import fused_forward_gather

            if case.fmt == "w8":
                ok = fused_forward_gather(x, fused_out[i], qweight=w[0], scales=w[1])
            elif case.fmt == "w4_ref":
                ok = fused_forward_gather(x, fused_out[i], packed=w[0], scales=w[1])
            else:
                ok = fused_forward_gather(x, fused_out[i], packed=w[0], scales=w[1], zeros=w[2])
            if ok:
                return fused_out[i].tensor
        y = forward(case, x, w)
        dist.all_gather_into_tensor(gathered[i], y)
        return y

    def one_step(variant: int, gather: bool = True):
        outs = []
        for i, case in enumerate(local_cases):
            sets = weight_sets[(case.fmt, case.name)]
            w = sets[(i + variant * len(local_cases)) % len(sets)]
            if world > 1 and gather:
                y = forward_gather(i, case, acts[i], w)
            else:
                y = forward(case, acts[i], w)
            outs.append(y)
        return outs

    step_weight_bytes = sum(c.weight_bytes() for c in local_cases)
    # enough step variants (each on its own weight copies) that >= 2 x L2 of distinct weights
    # pass between two uses of the same buffer
    variants = max(1, min(copies, -(-2 * L2_BYTES // step_weight_bytes)))
    if copies > 1:
        variants = max(2, variants)
    rotation = (f"inputs larger than L2: each case reads its own weight buffer and {variants} step "
                f"variant(s) alternate, {variants * step_weight_bytes / 2**20:.0f} MiB of distinct "
                f"weights between reuses (L2 = 126 MiB)")

    # eager warm-up (also sizes the workspace), then capture two step variants
    note("inputs ready")
    for v in range(variants):
        one_step(v)
    torch.cuda.synchronize()
    note("eager warm-up done")

    # ---- end to end (measured before any graph holds NCCL work): pinned host activations in, host results out, through the public API
    host_x = [torch.empty(c.m, c.k, dtype=c.dtype).pin_memory().copy_(acts[i].cpu()) for i, c in enumerate(cases)]
    host_y = [torch.empty(c.m, (c.n if fused_out is not None else c.n // world) // (2 if c.swiglu else 1),
                          dtype=c.dtype).pin_memory()
              for c in cases]
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
            sets = weight_sets[(case.fmt, case.name)]
            w = sets[(i + variant * len(local_cases)) % len(sets)]
            y = forward_gather(i, case, dev_x[i], w) if world > 1 else forward(case, dev_x[i], w)
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
    for v in range(variants):
        e2e_enqueue(v)
    torch.cuda.synchronize()
    e2e_graphs = []
    try:
        for v in range(variants):
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
        e2e_step(j % variants)
    barrier()
    e2e_steps = max(3, min(args.steps, 50))
    t0 = time.perf_counter()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for j in range(e2e_steps):
        e2e_step(j % variants)
    e.record()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks(max(s.elapsed_time(e), (time.perf_counter() - t0) * 1e3) / e2e_steps)
    note(f"e2e done: {e2e_ms:.4f} ms/step")

    launches_before = _lib.launch_count()
    graphs = []
    use_graph = True
    try:
        for v in range(variants):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                one_step(v)
            graphs.append(g)
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
            one_step(i % variants)

    sampler = ClockSampler(local)
    sampler.start()
    # bring the clocks up, then the requested warm-up steps.  A FIXED count: with more than
    # one rank every rank must issue the same number of collectives.
    for i in range(256):
        run_step(i)
        if i % 64 == 63:
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

    # ---- multi-rank only: the sharded GEMMs alone (no collective), same protocol, so the
    # line can show how the compute phase and the gather phase each scale
    gemm_only_ms = None
    if world > 1:
        torch.cuda.synchronize()
        for v in range(variants):
            one_step(v, gather=False)
        solo = []
        for v in range(variants):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                one_step(v, gather=False)
            solo.append(g)
        for j in range(16):
            solo[j % variants].replay()
        torch.cuda.synchronize()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for j in range(args.steps):
            solo[j % variants].replay()
        s1.record()
        torch.cuda.synchronize()
        gemm_only_ms = max_over_ranks(s0.elapsed_time(s1) / args.steps)
        note(f"gemm-only: {gemm_only_ms:.4f} ms/step")

    # ---- per-case latency (roofline): R back-to-back launches over rotating weight copies
    per_case = []
    # per-case latencies are a single-GPU diagnostic; the multi-rank run reports the step only
    for i, case in enumerate(local_cases if world == 1 else []):
        if args.workload == "c3":
            if not case.name.startswith("L00."):
                continue
            # the same projection of all 28 layers: 28 distinct weight buffers in rotation
            suffix = case.name.split(".", 1)[1]
            sets = [weight_sets[(c.fmt, c.name)][0] for c in local_cases if c.name.endswith("." + suffix)]
        else:
            sets = weight_sets[(case.fmt, case.name)]
        reps = len(sets)
        for w in sets[:2]:
            forward(case, acts[i], w)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for w in sets:
                forward(case, acts[i], w)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(7):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            g.replay()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e) / reps)
        sec = statistics.median(times) * 1e-3
        entry = {"case": case.key, "M": case.m, "K": case.k, "N": case.n, "us": round(sec * 1e6, 2),
                 "GBps": round(case.bytes / sec / 1e9, 1), "TFLOPs": round(case.flops / sec / 1e12, 2)}
        entry.update(roofline_entry(case, sec, pk))
        entry["frac_of_nominal"] = round(
            max(case.bytes / 8e12, case.flops / 2.25e15) / sec, 4)
        if args.workload == "head" and case.fmt != "w8":
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
                for _ in range(3):
                    g3.replay()
                torch.cuda.synchronize()
                t3 = []
                for _ in range(7):
                    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    s.record()
                    g3.replay()
                    e.record()
                    torch.cuda.synchronize()
                    t3.append(s.elapsed_time(e) / reps)
                entry[label] = round(statistics.median(t3) * 1e3, 2)
                del g3
        if case.swiglu:
            # the same work as two projections + an elementwise kernel, same protocol
            halves = [tuple(tuple(t[part::2].contiguous() for t in w) for part in (0, 1)) for w in sets]
            unfused_forward(case, acts[i], halves[0])
            torch.cuda.synchronize()
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2):
                for h in halves:
                    unfused_forward(case, acts[i], h)
            for _ in range(3):
                g2.replay()
            torch.cuda.synchronize()
            times2 = []
            for _ in range(7):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                g2.replay()
                e.record()
                torch.cuda.synchronize()
                times2.append(s.elapsed_time(e) / reps)
            entry["unfused_us"] = round(statistics.median(times2) * 1e3, 2)
            del g2, halves
        per_case.append(entry)
        del g
    clocks = sampler.stop()
    note("per-case timing done")

    status = _lib.library().b200q_workspace_status(_lib.workspace_for(device, 256).data_ptr(), None)
    if fused_out is not None:      # a bounded wait of the fused gather protocol expired somewhere
        status = status or (7 if any(o.status() for o in fused_out) else 0)

    if rank == 0:
        total_bytes = sum(c.bytes for c in cases)          # whole job, all ranks
        total_flops = sum(c.flops for c in cases)
        dominant = max(per_case, key=lambda r: r["us"]) if per_case else None
        step_us = sum(r["us"] for r in per_case) * (28 if args.workload == "c3" else 1)
        line = {
            "metric": METRIC, "value": round(total_bytes / (ms_step * 1e-3) / 1e9, 2), "unit": "GB/s",
            "tflops": round(total_flops / (ms_step * 1e-3) / 1e12, 3),
            "n_gpus": args.gpus, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": round(ms_step, 5), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16/bf16 activations, fp32 accumulate", "data": "synthetic",
            "config": config_dict(args, cases, rotation),
            "roofline": ({k: dominant[k] for k in ("bound", "achieved", "peak", "unit", "frac", "traffic")}
                         | {"kernel": dominant["case"], "share_of_step": round(dominant["us"] / step_us, 3),
                            "peak_source": pk["source"]}) if dominant else None,
            "per_case": per_case,
            "clocks": clocks,
            "e2e": {"value": round(total_bytes / (e2e_ms * 1e-3) / 1e9, 2), "unit": "GB/s",
                    "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": int(sum(2 * c.m * c.k for c in cases)),
                    "d2h_bytes_per_step": int(sum(hy.numel() * hy.element_size() for hy in host_y)),
                    "note": "weights stay resident on the device (module state); every step copies the "
                            "activations from pinned host memory, runs every forward and copies the "
                            "results back to pinned host memory (copy-in, compute and copy-out "
                            "streams overlapped inside one captured graph per step, "
                            + ("replayed" if e2e_graphs else "eager launches")
                            + "), then synchronises and reads a result on the host"},
            "gpu_launches": int(launches_per_step * args.steps),
            "timing": "cuda-graph replay" if use_graph else "eager launches",
            "phases": None if gemm_only_ms is None else {
                "sharded_gemm_only_ms_per_step": round(gemm_only_ms, 5),
                "with_all_gather_ms_per_step": round(ms_step, 5)},
            "device_status": status,
        }
        if world == 1:
            sec, steps, cores, sample = time_cpu(cases)
            line["cpu_baseline"] = {"value": round(total_bytes / sec / 1e9, 4), "unit": "GB/s",
                                    "cores": cores, "kind": "port", "sample": sample,
                                    "ms_per_step": round(sec * 1e3, 2)}
        print(json.dumps(line), flush=True)
    if world > 1:
        # leave without further collectives: tear the communicator down from a helper thread
        # and exit even if that blocks (every rank has synchronised its device by now)
        torch.cuda.synchronize()
        sys.stdout.flush()
        closer = threading.Thread(target=dist.destroy_process_group, daemon=True)
        closer.start()
        closer.join(timeout=10.0)
        os._exit(0)


def run_profile(args, cases):
    """Plain eager launches, one weight buffer per launch: the command ncu wraps."""
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    weight_sets = make_weight_sets(cases, 6, device)
    acts = [make_activation(c, 5000 + i, device) for i, c in enumerate(cases)]
    n = 0
    for step in range(max(1, args.warmup) + args.steps):
        for i, case in enumerate(cases):
            sets = weight_sets[(case.fmt, case.name)]
            forward(case, acts[i], sets[(step + i) % len(sets)])
            n += 1
    torch.cuda.synchronize()
    print(json.dumps({"profile_launches": n, "cases": [c.key for c in cases]}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c4", "c5", "mlp", "head"])
    ap.add_argument("--layout", default="asym", choices=["asym", "ref"])
    ap.add_argument("--cases", default="", help="comma list of substrings; keep only matching case keys")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="at --gpus > 1: all-gather inside the kernel epilogue, or a NCCL call after it")
    ap.add_argument("--verbose", action="store_true", help="progress notes on stderr")
    ap.add_argument("--profile", action="store_true",
                    help="eager launches of the selected cases only (for ncu): no graphs, no e2e, no CPU leg")
    args = ap.parse_args()
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
