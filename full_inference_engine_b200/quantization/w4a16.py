"""4-bit grouped weights installed on a model, served by the B200 kernels.

The module and installer surface of the reference's ``engine/quantization/w4a16.py``:
``W4A16Linear`` (buffers ``packed`` uint8 ``[N, K//2]``, ``scales`` fp16 ``[N, K//group]``,
optional fp16 ``bias``; ``quantize_from``, ``set_bias``, ``dequantized``, ``loaded``,
``reference``), ``install_w4a16`` for a model already in memory, ``load_w4a16_model`` for a
safetensors folder streamed through a ``meta``-device skeleton, ``reference_mode`` /
``w4a16_modules`` / ``describe`` / ``W4A16Report``.

What differs is below the module: every row count runs ONE fused kernel (CUDA-core split-K
for decode rows, tcgen05 tensor cores above), so there is no dequantise-into-scratch step
and no M-dependent detour through cuBLAS.  ``reference = True`` (or ``reference_mode``)
still runs the reference's arithmetic in torch over the same packed weights: that is the
identity gate's comparison target and the only path that accepts non-CUDA tensors.

Target discovery is structural, as in the reference: a Linear is a target because of its
attribute name inside a decoder block, or because the model names it as its output head.
"""

from __future__ import annotations

import contextlib
import glob
import os
from dataclasses import dataclass, field

import torch
from torch import nn
from torch.nn import functional as F

from .. import _lib
from ..kernels import w4a16_format as _fmt
from ..kernels import w4a16_linear as _k
from ..kernels.w4a16_format import GEMV_MAX_ROWS, GROUP_SIZE, unpack_w4_reference, weight_bytes

ATTENTION_PROJECTIONS = ("q_proj", "k_proj", "v_proj", "o_proj")
MLP_PROJECTIONS = ("gate_proj", "up_proj", "down_proj")
DEFAULT_TARGETS = ("attention", "mlp", "lm_head")


def kernel_available() -> bool:
    """Whether libb200q.so can be loaded in this process."""
    try:
        _lib.library()
        return True
    except Exception:
        return False


_SCRATCH: dict[torch.device, torch.Tensor] = {}


def dense_scratch(device: torch.device, out_features: int, in_features: int) -> torch.Tensor:
    """A persistent per-device fp16 buffer viewed as ``[out, in]`` (grown on demand).

    The kernels never need a dequantised tile; this stays for callers that want one
    (``w4_dequantize_into`` targets) without allocating inside a captured graph.
    """
    device = torch.device(device)
    count = out_features * in_features
    held = _SCRATCH.get(device)
    if held is None or held.numel() < count:
        held = torch.empty(count, dtype=torch.float16, device=device)
        _SCRATCH[device] = held
    return held[:count].view(out_features, in_features)


def _quantize(weight: torch.Tensor, group_size: int) -> tuple[torch.Tensor, torch.Tensor]:
    """The quantizer ``quantize_from`` uses; module-level so host-side tests can swap it."""
    return _fmt.quantize_weight_w4_grouped(weight, group_size)


class W4A16Linear(nn.Module):
    """``nn.Linear`` over 4-bit grouped weights in the reference's split-half layout."""

    # The reference sends M >= dense_threshold through a dequantised tile; here the value
    # only documents where the CUDA-core kernel hands over to the tensor-core kernel.
    dense_slab_bytes: int = 32 << 20       # reference-mode slab size (fp16 bytes at once)
    workspace_rows: int = 4096             # largest token count `dense_scratch_bytes` is sized for

    @property
    def dense_scratch_bytes(self) -> int:
        """Device scratch this module's forward needs, for engines that size their KV pool from
        it (the reference reads the attribute in ``_auto_kv_reserve``,
        engine/continuous_batching.py:823-828): the kernel workspace for up to
        ``workspace_rows`` tokens, in the 8 MiB granules the per-device workspace grows by.
        Assigning the attribute overrides the figure.  ``reserve_workspace(model)`` allocates it."""
        override = self.__dict__.get("_dense_scratch_override")
        if override is not None:
            return int(override)
        try:
            need = _lib.max_workspace_bytes(4, self.workspace_rows, self.out_features, self.in_features)
        except (OSError, RuntimeError):
            need = 0                       # the library is not built here: the floor below
        return max(_lib.WORKSPACE_GRANULE, -(-need // _lib.WORKSPACE_GRANULE) * _lib.WORKSPACE_GRANULE)

    @dense_scratch_bytes.setter
    def dense_scratch_bytes(self, value: int) -> None:
        self.__dict__["_dense_scratch_override"] = int(value)

    def __init__(self, in_features: int, out_features: int, *, group_size: int = GROUP_SIZE,
                 bias: bool = False, device=None):
        super().__init__()
        if in_features % group_size:
            raise ValueError(f"in_features {in_features} is not a multiple of group_size {group_size}")
        self.in_features = in_features
        self.out_features = out_features
        self.group_size = group_size
        self.reference = False
        self.dense_threshold = GEMV_MAX_ROWS + 1
        self.register_buffer("packed", torch.empty(out_features, in_features // 2,
                                                   dtype=torch.uint8, device=device))
        self.register_buffer("scales", torch.empty(out_features, in_features // group_size,
                                                   dtype=torch.float16, device=device))
        if bias:
            self.register_buffer("bias", torch.empty(out_features, dtype=torch.float16, device=device))
        else:
            self.bias = None

    @property
    def loaded(self) -> bool:
        return self.packed.device.type != "meta"

    def quantize_from(self, weight: torch.Tensor) -> None:
        """Quantize ``weight [out, in]`` into this layer (on the weight's device)."""
        if tuple(weight.shape) != (self.out_features, self.in_features):
            raise ValueError(f"weight {tuple(weight.shape)} does not match "
                             f"[{self.out_features}, {self.in_features}]")
        packed, scales = _quantize(weight.detach(), self.group_size)
        self.packed = packed.to(weight.device)
        self.scales = scales.to(weight.device)

    def set_bias(self, bias: torch.Tensor | None) -> None:
        self.bias = None if bias is None else bias.detach().to(torch.float16)

    def dequantized(self, dtype: torch.dtype = torch.float16) -> torch.Tensor:
        return unpack_w4_reference(self.packed, self.scales, self.in_features, self.group_size).to(dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.loaded:
            raise RuntimeError("W4A16Linear has no weights: load or quantize_from first")
        rows = x.reshape(-1, self.in_features)
        if self.reference:
            out = self._reference_forward(rows)
        elif rows.device.type != "cuda":
            raise RuntimeError("W4A16Linear runs on CUDA tensors; use reference_mode for the "
                               "torch arithmetic on other devices")
        else:
            compute = rows if rows.dtype in (torch.float16, torch.bfloat16) else rows.to(torch.float16)
            out = _k.w4a16_linear(compute, self.packed, self.scales, self.bias,
                                  group_size=self.group_size, static_weights=True).to(x.dtype)
        return out.reshape(*x.shape[:-1], self.out_features)

    def argmax(self, x: torch.Tensor) -> torch.Tensor:
        """``self(x).argmax(-1)`` (greedy decoding over an output head) without writing the
        ``[..., out_features]`` outputs: the kernel's epilogue keeps each row's maximum."""
        if self.reference or x.device.type != "cuda":
            return self.forward(x).argmax(dim=-1)
        from ..kernels.argmax import w4a16_linear_argmax

        rows = x.reshape(-1, self.in_features)
        compute = rows if rows.dtype in (torch.float16, torch.bfloat16) else rows.to(torch.float16)
        channels = w4a16_linear_argmax(compute, self.packed, self.scales, self.bias,
                                       group_size=self.group_size, static_weights=True)
        return channels.reshape(x.shape[:-1])

    def _reference_forward(self, rows: torch.Tensor) -> torch.Tensor:
        """Dequantise (whole, or in N slabs above ``dense_slab_bytes``) and ``F.linear``."""
        bias = None if self.bias is None else self.bias.to(rows.dtype)
        slab = self.out_features
        if 2 * self.out_features * self.in_features > self.dense_slab_bytes:
            slab = max(1, self.dense_slab_bytes // (2 * self.in_features))
        pieces = []
        for start in range(0, self.out_features, slab):
            stop = min(start + slab, self.out_features)
            weight = unpack_w4_reference(self.packed[start:stop], self.scales[start:stop],
                                         self.in_features, self.group_size).to(rows.dtype)
            pieces.append(F.linear(rows, weight, None if bias is None else bias[start:stop]))
        return pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=-1)

    def extra_repr(self) -> str:
        return (f"in={self.in_features}, out={self.out_features}, group={self.group_size}, "
                f"bias={self.bias is not None}, kernel={'reference' if self.reference else 'b200q'}")


@dataclass
class W4A16Report:
    """What an install or load replaced."""

    replaced: int = 0
    by_kind: dict = field(default_factory=dict)
    fp16_bytes: int = 0
    packed_bytes: int = 0
    skipped: list = field(default_factory=list)

    @property
    def ratio(self) -> float:
        return self.fp16_bytes / self.packed_bytes if self.packed_bytes else 0.0

    def count(self, kind: str, in_features: int, out_features: int, group_size: int) -> None:
        sizes = weight_bytes(in_features, out_features, group_size)
        self.replaced += 1
        self.by_kind[kind] = self.by_kind.get(kind, 0) + 1
        self.fp16_bytes += sizes["fp16"]
        self.packed_bytes += sizes["w4a16"]

    def as_dict(self) -> dict:
        mib = 2 ** 20
        return {"replaced": self.replaced, "by_kind": dict(self.by_kind),
                "fp16_mib": round(self.fp16_bytes / mib), "packed_mib": round(self.packed_bytes / mib),
                "ratio": round(self.ratio, 2), "skipped": list(self.skipped)}


# --------------------------------------------------------------------------- discovery
def _targets(model: nn.Module, targets) -> list[tuple[str, str, nn.Linear, str]]:
    """``(qualified name, kind, module, attribute)`` of every Linear an install owns."""
    wanted = set(targets)
    by_attribute = {}
    if "attention" in wanted:
        by_attribute.update({a: "attention" for a in ATTENTION_PROJECTIONS})
    if "mlp" in wanted:
        by_attribute.update({a: "mlp" for a in MLP_PROJECTIONS})
    found: dict[str, tuple[str, str, nn.Linear, str]] = {}
    for prefix, module in model.named_modules():
        for attribute, kind in by_attribute.items():
            child = getattr(module, attribute, None)
            if isinstance(child, nn.Linear):
                name = f"{prefix}.{attribute}" if prefix else attribute
                found.setdefault(name, (name, kind, child, attribute))
    if "lm_head" in wanted and hasattr(model, "get_output_embeddings"):
        head = model.get_output_embeddings()
        if isinstance(head, nn.Linear):
            for name, module in model.named_modules():
                if module is head:
                    found.setdefault(name, (name, "lm_head", module, name.rsplit(".", 1)[-1]))
                    break
    return list(found.values())


def _parent(model: nn.Module, qualified: str) -> tuple[nn.Module, str]:
    head, _, leaf = qualified.rpartition(".")
    return (model.get_submodule(head) if head else model), leaf


def _shell_for(linear: nn.Linear, group_size: int, device) -> W4A16Linear:
    return W4A16Linear(linear.in_features, linear.out_features, group_size=group_size,
                       bias=linear.bias is not None, device=device)


# --------------------------------------------------------------------------- install in place
@torch.no_grad()
def install_w4a16(model: nn.Module, *, group_size: int = GROUP_SIZE,
                  targets=DEFAULT_TARGETS) -> W4A16Report:
    """Quantize every target Linear of a loaded model in place, dropping each fp16 weight."""
    report = W4A16Report()
    for name, kind, linear, _ in _targets(model, targets):
        if linear.in_features % group_size:
            report.skipped.append(f"{name}: in_features {linear.in_features} % {group_size}")
            continue
        shell = _shell_for(linear, group_size, linear.weight.device)
        shell.quantize_from(linear.weight.data)
        shell.set_bias(None if linear.bias is None else linear.bias.data)
        owner, attribute = _parent(model, name)
        setattr(owner, attribute, shell)
        report.count(kind, linear.in_features, linear.out_features, group_size)
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return report


# --------------------------------------------------------------------------- streaming load
def _assign(model: nn.Module, key: str, tensor: torch.Tensor) -> bool:
    """Replace the meta placeholder ``key`` names (parameter or buffer); False if none."""
    owner_name, _, leaf = key.rpartition(".")
    try:
        owner = model.get_submodule(owner_name) if owner_name else model
    except AttributeError:
        return False
    if leaf in owner._parameters:
        owner._parameters[leaf] = nn.Parameter(tensor, requires_grad=False)
        return True
    if leaf in owner._buffers:
        owner._buffers[leaf] = tensor
        return True
    return False


def _reinit_rotary(model: nn.Module, config, device) -> int:
    """Rotary tables are built in ``__init__``: a meta-built model has meta tables; rebuild."""
    rebuilt = 0
    for name, module in list(model.named_modules()):
        if hasattr(module, "inv_freq"):
            owner, attribute = _parent(model, name)
            setattr(owner, attribute, type(module)(config).to(device))
            rebuilt += 1
    return rebuilt


def _meta_tensors(model: nn.Module) -> list[str]:
    return [n for n, t in (*model.named_parameters(), *model.named_buffers())
            if t.device.type == "meta"]


@torch.no_grad()
def load_w4a16_model(model_name: str, *, device, revision: str | None = None,
                     group_size: int = GROUP_SIZE, targets=DEFAULT_TARGETS,
                     dtype: torch.dtype = torch.float16) -> tuple[nn.Module, W4A16Report]:
    """Stream a safetensors checkpoint (local folder or Hub id) into a 4-bit model.

    The model is built on ``meta``, its target Linears are swapped for empty shells, and
    each checkpoint tensor is quantized on ``device`` as it arrives: the fp16 model never
    exists anywhere.
    """
    from transformers import AutoConfig, AutoModelForCausalLM

    device = torch.device(device)
    config = AutoConfig.from_pretrained(model_name, revision=revision)
    with torch.device("meta"):
        model = AutoModelForCausalLM.from_config(config, dtype=dtype)
    model.eval()

    report = W4A16Report()
    shells: dict[str, W4A16Linear] = {}
    for name, kind, linear, _ in _targets(model, targets):
        if linear.in_features % group_size:
            report.skipped.append(f"{name}: in_features {linear.in_features} % {group_size}")
            continue
        shell = _shell_for(linear, group_size, "meta")
        owner, attribute = _parent(model, name)
        setattr(owner, attribute, shell)
        shells[name] = shell
        report.count(kind, linear.in_features, linear.out_features, group_size)

    folder = model_name if os.path.isdir(model_name) else _download(model_name, revision)
    shards = sorted(glob.glob(os.path.join(folder, "*.safetensors")))
    if not shards:
        raise FileNotFoundError(f"no safetensors shards under {folder}")
    from safetensors import safe_open

    homeless = []
    for path in shards:
        with safe_open(path, framework="pt", device="cpu") as shard:
            for key in shard.keys():
                tensor = shard.get_tensor(key)
                owner_name, _, leaf = key.rpartition(".")
                shell = shells.get(owner_name)
                if shell is not None and leaf == "weight":
                    shell.quantize_from(tensor.to(device=device, dtype=torch.float16))
                elif shell is not None and leaf == "bias":
                    shell.set_bias(tensor.to(device=device, dtype=torch.float16))
                elif not _assign(model, key, tensor.to(device=device, dtype=dtype)):
                    homeless.append(key)
                del tensor
    if homeless:
        raise ValueError(f"checkpoint tensors with no home in the model: {homeless[:8]}"
                         + (" ..." if len(homeless) > 8 else ""))

    # a tied head ships no lm_head.weight: quantize it from the embedding table
    head = model.get_output_embeddings()
    tied = bool(getattr(config, "tie_word_embeddings", False))
    if isinstance(head, W4A16Linear) and not head.loaded:
        if not tied:
            raise ValueError("lm_head.weight missing from the checkpoint and the head is untied")
        head.quantize_from(model.get_input_embeddings().weight.data.to(torch.float16))
    elif isinstance(head, nn.Linear) and head.weight.device.type == "meta" and tied:
        head.weight = model.get_input_embeddings().weight

    _reinit_rotary(model, config, device)
    leftover = _meta_tensors(model)
    if leftover:
        raise ValueError(f"tensors never loaded (still on meta): {leftover[:8]}"
                         + (" ..." if len(leftover) > 8 else ""))
    if device.type == "cuda":
        torch.cuda.empty_cache()
    return model, report


def _download(model_name: str, revision: str | None) -> str:
    from huggingface_hub import snapshot_download

    return snapshot_download(model_name, revision=revision,
                             allow_patterns=["*.safetensors", "*.json", "*.txt", "*.model"])


# --------------------------------------------------------------------------- reference mode, reporting
def reserve_workspace(model: nn.Module, max_rows: int | None = None) -> int:
    """Allocate, once, the per-device kernel workspace that every quantized projection of
    ``model`` needs for up to ``max_rows`` tokens, and return its size in bytes.

    Call it after install and BEFORE an engine hands the remaining device memory to its KV
    pool: the workspace otherwise grows on the first forward that needs more (and cannot grow
    during CUDA-graph capture).  No counterpart in the reference, whose scratch is the
    dequantised tile ``dense_scratch`` grows on demand (engine/quantization/w4a16.py:62-76)."""
    need, device = 0, None
    for module in w4a16_modules(model):
        if module.packed.device.type != "cuda":
            continue
        rows = module.workspace_rows if max_rows is None else max_rows
        need = max(need, _lib.max_workspace_bytes(4, rows, module.out_features, module.in_features))
        device = module.packed.device
    if device is None:
        return 0
    return int(_lib.workspace_for(device, need).numel())


def w4a16_modules(model: nn.Module) -> list[W4A16Linear]:
    return [m for m in model.modules() if isinstance(m, W4A16Linear)]


@contextlib.contextmanager
def reference_mode(model: nn.Module):
    """Every ``W4A16Linear`` of ``model`` runs the torch arithmetic inside the ``with``."""
    modules = w4a16_modules(model)
    before = [m.reference for m in modules]
    for m in modules:
        m.reference = True
    try:
        yield
    finally:
        for m, flag in zip(modules, before):
            m.reference = flag


def describe(model: nn.Module) -> dict:
    modules = w4a16_modules(model)
    mib = 2 ** 20
    return {
        "w4a16_modules": len(modules),
        "packed_mib": round(sum(m.packed.numel() + 2 * m.scales.numel() for m in modules) / mib),
        "fp16_equivalent_mib": round(sum(2 * m.in_features * m.out_features for m in modules) / mib),
        "group_size": modules[0].group_size if modules else None,
        "kernel": "b200q (sm_100a)" if kernel_available() else "reference (libb200q.so not built)",
    }
