"""Pre-quantized 4-bit checkpoints: write an installed model once, load it without re-quantizing.

The reference quantizes on every load (``load_w4a16_model``, engine/quantization/w4a16.py:
314-391): each fp16 tensor crosses PCIe and is quantized on the device.  A serialised packed
format makes the second and later loads move a quarter of the bytes and run no quantizer:

* ``config.json`` (and whatever else ``config.save_pretrained`` writes),
* ``model-w4a16.safetensors``: every ``W4A16Linear`` as ``<name>.packed`` (uint8 ``[N, K/2]``,
  the reference's split-half layout), ``<name>.scales`` (fp16 ``[N, K/group]``) and, if present,
  ``<name>.bias``; every other parameter and buffer under its own name,
* ``b200q_quantization.json``: format tag, group size and the names of the quantized modules.

Tied tensors are stored once; rotary tables are rebuilt from the config, not stored.
"""

from __future__ import annotations

import json
import os

import torch
from torch import nn

from .w4a16 import (
    W4A16Linear, W4A16Report, _assign, _meta_tensors, _parent, _reinit_rotary,
)

FORMAT_TAG = "w4a16-split-half-sym"
WEIGHTS_FILE = "model-w4a16.safetensors"
META_FILE = "b200q_quantization.json"


def save_w4a16_checkpoint(model: nn.Module, folder: str) -> dict:
    """Write ``model`` (after ``install_w4a16`` / ``load_w4a16_model``) to ``folder``.

    Returns the metadata that was written.  Raises ``ValueError`` if the model holds no
    ``W4A16Linear`` or if its quantized modules disagree on the group size.
    """
    from safetensors.torch import save_file

    quantized = {name: m for name, m in model.named_modules() if isinstance(m, W4A16Linear)}
    if not quantized:
        raise ValueError("model holds no W4A16Linear: nothing to serialise")
    groups = {m.group_size for m in quantized.values()}
    if len(groups) != 1:
        raise ValueError(f"quantized modules disagree on the group size: {sorted(groups)}")
    unloaded = [n for n, m in quantized.items() if not m.loaded]
    if unloaded:
        raise ValueError(f"quantized modules without weights: {unloaded[:4]}")

    tensors: dict[str, torch.Tensor] = {}
    seen: dict[tuple, str] = {}
    aliases: dict[str, str] = {}
    skip_prefixes = tuple(name + "." for name, m in model.named_modules() if hasattr(m, "inv_freq"))
    named = list(model.named_parameters(remove_duplicate=False)) + list(model.named_buffers(remove_duplicate=False))
    for name, tensor in named:
        if tensor is None or name.startswith(skip_prefixes):
            continue
        key = (str(tensor.device), tensor.data_ptr(), tuple(tensor.shape), tensor.dtype)
        if tensor.numel() and key in seen:
            aliases[name] = seen[key]          # a tied tensor: stored once
            continue
        seen[key] = name
        tensors[name] = tensor.detach().to("cpu").contiguous()

    os.makedirs(folder, exist_ok=True)
    config = getattr(model, "config", None)
    if config is not None and hasattr(config, "save_pretrained"):
        config.save_pretrained(folder)
    meta = {
        "format": FORMAT_TAG,
        "group_size": groups.pop(),
        "modules": {name: {"in_features": m.in_features, "out_features": m.out_features,
                           "bias": m.bias is not None} for name, m in quantized.items()},
        "aliases": aliases,
    }
    save_file(tensors, os.path.join(folder, WEIGHTS_FILE), metadata={"format": FORMAT_TAG})
    with open(os.path.join(folder, META_FILE), "w") as fh:
        json.dump(meta, fh, indent=1, sort_keys=True)
    return meta


@torch.no_grad()
def load_w4a16_checkpoint(folder: str, *, device, dtype: torch.dtype = torch.float16,
                          model: nn.Module | None = None) -> tuple[nn.Module, W4A16Report]:
    """Load a folder written by ``save_w4a16_checkpoint`` straight into packed modules.

    The model skeleton is built on ``meta`` from ``config.json`` (or taken from ``model``, for
    architectures ``transformers`` does not know), the modules the metadata names become
    ``W4A16Linear`` shells, and every tensor goes from the file to ``device`` as it is: no
    fp16 weight exists and no quantizer runs.
    """
    from safetensors import safe_open

    device = torch.device(device)
    meta_path = os.path.join(folder, META_FILE)
    if not os.path.exists(meta_path):
        raise FileNotFoundError(f"{meta_path} is missing: not a pre-quantized checkpoint")
    with open(meta_path) as fh:
        meta = json.load(fh)
    if meta.get("format") != FORMAT_TAG:
        raise ValueError(f"unknown checkpoint format {meta.get('format')!r} (expected {FORMAT_TAG!r})")
    group_size = int(meta["group_size"])

    config = None
    if model is None:
        from transformers import AutoConfig, AutoModelForCausalLM

        config = AutoConfig.from_pretrained(folder)
        with torch.device("meta"):
            model = AutoModelForCausalLM.from_config(config, dtype=dtype)
    else:
        config = getattr(model, "config", None)
    model.eval()

    report = W4A16Report()
    shells: dict[str, W4A16Linear] = {}
    for name, spec in meta["modules"].items():
        try:
            current = model.get_submodule(name)
        except AttributeError as exc:
            raise ValueError(f"checkpoint names a module the model does not have: {name}") from exc
        if isinstance(current, nn.Linear) and (current.in_features != spec["in_features"]
                                               or current.out_features != spec["out_features"]):
            raise ValueError(f"{name}: checkpoint is [{spec['out_features']}, {spec['in_features']}], "
                             f"model is [{current.out_features}, {current.in_features}]")
        shell = W4A16Linear(spec["in_features"], spec["out_features"], group_size=group_size,
                            bias=bool(spec["bias"]), device="meta")
        owner, attribute = _parent(model, name)
        setattr(owner, attribute, shell)
        shells[name] = shell
        kind = "lm_head" if attribute == "lm_head" else ("mlp" if attribute.endswith(("gate_proj", "up_proj", "down_proj")) else "attention")
        report.count(kind, spec["in_features"], spec["out_features"], group_size)

    expected_dtype = {"packed": torch.uint8, "scales": torch.float16}
    homeless, loaded = [], {}
    with safe_open(os.path.join(folder, WEIGHTS_FILE), framework="pt", device="cpu") as shard:
        for key in shard.keys():
            tensor = shard.get_tensor(key)
            owner_name, _, leaf = key.rpartition(".")
            shell = shells.get(owner_name)
            if shell is not None and leaf in ("packed", "scales", "bias"):
                want = getattr(shell, leaf)
                if want is None or tuple(want.shape) != tuple(tensor.shape) \
                        or (leaf in expected_dtype and tensor.dtype is not expected_dtype[leaf]):
                    raise ValueError(f"{key}: stored {tuple(tensor.shape)} {tensor.dtype} does not fit "
                                     f"the module")
                placed = tensor.to(device) if leaf != "bias" else tensor.to(device=device, dtype=torch.float16)
                setattr(shell, leaf, placed)
            else:
                placed = tensor.to(device=device, dtype=dtype if tensor.is_floating_point() else tensor.dtype)
                if not _assign(model, key, placed):
                    homeless.append(key)
                    continue
            loaded[key] = placed
    if homeless:
        raise ValueError(f"checkpoint tensors with no home in the model: {homeless[:8]}")
    for alias, source in meta.get("aliases", {}).items():
        if source not in loaded:
            raise ValueError(f"alias {alias} points at {source}, which the file does not hold")
        owner_name, _, leaf = alias.rpartition(".")
        shell = shells.get(owner_name)
        if shell is not None:
            setattr(shell, leaf, loaded[source])
        elif not _assign(model, alias, loaded[source]):
            raise ValueError(f"alias {alias} has no home in the model")

    if config is not None:
        _reinit_rotary(model, config, device)
    leftover = _meta_tensors(model)
    if leftover:
        raise ValueError(f"tensors never loaded (still on meta): {leftover[:8]}"
                         + (" ..." if len(leftover) > 8 else ""))
    return model, report
