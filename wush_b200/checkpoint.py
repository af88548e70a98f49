"""Quantized checkpoints on disk, in the reference's export format.

Writer: what ``export_quantized_model`` (model_quant.py:47-128) produces from the dictionaries
``wush_quantization_gptq`` returns -- safetensors shards of at most ``max_shard_size`` bytes named
``model-0000i-of-0000n.safetensors``, ``model.safetensors.index.json`` mapping every tensor to its shard, and the
``quantization_config`` of src/quantization/qconfig.py:3-23 inside ``config.json``.  Per quantized linear layer the
tensors are those of wush_gptq.py:592-599: ``qweight`` u8 [out, in/2], ``scales`` u8 [out, in/G] (row-major),
``forward_hadamard_matrix`` = ``backward_hadamard_matrix`` [G, in] in the model dtype, ``weight_global_scale`` and
``act_global_scale`` fp32 [1].

Reader: ``load_checkpoint`` walks the index and ``load_quantized_layers`` fills ``FPQuantLinear`` modules through
their state dict (the reference leaves this to a fork of the transformers loader); the blocked weight-scale layout
the GEMM consumes is derived once per layer on first use, not stored.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Iterable, Optional, Tuple

import torch

QUANT_TENSORS = ("qweight", "scales", "forward_hadamard_matrix", "backward_hadamard_matrix", "weight_global_scale",
                 "act_global_scale")
INDEX_NAME = "model.safetensors.index.json"


def prepare_quantization_config(hadamard_group_size: int, format: str, pseudoquantization: bool = False,
                                transform_init: str = "hadamard") -> Dict[str, Any]:
    """The dictionary stored as ``config.quantization_config`` (src/quantization/qconfig.py:3-23)."""
    if format not in ("mxfp", "nvfp"):
        raise ValueError(f"Invalid format: {format}")
    return {
        "forward_dtype": f"{format}4",
        "backward_dtype": "bf16",
        "forward_method": "abs_max",
        "hadamard_group_size": hadamard_group_size,
        "modules_to_not_convert": ["lm_head"],
        "quant_method": "fp_quant",
        "store_master_weights": False,
        "pseudoquantization": pseudoquantization,
        "transform_init": transform_init,
    }


def flatten_state(quantized_state_dict: Dict[str, Dict[str, torch.Tensor]],
                  other_tensors: Optional[Dict[str, torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
    """{layer name: {tensor name: tensor}} + plain tensors -> one flat ``name -> CPU tensor`` dictionary, quantized
    layers first in their given order (model_quant.py:57-76 walks the blocks in order)."""
    flat: Dict[str, torch.Tensor] = {}
    for layer, entry in quantized_state_dict.items():
        for k, v in entry.items():
            flat[f"{layer}.{k}"] = v.detach().cpu().contiguous()
    for k, v in (other_tensors or {}).items():
        flat[k] = v.detach().cpu().contiguous()
    return flat


def split_into_shards(tensors: Dict[str, torch.Tensor], max_shard_size: int) -> list:
    """The reference's greedy split (model_quant.py:83-103): tensors in order, a new shard when the next tensor
    would overflow, a tensor larger than the limit in a shard of its own."""
    shards, current, size = [], {}, 0
    for k, v in tensors.items():
        nbytes = v.numel() * v.element_size()
        if size + nbytes > max_shard_size:
            shards.append(current)
            current, size = {}, 0
        if nbytes > max_shard_size:
            shards.append({k: v})
            continue
        current[k] = v
        size += nbytes
    if current:
        shards.append(current)
    return [s for s in shards if s]


def export_quantized_model(save_path: str, quantized_state_dict: Dict[str, Dict[str, torch.Tensor]],
                           other_tensors: Optional[Dict[str, torch.Tensor]] = None,
                           model_config: Optional[Dict[str, Any]] = None, *, hadamard_group_size: int = 32,
                           format: str = "mxfp", transform_class: str = "wush",
                           max_shard_size: int = 5 * 1024 ** 3) -> Dict[str, str]:
    """Write the checkpoint directory; returns the tensor -> shard file map."""
    from safetensors.torch import save_file
    os.makedirs(save_path, exist_ok=True)
    shards = split_into_shards(flatten_state(quantized_state_dict, other_tensors), max_shard_size)
    digits = len(str(max(len(shards), 1)))
    weight_map: Dict[str, str] = {}
    for i, shard in enumerate(shards):
        name = f"model-{str(i + 1).zfill(digits)}-of-{str(len(shards)).zfill(digits)}.safetensors"
        save_file(shard, os.path.join(save_path, name))
        for k in shard:
            weight_map[k] = name
    with open(os.path.join(save_path, INDEX_NAME), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    config = dict(model_config or {})
    config["quantization_config"] = prepare_quantization_config(
        hadamard_group_size, format, pseudoquantization=False,
        transform_init="wush" if transform_class == "wush" else transform_class)
    with open(os.path.join(save_path, "config.json"), "w") as f:
        json.dump(config, f, indent=2)
    return weight_map


def load_checkpoint(path: str, names: Optional[Iterable[str]] = None,
                    device: str = "cpu") -> Tuple[Dict[str, torch.Tensor], Dict[str, Any]]:
    """(tensors, quantization_config) of a checkpoint directory; `names` restricts the tensors that are read."""
    from safetensors import safe_open
    with open(os.path.join(path, INDEX_NAME)) as f:
        weight_map = json.load(f)["weight_map"]
    with open(os.path.join(path, "config.json")) as f:
        qcfg = json.load(f).get("quantization_config", {})
    wanted = set(names) if names is not None else None
    by_file: Dict[str, list] = {}
    for k, fname in weight_map.items():
        if wanted is None or k in wanted:
            by_file.setdefault(fname, []).append(k)
    out: Dict[str, torch.Tensor] = {}
    for fname, keys in by_file.items():
        with safe_open(os.path.join(path, fname), framework="pt", device=device) as f:
            for k in keys:
                out[k] = f.get_tensor(k)
    return out, qcfg


def config_from_checkpoint(qcfg: Dict[str, Any]):
    """FPQuantConfig for the layers of a checkpoint written with `quantization_config` qcfg."""
    from .linear import FPQuantConfig, FPQuantDtype
    if qcfg.get("quant_method", "fp_quant") != "fp_quant" or qcfg.get("pseudoquantization", False):
        raise NotImplementedError("only real-quant fp_quant checkpoints are loaded")
    return FPQuantConfig(forward_dtype=FPQuantDtype(qcfg["forward_dtype"]), forward_method=qcfg.get("forward_method", "abs_max"),
                         hadamard_group_size=int(qcfg["hadamard_group_size"]),
                         transform_init=qcfg.get("transform_init", "hadamard"),
                         modules_to_not_convert=list(qcfg.get("modules_to_not_convert", ["lm_head"])))


def load_quantized_layers(path: str, layers: Optional[Dict[str, Any]] = None, device="cuda", bias: bool = False) -> Dict[str, Any]:
    """Fill FPQuantLinear modules from a checkpoint directory.

    layers: {layer name: FPQuantLinear} to fill; None: one module is created per quantized layer found in the index
    (shapes from the stored tensors).  Returns the dictionary of modules.  Every module goes through the same steps
    as in the reference's loading flow: buffers copied in by ``load_state_dict``, then ``pre_forward()``."""
    from .linear import FPQuantLinear
    with open(os.path.join(path, INDEX_NAME)) as f:
        weight_map = json.load(f)["weight_map"]
    found = sorted({k.rsplit(".", 1)[0] for k in weight_map if k.endswith(".qweight")})
    names = found if layers is None else list(layers)
    tensors, qcfg = load_checkpoint(path, [f"{n}.{t}" for n in names for t in QUANT_TENSORS])
    cfg = config_from_checkpoint(qcfg)
    out = {}
    for n in names:
        entry = {t: tensors[f"{n}.{t}"] for t in QUANT_TENSORS if f"{n}.{t}" in tensors}
        if "qweight" not in entry:
            raise KeyError(f"{n}: no quantized tensors in the checkpoint")
        if layers is None:
            rows, half = entry["qweight"].shape
            mod = FPQuantLinear(half * 2, rows, cfg, bias=bias, device=device, dtype=entry["forward_hadamard_matrix"].dtype)
        else:
            mod = layers[n]
        mod.load_state_dict(entry, strict=False)
        mod.pre_forward()
        out[n] = mod
    return out
