"""From a model folder to a model on the device, and the random-weights mode."""
from __future__ import annotations

from typing import Any, Mapping, Optional, Union

import torch

from ..config import read_config_json, resolve
from ..weights import load_weights, random_weights, write_model_folder

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def compute_dtype(name) -> torch.dtype:
    try:
        return _DTYPES[name]
    except KeyError:
        raise ValueError(f"dtype is bfloat16 or float32, not {name}") from None


def load_model(model_dir: str, dtype="bfloat16", device="cuda"):
    """config.json chooses the architecture; model.safetensors gives the tensors by name."""
    cfg_json = read_config_json(model_dir)
    arch = resolve(cfg_json)
    cfg = arch.parse_config(cfg_json)
    weights = load_weights(model_dir, arch.manifest(cfg))
    return arch.build(cfg, weights, compute_dtype(dtype), device)


def write_random_model(model_dir: str, config_json: Mapping[str, Any], seed: int, *, std: float = 0.02,
                       norm_noise: float = 0.0, matrix_dtype: torch.dtype = torch.bfloat16,
                       norm_dtype: torch.dtype = torch.float32) -> None:
    """Write config.json and model.safetensors for the architecture that config_json names: matrices and
    embeddings N(0, std), norm weights 1 + N(0, norm_noise), from `seed` (see weights/random_init.py)."""
    arch = resolve(config_json)
    cfg = arch.parse_config(config_json)
    tensors = random_weights(arch.manifest(cfg), seed, is_norm=arch.is_norm_weight, std=std, norm_noise=norm_noise,
                             matrix_dtype=matrix_dtype, norm_dtype=norm_dtype)
    out_json = cfg.to_dict() if hasattr(cfg, "to_dict") else dict(config_json)
    write_model_folder(model_dir, out_json, tensors)


def random_model_on_device(config_json: Mapping[str, Any], seed: int, dtype="bfloat16", device="cuda", std: float = 0.02):
    """A model of the architecture config_json names with weights drawn on the device by torch's generator
    (matrices N(0, std), norm weights 1): for throughput measurements of sizes whose checkpoint would take a
    minute to write and read.  No folder is made, and the bits are torch's, not those of write_random_model."""
    arch = resolve(config_json)
    cfg = arch.parse_config(config_json)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    weights = {}
    for w in arch.manifest(cfg):
        if w.optional:
            continue
        if arch.is_norm_weight(w.name):
            weights[w.name] = torch.ones(w.shape, dtype=torch.float32, device=device)
        else:
            t = torch.empty(w.shape, dtype=torch.float32 if len(w.shape) < 2 else torch.bfloat16, device=device)
            t.normal_(0.0, std, generator=gen)
            weights[w.name] = t
    return arch.build(cfg, weights, compute_dtype(dtype), device)
