"""Random weights: a model folder from a configuration and a seed.

One documented generator, so that the same (configuration, seed) gives the
same bytes on every machine: a counter-based splitmix64 stream per tensor
(seeded from the run's seed and a hash of the tensor's name, so the order in
which tensors are made does not matter), two 53-bit uniforms per pair of
normals, Box-Muller in float64, then rounding to the stored dtype.
Matrices and embeddings are N(0, std); norm weights are 1 + N(0, norm_noise).
The reference has no such mode (its tests use real weights; the nearest
precedent is the synthetic two-layer model of engine/tests/unit_tests.c:2180-2335).
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Sequence

import numpy as np
import torch

from .loader import WeightSpec
from .safetensors_io import write_safetensors

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)


def _mix(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def _name_hash(name: str) -> int:
    h = 0xCBF29CE484222325  # FNV-1a, 64 bit
    for b in name.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def normal(name: str, seed: int, count: int) -> np.ndarray:
    """`count` standard normals (float64) for the tensor `name` under `seed`."""
    with np.errstate(over="ignore"):
        start = _mix(np.array([(seed & 0xFFFFFFFFFFFFFFFF) ^ _name_hash(name)], dtype=np.uint64))[0]
        pairs = (count + 1) // 2
        idx = np.arange(1, 2 * pairs + 1, dtype=np.uint64)
        bits = _mix(start + idx * _GOLDEN)
    u = ((bits >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / 9007199254740992.0)  # (0, 1)
    r = np.sqrt(-2.0 * np.log(u[0::2]))
    t = 2.0 * np.pi * u[1::2]
    return np.stack([r * np.cos(t), r * np.sin(t)], axis=1).reshape(-1)[:count]


def random_weights(manifest: Sequence[WeightSpec], seed: int, *, is_norm: Callable[[str], bool],
                   std: float = 0.02, norm_noise: float = 0.0,
                   matrix_dtype: torch.dtype = torch.bfloat16,
                   norm_dtype: torch.dtype = torch.float32) -> Dict[str, torch.Tensor]:
    out = {}
    for w in manifest:
        if w.optional:
            continue
        n = int(np.prod(w.shape))
        z = normal(w.name, seed, n).reshape(w.shape)
        if is_norm(w.name):
            out[w.name] = torch.from_numpy((1.0 + norm_noise * z).astype(np.float32)).to(norm_dtype)
        else:
            out[w.name] = torch.from_numpy((std * z).astype(np.float32)).to(matrix_dtype)
    return out


def write_model_folder(model_dir: str, config_json: dict, tensors: Dict[str, torch.Tensor]) -> None:
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_json, f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors)
