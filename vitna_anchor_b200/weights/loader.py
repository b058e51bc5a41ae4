"""Binding a model's weights by tensor name.

An architecture gives a manifest: the names it needs, their shapes, and
which names may be absent (a tied output matrix).  The loader opens
`model.safetensors`, or the shards that `model.safetensors.index.json`
names (engine/src/model.c:196-263), and returns host tensors in their
stored dtype.  Every mismatch is collected and reported in ONE error that
lists missing tensors, unexpected tensors and wrong shapes
(the reference stops at the first, engine/src/model.c:265-283).  Tensors the
model does not name are not an error by themselves: the reference binds by
name and never looks at the rest (older exports carry rotary_emb.inv_freq
buffers, for instance), so a checkpoint whose only difference is extra tensors
loads, with a warning that names them.
"""
from __future__ import annotations

import json
import os
import warnings
from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

import torch

from .safetensors_io import CheckpointError, SafetensorsFile


@dataclass(frozen=True)
class WeightSpec:
    name: str
    shape: Tuple[int, ...]
    optional: bool = False      # may be absent (the model says what stands in for it)
    floating: bool = True       # floating-point tensors; False for integer tables


class WeightMismatch(CheckpointError):
    """The checkpoint does not hold what the model needs."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str], wrong: List[str]):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong
        parts = [f"{where} does not fit the model:"]
        if missing:
            parts.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            parts.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            parts.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(parts))


def _open_shards(model_dir: str) -> List[SafetensorsFile]:
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.exists(single):
        return [SafetensorsFile(single)]
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if not os.path.exists(index):
        raise CheckpointError(f"{model_dir} has neither model.safetensors nor model.safetensors.index.json")
    with open(index, "r", encoding="utf-8") as f:
        weight_map = json.load(f).get("weight_map")
    if not isinstance(weight_map, dict):
        raise CheckpointError(f"{index}: weight_map is missing")
    files = sorted(set(weight_map.values()))
    for name in files:
        if not isinstance(name, str) or os.path.basename(name) != name:  # plain file names only
            raise CheckpointError(f"{index}: {name!r} is not a plain file name")
    shards = [SafetensorsFile(os.path.join(model_dir, name)) for name in files]
    by_file = dict(zip(files, shards))
    for tensor, fname in weight_map.items():
        if tensor not in by_file[fname].entries:
            raise CheckpointError(f"{index}: {fname} does not hold tensor {tensor}")
    return shards


def load_weights(model_dir: str, manifest: Sequence[WeightSpec]) -> Dict[str, torch.Tensor]:
    """Host tensors by name: bfloat16 and float32 stay as stored, float16 is
    widened to float32, integer tables are int32."""
    shards = _open_shards(model_dir)
    try:
        where = {}
        for sh in shards:
            for name in sh.entries:
                where[name] = sh
        wanted = {w.name: w for w in manifest}
        missing = [w.name for w in manifest if w.name not in where and not w.optional]
        unexpected = sorted(n for n in where if n not in wanted)
        wrong = []
        for w in manifest:
            sh = where.get(w.name)
            if sh is None:
                continue
            e = sh.entries[w.name]
            if tuple(e.shape) != tuple(w.shape):
                wrong.append(f"{w.name} is {list(e.shape)}, the model needs {list(w.shape)}")
            elif w.floating != (e.dtype in ("F32", "BF16", "F16")):
                wrong.append(f"{w.name} has dtype {e.dtype}")
        if missing or wrong:
            raise WeightMismatch(model_dir, missing, unexpected, wrong)
        if unexpected:
            shown = ", ".join(unexpected[:8]) + (f", ... ({len(unexpected)} in all)" if len(unexpected) > 8 else "")
            warnings.warn(f"{model_dir}: tensors the model does not use are ignored: {shown}", stacklevel=2)
        out = {}
        for w in manifest:
            if w.name in where:
                t = where[w.name].read(w.name)
                out[w.name] = t.float() if t.dtype == torch.float16 else t
        return out
    finally:
        for sh in shards:
            sh.close()
