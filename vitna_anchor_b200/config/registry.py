"""One registry from an architecture's name to what builds it.

config.json's `architectures[0]` chooses the entry (the reference compares
`model_type` instead, engine/src/model.c:61-75; that key is the fallback here).
An entry gives: how to read the typed configuration, the manifest of tensors,
how to build the model from host tensors, and which tensors random
initialisation treats as norm weights.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Mapping

from .errors import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], Any]        # config.json dict -> typed configuration
    manifest: Callable[[Any], List]                         # configuration -> [WeightSpec]
    build: Callable[..., Any]                               # (configuration, host tensors, dtype, device) -> DecoderModel
    is_norm_weight: Callable[[str], bool] = lambda name: False
    model_types: tuple = ()                                 # values of config.json's model_type that also choose it


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {arch.name} is already registered")
    _ARCHITECTURES[arch.name] = arch


def architectures() -> List[str]:
    return sorted(_ARCHITECTURES)


def resolve(config_json: Mapping[str, Any]) -> Architecture:
    names = config_json.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    mt = config_json.get("model_type")
    if not names:
        for arch in _ARCHITECTURES.values():
            if mt is not None and mt in arch.model_types:
                return arch
    asked = names[0] if names else (f"model_type {mt}" if mt else "nothing")
    raise ConfigError(f"config.json names {asked}; the registered architectures are: {', '.join(architectures())}")


def _register_builtin() -> None:
    from ..models.llama import build_llama, is_norm_weight, llama_manifest
    from .llama import LlamaConfig
    register_architecture(Architecture("LlamaForCausalLM", LlamaConfig.from_dict, llama_manifest, build_llama,
                                       is_norm_weight, model_types=("llama",)), replace=True)
