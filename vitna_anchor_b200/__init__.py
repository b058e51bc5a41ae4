"""A small, whole inference engine for one GPU (B200, sm_100a): the dense Llama decoder.

From a model folder (config.json, model.safetensors) to generated tokens:
typed configuration and registry (config/), weights by name (weights/), layers
put together from parts (parts/, models/), a paged cache with state slots
(cache/), one step function and a scheduler (engine/), sampling (sampling/),
and hand-written CUDA kernels (csrc/, ops/).
"""
from .config import registry as _registry

_registry._register_builtin()

__version__ = "0.1.0"
