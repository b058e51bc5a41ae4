"""A small, whole inference engine for one GPU (B200, sm_100a): the dense Llama decoder.

From a model folder (config.json, model.safetensors) to generated tokens:
typed configuration and registry (config/), weights by name (weights/), layers
put together from parts (parts/, models/), a paged cache with state slots
(cache/), one step function and a scheduler (engine/), sampling (sampling/),
and hand-written CUDA kernels (csrc/, ops/).
"""
from .config import registry as _registry

_registry._register_builtin()


def _load_plugins() -> None:
    """Modules named in VITNA_ANCHOR_PLUGINS (comma-separated, importable names) are imported once the built-in
    parts and architectures are registered.  A module registers its own parts and architectures when imported
    (register_part, register_architecture), which is how the command line and the replay program come to know
    an architecture that is defined outside this package."""
    import importlib
    import os
    for name in filter(None, (n.strip() for n in os.environ.get("VITNA_ANCHOR_PLUGINS", "").split(","))):
        importlib.import_module(name)


_load_plugins()

__version__ = "0.1.0"
