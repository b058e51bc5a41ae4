"""Names of the kinds of parts, so that a configuration can choose them layer by layer.

A builder (see models/) turns a list of LayerSpec into blocks by looking the
names up here.  Registering a new kind is one call; nothing else changes.
"""
from __future__ import annotations

from typing import Callable, Dict

MIXERS: Dict[str, Callable] = {}
FEED_FORWARDS: Dict[str, Callable] = {}
NORMS: Dict[str, Callable] = {}
POSITION_ENCODINGS: Dict[str, Callable] = {}
BLOCKS: Dict[str, Callable] = {}

_KINDS = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS, "position": POSITION_ENCODINGS, "block": BLOCKS}


def register_part(kind: str, name: str, factory: Callable) -> None:
    """factory(**params) -> the part.  `kind` is one of mixer, feed_forward, norm, position, block."""
    if kind not in _KINDS:
        raise KeyError(f"unknown kind of part {kind!r}; kinds are {sorted(_KINDS)}")
    _KINDS[kind][name] = factory


def make_part(kind: str, name: str, **params):
    table = _KINDS[kind]
    if name not in table:
        raise KeyError(f"no {kind} named {name!r}; registered: {sorted(table)}")
    return table[name](**params)


def _register_builtin() -> None:
    from .attention import PagedAttention
    from .block import PreNormBlock
    from .feed_forward import SwiGLU
    from .norms import RMSNorm
    from .rotary import NoPositionEncoding, Rotary
    register_part("mixer", "attention", PagedAttention)
    register_part("feed_forward", "swiglu", SwiGLU)
    register_part("norm", "rmsnorm", RMSNorm)
    register_part("position", "rotary", Rotary)
    register_part("position", "none", NoPositionEncoding)
    register_part("block", "pre_norm", PreNormBlock)


_register_builtin()
