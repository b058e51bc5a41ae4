"""Typed configuration of the dense Llama decoder, read from config.json.

Keys, defaults and refusals follow the reference's reader
(engine/src/model.c:48-136, sizes checked as in cfg_size, model.c:28-40):
required are num_hidden_layers, hidden_size, intermediate_size,
num_attention_heads, vocab_size and max_position_embeddings; optional are
num_key_value_heads (default: the number of heads), head_dim (default:
hidden_size / heads), rms_norm_eps (1e-6), rope_theta (10000.0) and
tie_word_embeddings (false).  A configuration that asks for something the
engine cannot check is refused with the name of the key.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, asdict
from typing import Any, Mapping, Optional

from .errors import ConfigError


def _size(cfg: Mapping[str, Any], key: str, required: bool, default: Optional[int] = None) -> Optional[int]:
    # model.c:28-40: a size is a positive integer of at most 1e9.
    v = cfg.get(key)
    if v is None:
        if required:
            raise ConfigError(f"config.json: {key} is missing")
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)) or v < 1 or v > 1e9 or v != int(v):
        raise ConfigError(f"config.json: {key} is not a positive integer")
    return int(v)


def _false_or_missing(cfg: Mapping[str, Any], key: str) -> bool:
    v = cfg.get(key)
    return v is None or v is False


def _number(cfg: Mapping[str, Any], key: str, default: float) -> float:
    v = cfg.get(key)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {key} is not a number")
    return float(v)


@dataclass(frozen=True)
class LlamaConfig:
    """The eleven numbers that define one Llama model (model.h:46-65)."""

    num_hidden_layers: int
    hidden_size: int
    intermediate_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None

    architecture = "LlamaForCausalLM"

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "LlamaConfig":
        model_type = cfg.get("model_type")
        archs = cfg.get("architectures") or []
        if model_type != "llama" and "LlamaForCausalLM" not in archs:
            raise ConfigError(
                f"config.json: model_type is {model_type if model_type else 'missing'}, and only llama is supported")
        act = cfg.get("hidden_act")
        if act != "silu":  # model.c:82-83
            raise ConfigError(f"config.json: hidden_act is {act if act else 'missing'}, and only silu is supported")
        if cfg.get("rope_scaling") is not None:  # model.c:84-85
            raise ConfigError("config.json: rope_scaling is not supported")
        if not _false_or_missing(cfg, "attention_bias") or not _false_or_missing(cfg, "mlp_bias"):  # model.c:86-87
            raise ConfigError("config.json: attention and MLP biases are not supported")
        if not _false_or_missing(cfg, "rope_interleaved"):  # model.c:88-91
            raise ConfigError("config.json: rope_interleaved true is not supported")
        n_layers = _size(cfg, "num_hidden_layers", True)
        hidden = _size(cfg, "hidden_size", True)
        inter = _size(cfg, "intermediate_size", True)
        n_heads = _size(cfg, "num_attention_heads", True)
        vocab = _size(cfg, "vocab_size", True)
        max_pos = _size(cfg, "max_position_embeddings", True)
        n_kv = _size(cfg, "num_key_value_heads", False, n_heads)
        head_dim = _size(cfg, "head_dim", False, hidden // n_heads)
        tp = _size(cfg, "pretraining_tp", False, 1)
        if tp != 1:  # model.c:105-106
            raise ConfigError("config.json: pretraining_tp other than 1 is not supported")
        if n_heads % n_kv != 0 or head_dim % 2 != 0 or head_dim < 2:  # model.c:107-108
            raise ConfigError("config.json: heads do not divide into key-value groups, or head_dim is odd")
        tied = cfg.get("tie_word_embeddings")
        if tied is None:
            tied = False
        if not isinstance(tied, bool):
            raise ConfigError("config.json: tie_word_embeddings is not true or false")

        def token_id(key: str) -> Optional[int]:
            v = cfg.get(key)
            if isinstance(v, list):
                v = v[0] if v else None
            if v is None:
                return None
            if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                raise ConfigError(f"config.json: {key} is not a token id")
            return int(v)

        return cls(
            num_hidden_layers=n_layers, hidden_size=hidden, intermediate_size=inter,
            num_attention_heads=n_heads, num_key_value_heads=n_kv, head_dim=head_dim,
            vocab_size=vocab, max_position_embeddings=max_pos,
            rms_norm_eps=_number(cfg, "rms_norm_eps", 1e-6),
            rope_theta=_number(cfg, "rope_theta", 10000.0),
            tie_word_embeddings=tied,
            bos_token_id=token_id("bos_token_id"), eos_token_id=token_id("eos_token_id"))

    def to_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        d = asdict(self)
        d = {k: v for k, v in d.items() if v is not None}
        d.update(model_type="llama", architectures=[self.architecture], hidden_act="silu",
                 attention_bias=False, mlp_bias=False, rope_scaling=None, pretraining_tp=1)
        return d


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            cfg = json.load(f)
    except OSError as e:
        raise ConfigError(f"cannot read {path}: {e.strerror}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"config.json: {e}") from None
    if not isinstance(cfg, dict):
        raise ConfigError("config.json: the document is not an object")
    return cfg
