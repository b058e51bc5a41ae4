"""Configuration: keys, defaults, refusals, and the registry."""
import json

import pytest

from vitna_anchor_b200.config import ConfigError, LlamaConfig, architectures, read_config_json, resolve
from tiny_configs import TINY_A, TINY_B


def test_reads_every_size_from_config():
    for tiny in (TINY_A, TINY_B):
        c = LlamaConfig.from_dict(tiny["config"])
        j = tiny["config"]
        assert (c.num_hidden_layers, c.hidden_size, c.intermediate_size) == (j["num_hidden_layers"], j["hidden_size"], j["intermediate_size"])
        assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (j["num_attention_heads"], j["num_key_value_heads"], j["head_dim"])
        assert (c.vocab_size, c.max_position_embeddings) == (j["vocab_size"], j["max_position_embeddings"])
        assert (c.rms_norm_eps, c.rope_theta, c.tie_word_embeddings) == (j["rms_norm_eps"], j["rope_theta"], j["tie_word_embeddings"])


def test_defaults():
    j = {k: v for k, v in TINY_A["config"].items() if k not in ("num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "tie_word_embeddings")}
    c = LlamaConfig.from_dict(j)
    assert c.num_key_value_heads == c.num_attention_heads
    assert c.head_dim == c.hidden_size // c.num_attention_heads
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0 and c.tie_word_embeddings is False


@pytest.mark.parametrize("change, word", [
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "linear", "factor": 2.0}}, "rope_scaling"),
    ({"attention_bias": True}, "biases"),
    ({"mlp_bias": True}, "biases"),
    ({"rope_interleaved": True}, "rope_interleaved"),
    ({"pretraining_tp": 2}, "pretraining_tp"),
    ({"num_key_value_heads": 3}, "key-value groups"),
    ({"head_dim": 15}, "head_dim is odd"),
    ({"hidden_size": None}, "hidden_size is missing"),
    ({"vocab_size": 0}, "vocab_size is not a positive integer"),
    ({"num_hidden_layers": 2.5}, "num_hidden_layers is not a positive integer"),
    ({"model_type": "gpt2", "architectures": ["GPT2LMHeadModel"]}, "registered architectures"),
])
def test_refusals_name_the_key(change, word):
    j = dict(TINY_A["config"]); j.update(change)
    with pytest.raises(ConfigError) as e:
        resolve(j).parse_config(j)
    assert word in str(e.value)


def test_registry_by_architecture_and_model_type():
    assert "LlamaForCausalLM" in architectures()
    assert resolve({"architectures": ["LlamaForCausalLM"]}).name == "LlamaForCausalLM"
    assert resolve({"model_type": "llama"}).name == "LlamaForCausalLM"
    with pytest.raises(ConfigError) as e:
        resolve({"architectures": ["MixtralForCausalLM"], "model_type": "mixtral"})
    assert "LlamaForCausalLM" in str(e.value)


def test_config_json_errors(tmp_path):
    with pytest.raises(ConfigError):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(TINY_B["config"]))
    assert LlamaConfig.from_dict(read_config_json(str(tmp_path))).num_hidden_layers == 3


def test_to_dict_round_trip():
    c = LlamaConfig.from_dict(TINY_B["config"])
    assert LlamaConfig.from_dict(c.to_dict()) == c
