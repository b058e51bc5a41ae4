"""Weights: safetensors reading and writing, binding by name, one error for everything that is wrong,
and the random-weights mode."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from vitna_anchor_b200.config import read_config_json, resolve
from vitna_anchor_b200.weights import (CheckpointError, SafetensorsFile, WeightMismatch, load_weights,
                                       write_safetensors)
from vitna_anchor_b200.weights.random_init import normal
from tiny_configs import TINY_A, TINY_B, write_tiny


def _manifest(model_dir):
    cj = read_config_json(model_dir)
    arch = resolve(cj)
    return arch.manifest(arch.parse_config(cj))


def test_round_trip_keeps_stored_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t)
    f = SafetensorsFile(p)
    assert f.read("a").dtype == torch.bfloat16 and torch.equal(f.read("a"), t["a"])
    assert f.read("b").dtype == torch.float32 and torch.equal(f.read("b"), t["b"])
    assert f.read("c").dtype == torch.int32 and torch.equal(f.read("c"), t["c"])
    f.close()


def test_loader_keeps_bf16_and_f32(tiny_dirs):
    wa = load_weights(tiny_dirs["tinyA"], _manifest(tiny_dirs["tinyA"]))
    assert wa["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16
    assert wa["model.norm.weight"].dtype == torch.float32          # stored in 32-bit, stays so
    assert "lm_head.weight" not in wa                               # tied: the embedding stands in
    wb = load_weights(tiny_dirs["tinyB"], _manifest(tiny_dirs["tinyB"]))
    assert wb["model.layers.2.mlp.down_proj.weight"].dtype == torch.float32
    assert wb["lm_head.weight"].shape == (384, 96)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path, tiny_dirs):
    src = SafetensorsFile(os.path.join(tiny_dirs["tinyB"], "model.safetensors"))
    tensors = {n: src.read(n) for n in src.names()}
    src.close()
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    tensors["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(64, 96)
    d = tmp_path / "broken"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(TINY_B["config"]))
    write_safetensors(str(d / "model.safetensors"), tensors)
    with pytest.raises(WeightMismatch) as e:
        load_weights(str(d), _manifest(str(d)))
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "lm_head.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert len(err.wrong_shape) == 1 and "k_proj" in err.wrong_shape[0] and "[32, 96]" in err.wrong_shape[0]
    msg = str(err)
    assert "missing tensors (2)" in msg and "unexpected tensors (1)" in msg and "wrong shapes (1)" in msg


def test_extra_tensors_alone_load_with_a_warning(tmp_path, tiny_dirs):
    """The reference binds by name and ignores the rest (engine/src/model.c:265-283): an old export's
    rotary_emb.inv_freq buffer must not refuse the checkpoint."""
    src = SafetensorsFile(os.path.join(tiny_dirs["tinyB"], "model.safetensors"))
    tensors = {n: src.read(n) for n in src.names()}
    src.close()
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    d = tmp_path / "extra"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(TINY_B["config"]))
    write_safetensors(str(d / "model.safetensors"), tensors)
    with pytest.warns(UserWarning, match="rotary_emb.inv_freq"):
        got = load_weights(str(d), _manifest(str(d)))
    assert "model.layers.0.self_attn.rotary_emb.inv_freq" not in got and len(got) == len(tensors) - 1


def test_malformed_files_are_refused(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(CheckpointError):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(CheckpointError):
        SafetensorsFile(str(p))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(CheckpointError) as e:
        SafetensorsFile(str(p))
    assert "do not match" in str(e.value)
    hdr = json.dumps({"t": {"dtype": "Q4", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(CheckpointError):
        SafetensorsFile(str(p))
    with pytest.raises(CheckpointError):
        load_weights(str(tmp_path / "nowhere"), [])


def test_sharded_checkpoint(tmp_path, tiny_dirs):
    src = SafetensorsFile(os.path.join(tiny_dirs["tinyA"], "model.safetensors"))
    names = src.names()
    half = len(names) // 2
    d = tmp_path / "sharded"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(TINY_A["config"]))
    write_safetensors(str(d / "s1.safetensors"), {n: src.read(n) for n in names[:half]})
    write_safetensors(str(d / "s2.safetensors"), {n: src.read(n) for n in names[half:]})
    wm = {n: "s1.safetensors" for n in names[:half]}
    wm.update({n: "s2.safetensors" for n in names[half:]})
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    w = load_weights(str(d), _manifest(str(d)))
    assert torch.equal(w[names[0]], src.read(names[0])) and torch.equal(w[names[-1]], src.read(names[-1]))
    src.close()


def test_random_weights_are_reproducible_and_distributed(tmp_path):
    a = write_tiny(str(tmp_path / "a"), TINY_B)
    b = write_tiny(str(tmp_path / "b"), TINY_B)
    assert open(os.path.join(a, "model.safetensors"), "rb").read() == open(os.path.join(b, "model.safetensors"), "rb").read()
    z = normal("some.tensor", 3, 200001)
    assert abs(z.mean()) < 0.01 and abs(z.std() - 1.0) < 0.01 and len(z) == 200001
    assert not np.allclose(normal("some.tensor", 3, 8), normal("other.tensor", 3, 8))
    w = load_weights(b, _manifest(b))
    assert abs(float(w["model.embed_tokens.weight"].float().std()) - 0.02) < 0.002
    n = w["model.layers.0.input_layernorm.weight"]
    assert abs(float(n.mean()) - 1.0) < 0.05 and 0.05 < float(n.std()) < 0.15
