"""The dense Llama decoder (LlamaForCausalLM): manifest of its tensors and how its layers are built.

Tensor names and shapes are Hugging Face's, as the reference binds them
(engine/src/model.c:313-365).  q, k and v are stacked into one matrix and gate
and up into another when the model is built; nothing else is renamed.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.llama import LlamaConfig
from ..parts.registry import make_part
from ..parts.embedding import Embedding, LMHead
from ..weights.loader import WeightSpec
from .decoder import DecoderModel, LayerRun


def llama_manifest(cfg: LlamaConfig) -> List[WeightSpec]:
    H, I, V, qd, kvd = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.q_size, cfg.kv_size
    m = [WeightSpec("model.embed_tokens.weight", (V, H))]
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        m += [
            WeightSpec(p + "input_layernorm.weight", (H,)),
            WeightSpec(p + "self_attn.q_proj.weight", (qd, H)),
            WeightSpec(p + "self_attn.k_proj.weight", (kvd, H)),
            WeightSpec(p + "self_attn.v_proj.weight", (kvd, H)),
            WeightSpec(p + "self_attn.o_proj.weight", (H, qd)),
            WeightSpec(p + "post_attention_layernorm.weight", (H,)),
            WeightSpec(p + "mlp.gate_proj.weight", (I, H)),
            WeightSpec(p + "mlp.up_proj.weight", (I, H)),
            WeightSpec(p + "mlp.down_proj.weight", (H, I)),
        ]
    m.append(WeightSpec("model.norm.weight", (H,)))
    # The output matrix is used if the checkpoint has it; a tied model may leave it out (model.c:315-321).
    m.append(WeightSpec("lm_head.weight", (V, H), optional=cfg.tie_word_embeddings))
    return m


def is_norm_weight(name: str) -> bool:
    return name.endswith("layernorm.weight") or name == "model.norm.weight"


def build_llama(cfg: LlamaConfig, weights: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> DecoderModel:
    """Move the host tensors to the device in the compute dtype (a float32 tensor is rounded to nearest-even
    for the bfloat16 path; a bfloat16 tensor is widened exactly for the float32 path; norm weights are float32
    in both) and put the layers together."""
    dev = torch.device(device)

    def mat(*names: str) -> torch.Tensor:
        parts = [weights[n].to(device=dev, dtype=dtype) for n in names]
        return parts[0].contiguous() if len(parts) == 1 else torch.cat(parts, dim=0).contiguous()

    def vec(name: str) -> torch.Tensor:
        return weights[name].to(device=dev, dtype=torch.float32)

    H = cfg.hidden_size
    position = make_part("position", "rotary", head_dim=cfg.head_dim, theta=cfg.rope_theta,
                         max_positions=cfg.max_position_embeddings, device=dev)
    blocks = []
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        mixer = make_part("mixer", "attention", hidden=H, num_heads=cfg.num_attention_heads,
                          num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                          wqkv=mat(p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight", p + "self_attn.v_proj.weight"),
                          wo=mat(p + "self_attn.o_proj.weight"), position=position)
        ffn = make_part("feed_forward", "swiglu", hidden=H, intermediate=cfg.intermediate_size,
                        w_gate_up=mat(p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight"),
                        w_down=mat(p + "mlp.down_proj.weight"))
        blocks.append(make_part(
            "block", "pre_norm",
            mixer_norm=make_part("norm", "rmsnorm", width=H, eps=cfg.rms_norm_eps, weight=vec(p + "input_layernorm.weight")),
            mixer=mixer,
            ffn_norm=make_part("norm", "rmsnorm", width=H, eps=cfg.rms_norm_eps, weight=vec(p + "post_attention_layernorm.weight")),
            ffn=ffn))
    embedding = Embedding(cfg.vocab_size, H, mat("model.embed_tokens.weight"))
    head_w = mat("lm_head.weight") if "lm_head.weight" in weights else embedding.table
    if "lm_head.weight" not in weights and not cfg.tie_word_embeddings:
        raise ValueError("the checkpoint has no lm_head.weight and the embeddings are not tied")
    return DecoderModel(
        embedding=embedding, blocks=blocks,
        schedule=[LayerRun(block=l, cache=l) for l in range(cfg.num_hidden_layers)],
        final_norm=make_part("norm", "rmsnorm", width=H, eps=cfg.rms_norm_eps, weight=vec("model.norm.weight")),
        lm_head=LMHead(cfg.vocab_size, H, head_w), position=position, dtype=dtype, vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings, config=cfg)
