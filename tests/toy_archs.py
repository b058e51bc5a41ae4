"""Toy parts and architectures defined outside the framework, with a plain NumPy statement of each.

Importing this module registers them (it is also named in VITNA_ANCHOR_PLUGINS for the child processes that the
tests start, so that the command line and the replay program know them too).  None of them is anybody's model:

  ToyRunningMeanLM   a mixer with state of its own: the running mean of its inputs, kept per request in the
                     request's state slot.  It plans its work per segment on the host, so it is not capture-safe.
  ToyLearnedLM       a position encoding that adds a learned row per position to the embeddings (the attention then
                     rotates nothing); everything it launches depends on device arrays alone, so it is capture-safe.
  ToyRoutedLM        the same with a feed-forward with routing: a float32 router picks one of three SwiGLU experts
                     per token and weighs it by its softmax probability.  The routing reads the picks on the host,
                     so it is not capture-safe.
"""
import json

import numpy as np
import torch

import plain_llama as P
from vitna_anchor_b200 import ops
from vitna_anchor_b200.cache import StateSpec
from vitna_anchor_b200.config import Architecture, register_architecture
from vitna_anchor_b200.models.decoder import DecoderModel, LayerRun
from vitna_anchor_b200.parts import FeedForward, Mixer, PositionEncoding, make_part, register_part
from vitna_anchor_b200.parts.embedding import Embedding, LMHead
from vitna_anchor_b200.weights import WeightSpec

EXPERTS = 3


# ---------------------------------------------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------------------------------------------

class RunningMean(Mixer):
    """state = (sum of inputs so far [H], count); output_t = W (sum_t / count_t)."""

    capture_safe = False          # it reads the segments' lengths and slots on the host

    def __init__(self, hidden, w):
        self.hidden, self.w = hidden, w

    def tensors(self):
        return [self.w]

    def cache_spec(self):
        return StateSpec((self.hidden + 1,), torch.float32)

    def forward(self, xn, ctx, cache, residual, write_cache=True, norm=None):
        start = 0
        outs = []
        for n, slot in zip(ctx.host_seg_lens, ctx.host_seg_slots):
            st = cache.state[slot]
            x = xn[start:start + n].float()
            sums = st[:self.hidden] + torch.cumsum(x, 0)
            counts = st[self.hidden] + torch.arange(1, n + 1, device=x.device)
            outs.append(sums / counts[:, None])
            st[:self.hidden] = sums[-1]; st[self.hidden] = counts[-1]
            start += n
        mean = torch.cat(outs).to(xn.dtype).contiguous()
        ops.linear(mean, self.w, residual, ops.LINEAR_ACC_F32)


class LearnedPositions(PositionEncoding):
    def __init__(self, table):
        self.table = table                      # float32 [max_positions, hidden]

    def tensors(self):
        return [self.table]

    def on_embeddings(self, x, ctx):
        x += self.table[ctx.positions.long()]


class Top1Experts(FeedForward):
    capture_safe = False          # torch.nonzero brings the picks to the host

    def __init__(self, hidden, inter, router, gate_up, down):
        self.hidden, self.inter, self.router, self.gate_up, self.down = hidden, inter, router, gate_up, down

    def tensors(self):
        return [self.router] + self.gate_up + self.down

    def forward(self, xn, ctx, residual, norm=None):
        logits = xn.float() @ self.router.t()                       # router logits in float32
        prob = torch.softmax(logits, dim=-1)
        pick = torch.argmax(logits, dim=-1)                         # the lowest id among equal maxima
        for e in range(len(self.gate_up)):
            idx = torch.nonzero(pick == e).flatten()
            if idx.numel() == 0:
                continue
            xe = xn[idx].contiguous()
            gu = torch.empty(idx.numel(), 2 * self.inter, dtype=xn.dtype, device=xn.device)
            ops.linear(xe, self.gate_up[e], gu, ops.LINEAR_SAME)
            act = torch.empty(idx.numel(), self.inter, dtype=xn.dtype, device=xn.device)
            ops.silu_mul(gu, act)
            y = torch.empty(idx.numel(), self.hidden, dtype=torch.float32, device=xn.device)
            ops.linear(act, self.down[e], y, ops.LINEAR_F32)
            residual.index_add_(0, idx, y * prob[idx, e][:, None])


register_part("mixer", "toy_running_mean", RunningMean)
register_part("position", "toy_learned", LearnedPositions)
register_part("feed_forward", "toy_top1_experts", Top1Experts)


# ---------------------------------------------------------------------------------------------------------------
# ToyRunningMeanLM
# ---------------------------------------------------------------------------------------------------------------

def _rm_parse(cj):
    return dict(H=cj["hidden_size"], V=cj["vocab_size"], L=cj["num_hidden_layers"], I=cj["intermediate_size"])


def _rm_manifest(c):
    m = [WeightSpec("embed.weight", (c["V"], c["H"])), WeightSpec("norm.weight", (c["H"],))]
    for l in range(c["L"]):
        m += [WeightSpec(f"layers.{l}.mix.weight", (c["H"], c["H"])), WeightSpec(f"layers.{l}.norm1.weight", (c["H"],)),
              WeightSpec(f"layers.{l}.norm2.weight", (c["H"],)), WeightSpec(f"layers.{l}.gate_up.weight", (2 * c["I"], c["H"])),
              WeightSpec(f"layers.{l}.down.weight", (c["H"], c["I"]))]
    return m


def _rm_build(c, w, dtype, device):
    d = lambda n: w[n].to(device=device, dtype=dtype)
    f = lambda n: w[n].to(device=device, dtype=torch.float32)
    blocks = [make_part("block", "pre_norm",
                        mixer_norm=make_part("norm", "rmsnorm", width=c["H"], eps=1e-5, weight=f(f"layers.{l}.norm1.weight")),
                        mixer=make_part("mixer", "toy_running_mean", hidden=c["H"], w=d(f"layers.{l}.mix.weight")),
                        ffn_norm=make_part("norm", "rmsnorm", width=c["H"], eps=1e-5, weight=f(f"layers.{l}.norm2.weight")),
                        ffn=make_part("feed_forward", "swiglu", hidden=c["H"], intermediate=c["I"],
                                      w_gate_up=d(f"layers.{l}.gate_up.weight"), w_down=d(f"layers.{l}.down.weight")))
              for l in range(c["L"])]
    emb = Embedding(c["V"], c["H"], d("embed.weight"))
    return DecoderModel(embedding=emb, blocks=blocks, schedule=[LayerRun(l, l) for l in range(c["L"])],
                        final_norm=make_part("norm", "rmsnorm", width=c["H"], eps=1e-5, weight=f("norm.weight")),
                        lm_head=LMHead(c["V"], c["H"], emb.table), position=None, dtype=dtype, vocab_size=c["V"], max_positions=512)


register_architecture(Architecture("ToyRunningMeanLM", _rm_parse, _rm_manifest, _rm_build, lambda n: "norm" in n), replace=True)

RUNNING_MEAN_CONFIG = dict(architectures=["ToyRunningMeanLM"], hidden_size=24, vocab_size=50, num_hidden_layers=2, intermediate_size=40)


def plain_running_mean(model_dir, ids):
    """Logits [len(ids), V] of the running-mean model for one whole sequence."""
    W = {k: v.astype(np.float32) for k, v in P.read_safetensors(f"{model_dir}/model.safetensors").items()}
    c = _rm_parse(json.load(open(f"{model_dir}/config.json")))
    x = P.embed(W["embed.weight"], ids)
    n = np.arange(1, len(ids) + 1, dtype=np.float32)[:, None]
    for l in range(c["L"]):
        p = f"layers.{l}."
        xn = P.rms_norm(x, W[p + "norm1.weight"], 1e-5)
        x = x + P.linear((np.cumsum(xn, axis=0, dtype=np.float32) / n).astype(np.float32), W[p + "mix.weight"])
        xn = P.rms_norm(x, W[p + "norm2.weight"], 1e-5)
        gu = W[p + "gate_up.weight"]
        x = x + P.swiglu(xn, gu[:c["I"]], gu[c["I"]:], W[p + "down.weight"])
    return P.linear(P.rms_norm(x, W["norm.weight"], 1e-5), W["embed.weight"])


# ---------------------------------------------------------------------------------------------------------------
# ToyLearnedLM and ToyRoutedLM
# ---------------------------------------------------------------------------------------------------------------

def _lp_parse(cj):
    return dict(H=cj["hidden_size"], V=cj["vocab_size"], L=cj["num_hidden_layers"], I=cj["intermediate_size"],
                nh=cj["num_attention_heads"], nkv=cj["num_key_value_heads"], hd=cj["head_dim"], P=cj["max_position_embeddings"])


def _lp_manifest(routed):
    def manifest(c):
        m = [WeightSpec("embed.weight", (c["V"], c["H"])), WeightSpec("positions.weight", (c["P"], c["H"])), WeightSpec("norm.weight", (c["H"],))]
        for l in range(c["L"]):
            p = f"layers.{l}."
            m += [WeightSpec(p + "qkv.weight", ((c["nh"] + 2 * c["nkv"]) * c["hd"], c["H"])), WeightSpec(p + "o.weight", (c["H"], c["nh"] * c["hd"])),
                  WeightSpec(p + "norm1.weight", (c["H"],)), WeightSpec(p + "norm2.weight", (c["H"],))]
            if routed:
                m.append(WeightSpec(p + "router.weight", (EXPERTS, c["H"])))
                for e in range(EXPERTS):
                    m += [WeightSpec(p + f"experts.{e}.gate_up.weight", (2 * c["I"], c["H"])), WeightSpec(p + f"experts.{e}.down.weight", (c["H"], c["I"]))]
            else:
                m += [WeightSpec(p + "gate_up.weight", (2 * c["I"], c["H"])), WeightSpec(p + "down.weight", (c["H"], c["I"]))]
        return m
    return manifest


def _lp_build(routed):
    def build(c, w, dtype, device):
        d = lambda n: w[n].to(device=device, dtype=dtype).contiguous()
        f = lambda n: w[n].to(device=device, dtype=torch.float32)
        position = make_part("position", "toy_learned", table=f("positions.weight"))
        blocks = []
        for l in range(c["L"]):
            p = f"layers.{l}."
            if routed:
                ffn = make_part("feed_forward", "toy_top1_experts", hidden=c["H"], inter=c["I"], router=f(p + "router.weight"),
                                gate_up=[d(p + f"experts.{e}.gate_up.weight") for e in range(EXPERTS)],
                                down=[d(p + f"experts.{e}.down.weight") for e in range(EXPERTS)])
            else:
                ffn = make_part("feed_forward", "swiglu", hidden=c["H"], intermediate=c["I"], w_gate_up=d(p + "gate_up.weight"),
                                w_down=d(p + "down.weight"))
            blocks.append(make_part(
                "block", "pre_norm",
                mixer_norm=make_part("norm", "rmsnorm", width=c["H"], eps=1e-5, weight=f(p + "norm1.weight")),
                mixer=make_part("mixer", "attention", hidden=c["H"], num_heads=c["nh"], num_kv_heads=c["nkv"], head_dim=c["hd"],
                                wqkv=d(p + "qkv.weight"), wo=d(p + "o.weight"), position=position),
                ffn_norm=make_part("norm", "rmsnorm", width=c["H"], eps=1e-5, weight=f(p + "norm2.weight")), ffn=ffn))
        emb = Embedding(c["V"], c["H"], d("embed.weight"))
        return DecoderModel(embedding=emb, blocks=blocks, schedule=[LayerRun(l, l) for l in range(c["L"])],
                            final_norm=make_part("norm", "rmsnorm", width=c["H"], eps=1e-5, weight=f("norm.weight")),
                            lm_head=LMHead(c["V"], c["H"], emb.table), position=position, dtype=dtype, vocab_size=c["V"],
                            max_positions=c["P"])
    return build


register_architecture(Architecture("ToyLearnedLM", _lp_parse, _lp_manifest(False), _lp_build(False), lambda n: "norm" in n), replace=True)
register_architecture(Architecture("ToyRoutedLM", _lp_parse, _lp_manifest(True), _lp_build(True), lambda n: "norm" in n), replace=True)

LEARNED_CONFIG = dict(hidden_size=40, vocab_size=61, num_hidden_layers=2, intermediate_size=24, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=12, max_position_embeddings=96)


def plain_learned(model_dir, ids, routed):
    """(logits [len(ids), V], the experts picked per layer) of ToyLearnedLM / ToyRoutedLM for one whole sequence."""
    W = {k: v.astype(np.float32) for k, v in P.read_safetensors(f"{model_dir}/model.safetensors").items()}
    c = _lp_parse(json.load(open(f"{model_dir}/config.json")))
    x = P.embed(W["embed.weight"], ids) + W["positions.weight"][:len(ids)]
    picks = []
    for l in range(c["L"]):
        p = f"layers.{l}."
        xn = P.rms_norm(x, W[p + "norm1.weight"], 1e-5)
        qkv = P.linear(xn, W[p + "qkv.weight"])
        qd, kd = c["nh"] * c["hd"], c["nkv"] * c["hd"]
        q = qkv[:, :qd].reshape(-1, c["nh"], c["hd"]); k = qkv[:, qd:qd + kd].reshape(-1, c["nkv"], c["hd"]); v = qkv[:, qd + kd:].reshape(-1, c["nkv"], c["hd"])
        x = x + P.linear(P.causal_attention(q, k, v), W[p + "o.weight"])
        xn = P.rms_norm(x, W[p + "norm2.weight"], 1e-5)
        if not routed:
            gu = W[p + "gate_up.weight"]
            x = x + P.swiglu(xn, gu[:c["I"]], gu[c["I"]:], W[p + "down.weight"])
            continue
        logits = P.linear(xn, W[p + "router.weight"])
        prob = np.exp(logits - logits.max(-1, keepdims=True)); prob /= prob.sum(-1, keepdims=True)
        pick = logits.argmax(-1)
        picks.append(pick)
        y = np.zeros_like(x)
        for t in range(len(ids)):
            e = int(pick[t])
            gu = W[p + f"experts.{e}.gate_up.weight"]
            y[t] = P.swiglu(xn[t:t + 1], gu[:c["I"]], gu[c["I"]:], W[p + f"experts.{e}.down.weight"])[0] * prob[t, e]
        x = x + y
    return P.linear(P.rms_norm(x, W["norm.weight"], 1e-5), W["embed.weight"]), picks


def write_toy(model_dir, config_json, seed, std):
    """A model folder for one of the toy architectures (config.json as given, random weights)."""
    from vitna_anchor_b200.engine.loading import write_random_model
    write_random_model(model_dir, config_json, seed, std=std)
    with open(f"{model_dir}/config.json", "w") as f:
        json.dump(config_json, f)
    return model_dir
