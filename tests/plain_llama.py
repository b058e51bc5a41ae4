"""A plain, slow statement of the dense Llama decoder, in NumPy float32.

Whole sequences, no cache, one function for each part.  It shares no code with
the engine: it has its own reader for config.json and model.safetensors, and
every function is written from the formulas of the reference's CPU forward
pass (cited as file:line within the reference project).  tests/golden/ holds
logits of the reference's own CPU program on two tiny random models, and
test_plain.py checks this file against them, so the formulas here do not rest
on reading alone.

Everything is float32: a stored bfloat16 value is widened exactly
(engine/src/ops.c:25-30), and sums are float32 sums.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np

F32 = np.float32


def bf16_round(x):
    """x rounded to the nearest bfloat16 (ties to even) and widened back to float32: the value a tensor has after
    it has been stored in 16 bits (the upper half of a float32, engine/src/ops.c:25-30 read the other way)."""
    u = np.ascontiguousarray(x, dtype=F32).view(np.uint32)
    r = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return r.view(F32).reshape(np.shape(x))


# ----------------------------------------------------------------------------
# Reading a model folder
# ----------------------------------------------------------------------------

def read_safetensors(path):
    """name -> float32 array.  8-byte little-endian header length, a JSON
    directory, then the bytes (engine/src/safetensors.c:105-191)."""
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    directory = json.loads(raw[8:8 + n].decode("utf-8"))
    base = 8 + n
    out = {}
    for name, d in directory.items():
        if name == "__metadata__":
            continue
        lo, hi = d["data_offsets"]
        blob = raw[base + lo:base + hi]
        if d["dtype"] == "F32":
            a = np.frombuffer(blob, "<f4")
        elif d["dtype"] == "BF16":
            # ops.c:25-30: the 16 stored bits are the high half of a float32.
            a = (np.frombuffer(blob, "<u2").astype(np.uint32) << 16).view("<f4")
        elif d["dtype"] == "F16":
            a = np.frombuffer(blob, "<f2").astype(F32)
        else:
            raise ValueError(f"{name}: dtype {d['dtype']}")
        out[name] = a.reshape(d["shape"]).astype(F32)
    return out


def read_model(model_dir):
    """(config dict with defaults filled in as engine/src/model.c:92-124, weights)."""
    with open(os.path.join(model_dir, "config.json")) as f:
        c = json.load(f)
    cfg = dict(
        L=c["num_hidden_layers"], H=c["hidden_size"], I=c["intermediate_size"],
        nh=c["num_attention_heads"], V=c["vocab_size"],
        nkv=c.get("num_key_value_heads") or c["num_attention_heads"],
        hd=c.get("head_dim") or c["hidden_size"] // c["num_attention_heads"],
        eps=c["rms_norm_eps"] if c.get("rms_norm_eps") is not None else 1e-6,
        theta=c["rope_theta"] if c.get("rope_theta") is not None else 10000.0,
        tied=bool(c.get("tie_word_embeddings", False)),
    )
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ----------------------------------------------------------------------------
# One function for each part
# ----------------------------------------------------------------------------

def embed(table, ids):
    """x = the token's row, no scaling (engine/src/model.c:893-895)."""
    return table[np.asarray(ids, dtype=np.int64)].astype(F32)


def rms_norm(x, w, eps):
    """y_i = (x_i * (1 / sqrt(sum(x^2)/n + eps))) * w_i, the weight used as it
    is (engine/src/kernels.c:94-111)."""
    x = x.astype(F32)
    ss = np.sum(x * x, axis=-1, keepdims=True, dtype=F32)
    inv = F32(1.0) / np.sqrt(ss / F32(x.shape[-1]) + F32(eps), dtype=F32)
    return ((x * inv) * w.astype(F32)).astype(F32)


def rope_tables(positions, hd, theta):
    """inv_freq[j] = 1 / theta^(2j/hd); angle = (float)pos * inv_freq[j]
    (engine/src/model.c:408-413, 899-904).  Returns cos, sin [T, hd/2]."""
    j2 = np.arange(0, hd, 2, dtype=F32)
    inv_freq = (F32(1.0) / np.power(F32(theta), j2 / F32(hd), dtype=F32)).astype(F32)
    ang = (np.asarray(positions, dtype=F32)[:, None] * inv_freq[None, :]).astype(F32)
    return np.cos(ang).astype(F32), np.sin(ang).astype(F32)


def rope_half(v, cos, sin):
    """Half-split rotation of v [T, heads, hd]: the pair is (j, j + hd/2)
    (engine/src/ops.c:273-281)."""
    half = v.shape[-1] // 2
    a, b = v[..., :half], v[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return np.concatenate([a * c - b * s, b * c + a * s], axis=-1).astype(F32)


def causal_attention(q, k, v, window=None, scale=None):
    """q [T, nh, hd], k and v [T, nkv, hd] -> [T, nh*hd].

    Query head h reads key-value head h // (nh/nkv); the score is the dot
    product times 1/sqrt(hd), scaled after the sum; position t sees keys
    0..t; softmax with the maximum taken out; the output is the sum of
    p_t * v_t (engine/src/model.c:890-891, 932-956).  `window` (not part of
    the reference's Llama) limits a query at t to keys t-window+1..t."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    sc = F32(1.0) / np.sqrt(F32(hd)) if scale is None else F32(scale)
    out = np.zeros((T, nh, hd), F32)
    for h in range(nh):
        kh, vh = k[:, h // g], v[:, h // g]
        for t in range(T):
            lo = 0 if window is None else max(0, t - window + 1)
            s = (kh[lo:t + 1] @ q[t, h]).astype(F32) * sc
            e = np.exp(s - s.max(), dtype=F32)
            p = e * (F32(1.0) / e.sum(dtype=F32))
            out[t, h] = p @ vh[lo:t + 1]
    return out.reshape(T, nh * hd)


def linear(x, w):
    """y = W x for each row of x; W is [rows, cols] (engine/src/ops.c:101-119)."""
    return (x.astype(F32) @ w.astype(F32).T).astype(F32)


def swiglu(xn, w_gate, w_up, w_down, rnd=None):
    """act_i = (g_i / (1 + exp(-g_i))) * u_i; y = W_down act
    (engine/src/model.c:966-971, engine/src/ops.c:283-288).  rnd: applied to what a 16-bit engine stores (the gate
    and up products, then the activation)."""
    rnd = rnd or (lambda a: a)
    g = rnd(linear(xn, w_gate))
    u = rnd(linear(xn, w_up))
    act = rnd((g / (F32(1.0) + np.exp(-g, dtype=F32))) * u)
    return linear(act.astype(F32), w_down)


def attention_block(x, W, prefix, cfg, positions, window=None, kv=None, return_kv=False, rnd=None):
    """RMSNorm, q/k/v, rotation of q and k, attention, output projection,
    residual sum (engine/src/model.c:912-959).  kv: rotated keys and values of
    another run to attend over instead of this one's own.  rnd: applied to every tensor that a 16-bit engine
    stores between two kernels (normed activations; q, k, v before and after the rotation, so the cache too; the
    attention's output); the residual stream and all sums stay float32."""
    rnd = rnd or (lambda a: a)
    T = x.shape[0]
    xn = rnd(rms_norm(x, W[prefix + "input_layernorm.weight"], cfg["eps"]))
    q = rnd(linear(xn, W[prefix + "self_attn.q_proj.weight"])).reshape(T, cfg["nh"], cfg["hd"])
    k = rnd(linear(xn, W[prefix + "self_attn.k_proj.weight"])).reshape(T, cfg["nkv"], cfg["hd"])
    v = rnd(linear(xn, W[prefix + "self_attn.v_proj.weight"])).reshape(T, cfg["nkv"], cfg["hd"])
    cos, sin = rope_tables(positions, cfg["hd"], cfg["theta"])
    q, k = rnd(rope_half(q, cos, sin)), rnd(rope_half(k, cos, sin))
    if kv is not None:
        k, v = kv
    att = rnd(causal_attention(q, k, v, window))
    y = (x + linear(att, W[prefix + "self_attn.o_proj.weight"])).astype(F32)
    return (y, (k, v)) if return_kv else y


def mlp_block(x, W, prefix, cfg, rnd=None):
    """RMSNorm, SwiGLU, residual sum (engine/src/model.c:962-972)."""
    rnd = rnd or (lambda a: a)
    xn = rnd(rms_norm(x, W[prefix + "post_attention_layernorm.weight"], cfg["eps"]))
    return (x + swiglu(xn, W[prefix + "mlp.gate_proj.weight"], W[prefix + "mlp.up_proj.weight"],
                       W[prefix + "mlp.down_proj.weight"], rnd)).astype(F32)


def lm_head(x, W, cfg, rnd=None):
    """Final RMSNorm and the output matrix; the embedding stands in for a
    missing lm_head.weight when the two are tied (engine/src/model.c:315-321,
    975-978)."""
    rnd = rnd or (lambda a: a)
    xn = rnd(rms_norm(x, W["model.norm.weight"], cfg["eps"]))
    head = W["lm_head.weight"] if "lm_head.weight" in W else W["model.embed_tokens.weight"]
    return linear(xn, head)


def forward(cfg, W, ids, layer_order=None, reads=None, bf16=False):
    """Logits [len(ids), V] of one whole sequence starting at position 0.
    `layer_order` names the layers to run, in order (default: 0..L-1,
    engine/src/model.c:906-972).  reads[i] = j: run i attends over the keys and
    values that run j (an earlier one) made, and makes none of its own.
    bf16: the same computation with the matrices and every tensor between two kernels rounded to bfloat16 where a
    16-bit engine stores them (norm weights, the residual stream, softmax and every sum stay float32): what the
    bfloat16 path is held to, more tightly than to the unrounded computation."""
    rnd = bf16_round if bf16 else None
    if bf16:
        W = {k: (v if v.ndim < 2 else bf16_round(v)) for k, v in W.items()}
    positions = np.arange(len(ids))
    x = embed(W["model.embed_tokens.weight"], ids)
    order = list(range(cfg["L"]) if layer_order is None else layer_order)
    made = {}
    for i, l in enumerate(order):
        p = f"model.layers.{l}."
        src = None if reads is None else reads.get(i)
        x, made[i] = attention_block(x, W, p, cfg, positions, kv=None if src is None else made[src], return_kv=True, rnd=rnd)
        x = mlp_block(x, W, p, cfg, rnd)
    return lm_head(x, W, cfg, rnd)


# ----------------------------------------------------------------------------
# Sampling (engine/src/sampler.c)
# ----------------------------------------------------------------------------

class PlainSampler:
    """splitmix64 and the reference's order of operations: temperature,
    softmax, sort by probability (lower id first among equals), top-k,
    top-p, one draw (engine/src/sampler.c:31-49, 96-139)."""

    MASK = (1 << 64) - 1

    def __init__(self, seed):
        self.state = seed & self.MASK

    def uniform(self):
        self.state = (self.state + 0x9E3779B97F4A7C15) & self.MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & self.MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & self.MASK
        z = z ^ (z >> 31)
        return (z >> 11) * (1.0 / 9007199254740992.0)

    @staticmethod
    def argmax(logits):
        return int(np.argmax(logits))  # the first of equal maxima, as sampler.c:31-38

    def distribution(self, logits, temperature, top_k=0, top_p=1.0):
        """(ids in sorted order, their probabilities as float64, kept count, kept mass)."""
        l = np.asarray(logits, F32)
        probs = np.exp((l - l.max()) / F32(temperature), dtype=F32)
        total = float(np.sum(probs.astype(np.float64)))
        probs = (probs.astype(np.float64) / total).astype(F32)
        order = np.lexsort((np.arange(len(l)), -probs.astype(np.float64)))
        p = probs[order].astype(np.float64)
        keep = top_k if 0 < top_k < len(l) else len(l)
        mass = float(p[:keep].sum())
        if 0.0 < top_p < 1.0:
            cum = np.cumsum(p[:keep] / mass)
            hit = np.nonzero(cum >= top_p)[0]
            keep = int(hit[0]) + 1 if len(hit) else keep
            mass = float(p[:keep].sum())
        return order, p, keep, mass

    def sample(self, logits, temperature, top_k=0, top_p=1.0):
        if temperature <= 0.0:
            return self.argmax(logits)
        order, p, keep, mass = self.distribution(logits, temperature, top_k, top_p)
        u = self.uniform() * mass
        cum = np.cumsum(p[:keep])
        hit = np.nonzero(u < cum)[0]
        return int(order[hit[0]] if len(hit) else order[keep - 1])
