"""The plain implementation against the reference's own CPU program (tests/golden/), and its parts
against direct restatements."""
import json
import os

import numpy as np

import plain_llama as P

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_plain_matches_reference_program(tiny_dirs):
    with open(os.path.join(GOLDEN, "golden.json")) as f:
        meta = json.load(f)
    for name, m in meta.items():
        ref = np.fromfile(os.path.join(GOLDEN, m["file"]), "<f4").reshape(len(m["ids"]), m["vocab"])
        cfg, W = P.read_model(tiny_dirs[name])
        mine = P.forward(cfg, W, m["ids"])
        # two float32 implementations with different summation orders; a wrong formula moves logits by far more
        assert np.abs(mine - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max()), name


def test_prefix_property(tiny_dirs):
    """Causality: the logits of a prefix are the first rows of the logits of the whole."""
    cfg, W = P.read_model(tiny_dirs["tinyB"])
    ids = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5]
    whole = P.forward(cfg, W, ids)
    part = P.forward(cfg, W, ids[:6])
    assert np.abs(whole[:6] - part).max() < 1e-6


def test_rms_norm_formula():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 37)).astype(np.float32)
    w = rng.standard_normal(37).astype(np.float32)
    want = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-5) * w
    assert np.abs(P.rms_norm(x, w, 1e-5) - want).max() < 1e-5


def test_rope_is_a_rotation_of_half_split_pairs():
    cos, sin = P.rope_tables([0, 1, 7], 8, 10000.0)
    v = np.arange(3 * 2 * 8, dtype=np.float32).reshape(3, 2, 8)
    r = P.rope_half(v, cos, sin)
    assert np.allclose(r[0], v[0])                               # position 0: identity
    assert np.allclose((r ** 2).sum(-1), (v ** 2).sum(-1), rtol=1e-5)   # norms are kept
    j = 1
    a, b = v[2, 1, j], v[2, 1, j + 4]
    ang = 7.0 * (1.0 / 10000.0 ** (2 * j / 8))
    assert np.isclose(r[2, 1, j], a * np.cos(ang) - b * np.sin(ang), rtol=1e-5)
    assert np.isclose(r[2, 1, j + 4], b * np.cos(ang) + a * np.sin(ang), rtol=1e-5)


def test_attention_window_and_groups():
    rng = np.random.default_rng(1)
    q = rng.standard_normal((6, 4, 8)).astype(np.float32)
    k = rng.standard_normal((6, 2, 8)).astype(np.float32)
    v = rng.standard_normal((6, 2, 8)).astype(np.float32)
    full = P.causal_attention(q, k, v).reshape(6, 4, 8)
    assert np.allclose(full[0, 3], v[0, 1], atol=1e-6)            # one key: its value; head 3 reads kv head 1
    win = P.causal_attention(q, k, v, window=1).reshape(6, 4, 8)
    assert np.allclose(win[5, 0], v[5, 0], atol=1e-6)             # window 1: only itself


def test_sampler_follows_the_reference_order():
    s = P.PlainSampler(7)
    logits = np.array([0.0, 2.0, 2.0, -1.0], np.float32)
    assert P.PlainSampler.argmax(logits) == 1                     # lowest id among equal maxima
    assert s.sample(logits, 0.0) == 1
    assert s.sample(logits, 0.8, top_k=1) == 1                    # top-k 1 keeps the first of the order
    assert s.sample(logits, 0.8, top_p=1e-6) == 1
    a = [P.PlainSampler(11).sample(logits, 1.0) for _ in range(3)]
    assert a[0] == a[1] == a[2]                                   # a seed gives the same draw
    draws = np.bincount([s.sample(logits, 1.0) for _ in range(4000)], minlength=4) / 4000.0
    p = np.exp(logits - logits.max()); p /= p.sum()
    assert np.abs(draws - p).max() < 0.03
