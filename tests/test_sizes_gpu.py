"""The engine at the layer sizes of SmolLM2-135M, 360M and 1.7B (two layers each, random weights), and a tiny
model with a long context: prompts long enough for the tensor-core kernels' tiles, portions, and decoded
tokens whose keys span several splits; float32 and bfloat16 against the plain implementation."""
import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu

BASE = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", rms_norm_eps=1e-5,
            tie_word_embeddings=True, max_position_embeddings=8192, num_hidden_layers=2)
SIZES = {
    # the 135M model keeps its vocabulary; the larger two use a smaller one so that the test stays quick
    "135M": dict(BASE, hidden_size=576, intermediate_size=1536, num_attention_heads=9, num_key_value_heads=3, head_dim=64,
                 vocab_size=49152, rope_theta=100000.0),
    "360M": dict(BASE, hidden_size=960, intermediate_size=2560, num_attention_heads=15, num_key_value_heads=5, head_dim=64,
                 vocab_size=8192, rope_theta=100000.0),
    "1.7B": dict(BASE, hidden_size=2048, intermediate_size=8192, num_attention_heads=32, num_key_value_heads=32, head_dim=64,
                 vocab_size=8192, rope_theta=130000.0),
}


@pytest.fixture(scope="module")
def size_dirs(tmp_path_factory):
    from vitna_anchor_b200.engine.loading import write_random_model
    root = tmp_path_factory.mktemp("sizes")
    out = {}
    for name, cfg in SIZES.items():
        out[name] = str(root / name)
        write_random_model(out[name], cfg, seed=7, std=0.05)      # sharper than 0.02, so that a wrong key shows
    return out


def _run(model_dir, dtype, ids, cuts, decode):
    """Logits of every position: the prompt in portions `cuts`, then `decode` tokens one by one."""
    from vitna_anchor_b200.engine.loading import load_model
    from vitna_anchor_b200.engine.runner import ModelRunner, StepEntry
    from vitna_anchor_b200 import ops
    runner = ModelRunner(load_model(model_dir, dtype), page_size=16, num_pages=64, max_requests=2, max_batch_tokens=512,
                         max_model_len=1024)
    runner.open("r")
    rows, p = [], 0
    for n in cuts:
        rows.append(runner.step([StepEntry("r", ids[p:p + n], range(n))]).float().cpu().numpy())
        p += n
    for _ in range(decode):
        rows.append(runner.step([StepEntry("r", ids[p:p + 1], [0])]).float().cpu().numpy())
        p += 1
    torch.cuda.synchronize()
    ops.check_device_errors()
    runner.check(sync=False)
    runner.close("r")
    return np.concatenate(rows)


@pytest.mark.parametrize("name", ["135M", "360M", "1.7B"])
def test_real_layer_sizes(name, size_dirs):
    cfg, W = P.read_model(size_dirs[name])
    rng = np.random.default_rng(3)
    ids = [int(t) for t in rng.integers(0, cfg["V"], 216)]
    plain = P.forward(cfg, W, ids)
    scale = max(1.0, float(np.abs(plain).max()))
    f32 = _run(size_dirs[name], "float32", ids, [200], 16)
    assert np.abs(f32 - plain).max() <= 2e-5 * scale
    f32_cut = _run(size_dirs[name], "float32", ids, [70, 2, 128], 16)
    assert np.array_equal(f32_cut, f32)                 # the 32-bit path: the same bytes however the prompt is cut
    bf = _run(size_dirs[name], "bfloat16", ids, [200], 16)
    assert np.abs(bf - plain).max() <= 8e-2 * scale
    rounded = P.forward(cfg, W, ids, bf16=True)          # the plain implementation rounding where a 16-bit engine stores
    print(f"\n{name}: bfloat16 against plain {np.abs(bf - plain).max() / scale:.3e}, against plain with 16-bit rounding "
          f"{np.abs(bf - rounded).max() / scale:.3e} of scale")
    assert np.abs(bf - rounded).max() <= 1.5e-2 * scale
    bf_cut = _run(size_dirs[name], "bfloat16", ids, [70, 2, 128], 16)
    assert np.abs(bf_cut - bf).max() <= 1e-2 * scale
    bf_dec = _run(size_dirs[name], "bfloat16", ids, [150], 66)         # the last 66 tokens decoded one by one
    assert np.abs(bf_dec - bf).max() <= 1e-2 * scale


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 8e-2)])
def test_long_context_spans_several_key_splits(dtype, tol, tmp_path):
    """900 positions: prompt portions whose tiles cross several key tiles, then decoded tokens at 760..899 whose
    keys lie in four splits of 256.  One far key is what matters for many queries (sharp weights)."""
    from tiny_configs import TINY_B
    from vitna_anchor_b200.engine.loading import write_random_model
    cfg_json = dict(TINY_B["config"], max_position_embeddings=2048)
    write_random_model(str(tmp_path / "long"), cfg_json, 5, std=0.15, norm_noise=0.1)
    cfg, W = P.read_model(str(tmp_path / "long"))
    rng = np.random.default_rng(9)
    ids = [int(t) for t in rng.integers(0, cfg["V"], 900)]
    plain = P.forward(cfg, W, ids)
    got = _run(str(tmp_path / "long"), dtype, ids, [300, 129, 331], 140)
    assert np.abs(got - plain).max() <= tol * max(1.0, float(np.abs(plain).max()))


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 8e-2)])
@pytest.mark.parametrize("name", ["135M", "1.7B"])
def test_large_portions_beside_decoded_tokens_at_real_sizes(name, dtype, tol, size_dirs):
    """Steps of more than 64 tokens that hold prompt portions AND single decoded tokens, at head size 64: in bfloat16
    one step runs the tcgen05 products with the rotation and cache write in their epilogue over a mixed batch's slot
    mapping, the tcgen05 prompt attention and the split-key decode attention.  The same counts come four times with
    different segment lengths ([100, 28] and [90, 38] beside two decoded tokens), other tokens, positions and pages:
    the first is run eagerly, the second captured, the third and fourth are replays of that graph.  Every wanted row
    against the plain implementation."""
    from vitna_anchor_b200.engine.loading import load_model
    from vitna_anchor_b200.engine.runner import ModelRunner, StepEntry
    cfg, W = P.read_model(size_dirs[name])
    rng = np.random.default_rng(12)
    seqs = {k: [int(t) for t in rng.integers(0, cfg["V"], n)] for k, n in (("A", 400), ("D", 140), ("B", 160), ("C", 130))}
    plain = {k: P.forward(cfg, W, v) for k, v in seqs.items()}
    scale = max(1.0, max(float(np.abs(p).max()) for p in plain.values()))
    runner = ModelRunner(load_model(size_dirs[name], dtype), page_size=16, num_pages=80, max_requests=4, max_batch_tokens=256,
                         max_model_len=1024)
    at = {k: 0 for k in seqs}
    worst = 0.0

    def step(parts):
        """parts: [(request, n tokens, wanted places)]"""
        nonlocal worst
        entries = [StepEntry(k, seqs[k][at[k]:at[k] + n], want) for k, n, want in parts]
        got = runner.step(entries).float().cpu().numpy()
        r = 0
        for k, n, want in parts:
            for w in want:
                worst = max(worst, float(np.abs(got[r] - plain[k][at[k] + w]).max()))
                r += 1
            at[k] += n
    for k in seqs:
        runner.open(k)
    step([("B", 150, [0, 149])])
    step([("C", 120, [119])])
    replays = runner.graph_replays
    for a, d in ((100, 28), (90, 38), (100, 28), (90, 38)):
        step([("A", a, [0, 63, 64, a - 1]), ("B", 1, [0]), ("D", d, [1, d - 1]), ("C", 1, [0])])
    runner.check(sync=True)
    if runner.cuda_graphs:
        assert runner.graph_replays - replays >= 2, "the third and fourth step of the same counts were meant to be replays"
    assert worst <= tol * scale, f"largest difference {worst / scale:.3e} of scale"
