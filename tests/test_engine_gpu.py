"""The engine through its entry points: greedy and sampled generation against the plain implementation,
long decoding, the first tokens of a sequence, several requests with too few pages (preemption),
a failed step, and the command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as P
from tiny_configs import TINIES, write_tiny

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def sharp_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("sharp_engine")
    return {name: write_tiny(str(root / name), tiny, std=0.15) for name, tiny in TINIES.items()}


def plain_generate(cfg, W, prompt, max_new, temperature=0.0, top_k=0, top_p=1.0, seed=0):
    """Greedy or sampled continuation by running the whole sequence again for every new token."""
    ids, out, rows = list(prompt), [], []
    sampler = P.PlainSampler(seed)
    for _ in range(max_new):
        row = P.forward(cfg, W, ids)[-1]
        tok = sampler.sample(row, temperature, top_k, top_p)
        rows.append(row); out.append(tok); ids.append(tok)
    return out, np.stack(rows)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tinyA", "tinyB"])
def test_greedy_generation_matches_plain(name, dtype, sharp_dirs, tmp_path):
    from vitna_anchor_b200.engine.engine import Engine
    cfg, W = P.read_model(sharp_dirs[name])
    rng = np.random.default_rng(11)
    prompt = [int(t) for t in rng.integers(0, cfg["V"], 9)]
    eng = Engine(sharp_dirs[name], dtype=dtype, kv_block=TINIES[name]["page_size"], parallel=2)
    out_file = str(tmp_path / "rows.f32")
    got = eng.generate(prompt, max_new=40, logits_out=out_file)
    want, rows = plain_generate(cfg, W, prompt, 40)
    mine = np.fromfile(out_file, "<f4").reshape(40, cfg["V"])
    if dtype == "float32":
        assert got == want
        assert np.abs(mine - rows).max() <= 2e-5 * max(1.0, np.abs(rows).max())
    else:
        # the same tokens as long as the plain margin between the best two is not within bfloat16's error
        for i, (g, w) in enumerate(zip(got, want)):
            if g != w:
                top2 = np.sort(rows[i])[-2:]
                assert top2[1] - top2[0] < 0.16 * max(1.0, np.abs(rows[i]).max()), f"token {i}: {g} != {w}"
                break
            assert np.abs(mine[i] - rows[i]).max() <= 8e-2 * max(1.0, np.abs(rows).max())
    assert eng.runner.graph_replays > 20            # decoding went through captured graphs
    assert eng.runner.cache.free_pages() == [eng.runner.cache.tables.pools[0].num_pages]


def test_sampled_generation_matches_plain_sampler(sharp_dirs):
    from vitna_anchor_b200.engine.engine import Engine
    cfg, W = P.read_model(sharp_dirs["tinyB"])
    prompt = [5, 9, 200, 31, 7]
    eng = Engine(sharp_dirs["tinyB"], dtype="float32", kv_block=8, parallel=2)
    for kw in (dict(temperature=0.8, seed=7), dict(temperature=1.1, top_k=20, seed=3), dict(temperature=0.8, top_p=0.9, seed=5)):
        got = eng.generate(prompt, max_new=16, **kw)
        want, _ = plain_generate(cfg, W, prompt, 16, **kw)
        assert got == want, kw
    again = eng.generate(prompt, max_new=16, temperature=0.8, seed=7)
    assert again == eng.generate(prompt, max_new=16, temperature=0.8, seed=7)       # a seed gives the same tokens


def test_long_decoding_and_first_tokens(sharp_dirs):
    """A prompt of one token, then 150 decoded tokens across many pages: every logits row against plain."""
    from vitna_anchor_b200.engine.runner import ModelRunner, StepEntry
    from vitna_anchor_b200.engine.loading import load_model
    cfg, W = P.read_model(sharp_dirs["tinyB"])
    rng = np.random.default_rng(2)
    ids = [int(t) for t in rng.integers(0, cfg["V"], 151)]
    plain = P.forward(cfg, W, ids)
    for dtype, tol in (("float32", 2e-5), ("bfloat16", 8e-2)):
        runner = ModelRunner(load_model(sharp_dirs["tinyB"], dtype), page_size=8, num_pages=24, max_requests=2, max_batch_tokens=64)
        runner.open("r")
        worst = 0.0
        for p, t in enumerate(ids):
            row = runner.step([StepEntry("r", [t], [0])])[0].cpu().numpy()
            worst = max(worst, np.abs(row - plain[p]).max())
        assert worst <= tol * max(1.0, np.abs(plain).max()), (dtype, worst)
        assert runner.graph_replays >= 149
        runner.close("r")
        runner.cache.check()


def test_requests_together_with_few_pages_equal_requests_alone(sharp_dirs):
    """Six requests, four at a time, in a pool so small that the newest is preempted and recomputed:
    every request's tokens are those it gets alone (float32: greedy and seeded sampling)."""
    from vitna_anchor_b200.engine.engine import Engine
    rng = np.random.default_rng(4)
    cfgA = TINIES["tinyA"]["config"]
    prompts = [[int(t) for t in rng.integers(0, cfgA["vocab_size"], n)] for n in (5, 17, 33, 12, 26, 8)]
    alone = Engine(sharp_dirs["tinyA"], dtype="float32", kv_block=4, parallel=1)
    want_greedy = [alone.generate(p, max_new=20) for p in prompts]
    want_sampled = [alone.generate(p, max_new=20, temperature=0.8, seed=100 + i) for i, p in enumerate(prompts)]
    small = Engine(sharp_dirs["tinyA"], dtype="float32", kv_block=4, parallel=4, num_pages=34, max_batch_tokens=24)
    assert small.generate(prompts, max_new=20) == want_greedy
    assert small.scheduler.preempted_total > 0, "the pool was meant to be too small"
    assert small.generate(prompts, max_new=20, temperature=0.8, seed=100) == want_sampled
    small.runner.cache.check()
    assert small.runner.cache.free_pages() == [34]


def test_failed_step_ends_the_request_and_changes_nothing(sharp_dirs):
    from vitna_anchor_b200.engine.engine import Engine
    from vitna_anchor_b200.engine.runner import StepFailed
    eng = Engine(sharp_dirs["tinyA"], dtype="float32", kv_block=4, parallel=2)
    want = eng.generate([1, 2, 3, 4], max_new=8)
    eng.runner.fail_step_once(6)                   # the step that computes position 6: the third decoded token
    with pytest.raises(StepFailed):
        eng.generate([1, 2, 3, 4], max_new=8)
    assert eng.scheduler.finished[-1].output == want[:3]
    assert eng.runner.cache.free_pages() == [eng.runner.cache.tables.pools[0].num_pages]
    assert eng.generate([1, 2, 3, 4], max_new=8) == want          # the engine goes on


def test_refusals(sharp_dirs):
    from vitna_anchor_b200.engine.engine import Engine, RequestRefused
    eng = Engine(sharp_dirs["tinyA"], dtype="float32", kv_block=4, parallel=1, ctx=64)
    with pytest.raises(RequestRefused):
        eng.generate([1] * 60, max_new=8)
    with pytest.raises(RequestRefused):
        eng.generate([1, 999], max_new=2)
    with pytest.raises(ValueError):
        Engine(sharp_dirs["tinyA"], device="cpu")


def test_command_line(sharp_dirs, tmp_path):
    exe = [sys.executable, os.path.join(ROOT, "bin", "vitna-anchor")]
    model = sharp_dirs["tinyB"]
    cfg, W = P.read_model(model)
    ids = [3, 1, 4, 1, 5, 9, 2, 6]
    r = subprocess.run(exe + ["generate", "--model", model, "--ids", ",".join(map(str, ids)), "--max-new", "6", "--greedy",
                              "--dtype", "float32", "--timing"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["prompt_ids"] == ids and out["ids"] == plain_generate(cfg, W, ids, 6)[0]
    assert "timing: 8 prompt tokens in" in r.stderr
    f = tmp_path / "l.f32"
    r = subprocess.run(exe + ["logits", "--model", model, "--ids", ",".join(map(str, ids)), "--out", str(f), "--dtype", "float32"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    rows = np.fromfile(str(f), "<f4").reshape(len(ids), cfg["V"])
    assert np.abs(rows - P.forward(cfg, W, ids)).max() <= 2e-5 * 5
    r = subprocess.run(exe + ["generate", "--model", model, "--ids", "1,2", "--device", "cpu"], capture_output=True, text=True)
    assert r.returncode == 1 and "cuda" in r.stderr
    r = subprocess.run(exe + ["generate", "--model", model, "--ids", "1,2", "--speculate", "4"], capture_output=True, text=True)
    assert r.returncode == 1 and "Unknown or incomplete option: --speculate" in r.stderr


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 8e-2)])
def test_steps_with_the_same_counts_replay_a_captured_graph(dtype, tol, sharp_dirs):
    """Three requests run the same schedule of steps (a prompt portion of 70 beside... the same counts each time):
    the first time eagerly, the second time while being captured, from then on as replays of that graph, with other
    tokens, positions and pages each time.  Every logits row against the plain implementation."""
    from vitna_anchor_b200.engine.loading import load_model
    from vitna_anchor_b200.engine.runner import ModelRunner, StepEntry
    cfg, W = P.read_model(sharp_dirs["tinyB"])
    rng = np.random.default_rng(21)
    runner = ModelRunner(load_model(sharp_dirs["tinyB"], dtype), page_size=8, num_pages=64, max_requests=4, max_batch_tokens=128)
    worst, replays_before = 0.0, runner.graph_replays
    for round_ in range(4):
        a = [int(t) for t in rng.integers(0, cfg["V"], 90)]
        b = [int(t) for t in rng.integers(0, cfg["V"], 40)]
        pa, pb = P.forward(cfg, W, a), P.forward(cfg, W, b)
        ra, rb = f"a{round_}", f"b{round_}"
        runner.open(ra); runner.open(rb)
        got = runner.step([StepEntry(ra, a[:70], [69])]).cpu().numpy()                                  # a prompt portion alone
        worst = max(worst, np.abs(got[0] - pa[69]).max())
        got = runner.step([StepEntry(ra, a[70:71], [0]), StepEntry(rb, b[:33], [0, 32])]).cpu().numpy()    # a decoded token beside a portion
        worst = max(worst, np.abs(got[0] - pa[70]).max(), np.abs(got[1] - pb[0]).max(), np.abs(got[2] - pb[32]).max())
        got = runner.step([StepEntry(rb, b[33:40], [6]), StepEntry(ra, a[71:90], [18])]).cpu().numpy()     # two portions
        worst = max(worst, np.abs(got[0] - pb[39]).max(), np.abs(got[1] - pa[89]).max())
        if round_ % 2:            # leave pages held in odd rounds so that later rounds land on other pages
            runner.close(ra)
        else:
            runner.close(ra); runner.close(rb)
    assert runner.graph_replays - replays_before >= 6, "the repeated steps were meant to be replayed"
    assert worst <= tol * max(1.0, float(np.abs(pa).max()))
    runner.cache.check()


def test_decoding_a_step_ahead_of_the_host_gives_the_same_tokens(sharp_dirs):
    """With the overlap (ids stay on the device and feed the next step; the host reads them a step later) and
    without it: the same tokens, greedy and sampled, for requests that end at different steps, are admitted while
    others decode, and are preempted for want of pages; no placeholder is left in any output."""
    from vitna_anchor_b200.engine.engine import Engine
    rng = np.random.default_rng(17)
    V = TINIES["tinyA"]["config"]["vocab_size"]
    prompts = [[int(t) for t in rng.integers(0, V, n)] for n in (3, 11, 20, 6, 9)]
    new = [5, 23, 9, 31, 2]
    outs = {}
    for pipeline in (False, True):
        eng = Engine(sharp_dirs["tinyA"], dtype="float32", kv_block=4, parallel=3, num_pages=26, max_batch_tokens=16, pipeline=pipeline)
        for kw in (dict(), dict(temperature=0.9, top_p=0.9)):
            reqs = [eng.add_request(p, max_new=n, seed=40 + i, **kw) for i, (p, n) in enumerate(zip(prompts, new))]
            finished = eng.run()
            assert sorted(id(r) for r in finished) == sorted(id(r) for r in reqs)
            for r, n in zip(reqs, new):
                assert len(r.output) == n and all(0 <= t < V for t in r.output)
            outs[(pipeline, bool(kw))] = [list(r.output) for r in reqs]
        assert eng.runner.cache.free_pages() == [26]
        if pipeline:
            assert eng.runner.graph_replays > 10
    assert outs[(True, False)] == outs[(False, False)]
    assert outs[(True, True)] == outs[(False, True)]


def test_logits_handed_out_by_the_entry_point_do_not_change_with_later_steps(sharp_dirs):
    """The step function's result is valid until the next step (replayed graphs share one logits buffer); what
    the entry point hands out is a copy: rows kept across many later steps of the same shape stay as they were."""
    from vitna_anchor_b200.engine.engine import Engine
    from vitna_anchor_b200.engine.runner import StepEntry
    cfg, W = P.read_model(sharp_dirs["tinyA"])
    eng = Engine(sharp_dirs["tinyA"], dtype="float32", kv_block=4, parallel=2)
    ids = [int(t) for t in np.random.default_rng(1).integers(0, cfg["V"], 40)]
    rows = eng.logits(ids, piece=1)                     # 40 single-token steps: from the second on they are replays
    kept = rows.clone()
    eng.logits(ids[::-1], piece=1)                      # later steps of the same shape
    assert torch.equal(rows, kept)
    assert np.abs(rows.cpu().numpy() - P.forward(cfg, W, ids)).max() <= 2e-5 * 5
    # the raw step function does reuse the buffer, as its docstring says
    runner = eng.runner
    runner.open("x")
    first = runner.step([StepEntry("x", ids[:1], [0])])
    second = runner.step([StepEntry("x", ids[1:2], [0])])
    third = runner.step([StepEntry("x", ids[2:3], [0])])
    assert second.data_ptr() == third.data_ptr()
    runner.close("x")


@pytest.mark.parametrize("family,cuts", [("linear_tcgen05", [100]), ("attention_prefill_tcgen05", [200])])
def test_a_kernel_that_gives_up_a_wait_fails_the_step_and_the_engine_goes_on(family, cuts, tmp_path):
    """A wait inside a tcgen05 kernel runs out (the test's hook makes the producer leave one stage unarmed; the limit
    of a wait is set to 5 ms): the kernel returns by itself, the step function reports it, the request is back
    where it was, and the same step again gives the right logits."""
    from vitna_anchor_b200 import ops
    from vitna_anchor_b200.engine.loading import load_model, write_random_model
    from vitna_anchor_b200.engine.runner import DeviceStepFailed, ModelRunner, StepEntry
    cfg_json = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", rms_norm_eps=1e-5,
                    tie_word_embeddings=True, max_position_embeddings=1024, num_hidden_layers=2, hidden_size=128,
                    intermediate_size=256, num_attention_heads=2, num_key_value_heads=1, head_dim=64, vocab_size=320,
                    rope_theta=10000.0)
    write_random_model(str(tmp_path / "m"), cfg_json, seed=3, std=0.1)
    cfg, W = P.read_model(str(tmp_path / "m"))
    ids = [int(t) for t in np.random.default_rng(5).integers(0, cfg["V"], 260)]
    plain = P.forward(cfg, W, ids)
    runner = ModelRunner(load_model(str(tmp_path / "m"), "bfloat16"), page_size=16, num_pages=64, max_requests=2, max_batch_tokens=256)
    runner.open("r")
    n = cuts[0]
    good = runner.step([StepEntry("r", ids[:40], [39])]).float().cpu().numpy()
    runner.check(sync=True)
    free_before = runner.cache.free_pages()
    ops.set_wait_limit_ms(5.0)
    try:
        ops.skip_stage_once(family, 0)
        bad = runner.step([StepEntry("r", ids[40:40 + n], [n - 1])])
        with pytest.raises(DeviceStepFailed) as e:
            runner.check(sync=True)
        assert e.value.request_ids == ["r"]
    finally:
        ops.set_wait_limit_ms(0)
    assert runner.length("r") == 40 and runner.cache.free_pages() == free_before
    assert ops.device_error_code() == 0
    again = runner.step([StepEntry("r", ids[40:40 + n], [n - 1])]).float().cpu().numpy()
    runner.check(sync=True)
    scale = max(1.0, float(np.abs(plain).max()))
    assert np.abs(good[0] - plain[39]).max() <= 8e-2 * scale
    assert np.abs(again[0] - plain[40 + n - 1]).max() <= 8e-2 * scale
    runner.cache.check()


def test_a_kernel_that_gives_up_ends_the_requests_of_that_step_only(tmp_path):
    """Through the entry point: two requests are in the step that meets the failed wait (one decoding, one with its
    prompt): both end with an error and keep what they had.  A third that was still waiting is admitted afterwards
    and gets the tokens it gets alone."""
    from vitna_anchor_b200 import ops
    from vitna_anchor_b200.engine.engine import Engine
    from vitna_anchor_b200.engine.loading import write_random_model
    cfg_json = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", rms_norm_eps=1e-5,
                    tie_word_embeddings=True, max_position_embeddings=1024, num_hidden_layers=2, hidden_size=128,
                    intermediate_size=256, num_attention_heads=2, num_key_value_heads=1, head_dim=64, vocab_size=320,
                    rope_theta=10000.0)
    write_random_model(str(tmp_path / "m"), cfg_json, seed=3, std=0.1)
    rng = np.random.default_rng(9)
    short, long_ = [int(t) for t in rng.integers(0, 320, 12)], [int(t) for t in rng.integers(0, 320, 150)]
    eng = Engine(str(tmp_path / "m"), dtype="bfloat16", parallel=2, max_batch_tokens=256)
    want = eng.generate(short, max_new=20)
    a = eng.add_request(short, max_new=20)
    for _ in range(4):
        eng.step()                                  # a is decoding
    eng.flush()
    b = eng.add_request(long_, max_new=5)
    c = eng.add_request(short, max_new=20)          # waits: both slots are taken
    ops.set_wait_limit_ms(5.0)
    try:
        ops.skip_stage_once("linear_tcgen05", 0)    # the next prompt-sized product: b's portion beside a's token
        done = eng.step()
        done += eng.flush()
    finally:
        ops.set_wait_limit_ms(0)
    assert b.finish_reason == "error" and a.finish_reason == "error" and set(map(id, done)) == {id(a), id(b)}
    assert a.output == want[:len(a.output)] and len(a.output) >= 4 and b.output == []
    finished = eng.run()
    assert [id(r) for r in finished] == [id(c)] and c.output == want and c.finish_reason == "length"
    assert eng.runner.cache.free_pages() == [eng.runner.cache.tables.pools[0].num_pages]
