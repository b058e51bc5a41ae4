"""Trace replay on the GPU against the plain implementation: each request whole; most of it in one
step and the last 32 tokens one by one; in portions of changing size down to two tokens; and mixed,
up to four live requests with so few pages that they are used again, with small portions and with
portions of 65 to 200 tokens beside decoded tokens (what the scheduler produces by default).  In 32-bit
and in bfloat16, for both tiny configurations with their own page sizes, through bin/trace_run as a
user runs it.

In 32-bit every way of cutting must give the same BYTES as the request whole (the exact routing has
one kernel per operation and an order of sums that depends on the output element alone)."""
import numpy as np
import pytest

import plain_llama as P
from replay_util import Replay, changing_portions, mixed, tail_one_by_one, whole
from tiny_configs import TINIES, write_tiny

pytestmark = pytest.mark.gpu

# Largest |difference| allowed, as a fraction of max(1, largest |logit| of the plain implementation).
# Against the plain implementation: float32 is two float32 implementations that add in different
# orders; in bfloat16 the activations between kernels and the cache are rounded to 8 bits of mantissa
# (and a checkpoint stored in float32, as tinyB's, has its matrices rounded too).  The bfloat16 bounds are
# about twice the worst case measured on these models (the test prints what it measures).
# Between two ways of cutting the same request: float32 must agree bit for bit; "float32-fast" (the float32
# twins of the serving kernels, chosen by batch size) differs by the order of float32 sums; in bfloat16
# that order now and then flips the rounding of an activation by one unit in the last place.
TOL = {"float32": 2e-5, "float32-fast": 2e-5, "bfloat16": 8e-2}
TOL_CUT = {"float32": 0.0, "float32-fast": 2e-5, "bfloat16": 1e-2}
# bfloat16 against the plain implementation told to round where a 16-bit engine stores (plain_llama.forward(bf16=True)):
# what is left is the order of float32 sums and the exponential's last bits, which now and then flip a rounding.
TOL_ROUNDED = 1.5e-2

LENGTHS = {"tinyA": [5, 17, 33, 100, 64, 47], "tinyB": [1, 9, 40, 100, 130, 77]}
LONG_LENGTHS = {"tinyA": [260, 150, 330, 90, 210, 75, 180, 240], "tinyB": [240, 131, 300, 70, 201, 66, 170, 222]}


@pytest.fixture(scope="module")
def sharp_dirs(tmp_path_factory):
    """The tiny models with weights of std 0.15: attention is then far from uniform, so a wrong key,
    position or page changes the logits by much more than the tolerance.  The "-long" ones differ only in
    max_position_embeddings (512), so that portions of up to 200 tokens fit."""
    root = tmp_path_factory.mktemp("sharp")
    out = {name: write_tiny(str(root / name), tiny, std=0.15) for name, tiny in TINIES.items()}
    for name, tiny in TINIES.items():
        longer = dict(tiny, config=dict(tiny["config"], max_position_embeddings=512))
        out[name + "-long"] = write_tiny(str(root / (name + "-long")), longer, std=0.15)
    return out


def _requests(name, lengths, vocab, rng):
    return {f"{name}-{i}": [int(t) for t in rng.integers(0, vocab, n)] for i, n in enumerate(lengths)}


def _compare(got, want, tol, what):
    """want: {request: [positions, vocab]}.  tol 0 asks for the same bytes."""
    worst = 0.0
    for (rid, pos), row in got.items():
        ref = want[rid][pos]
        if tol == 0.0:
            assert np.array_equal(row, ref), f"{what}: position {pos} of {rid} differs by {np.abs(row - ref).max():.3e}; the same bytes are asked for"
            continue
        worst = max(worst, float(np.abs(row - ref).max()) / max(1.0, float(np.abs(want[rid]).max())))
    assert worst <= tol, f"{what}: largest difference {worst:.3e} of the logits' scale, allowed {tol:.1e}"
    return worst


def _replay(model_dir, mode, out_dir, max_tokens, kv_block, monkeypatch):
    dtype = "bfloat16" if mode == "bfloat16" else "float32"
    if mode == "float32-fast":
        monkeypatch.setenv("VITNA_FLOAT32_FAST", "1")
    else:
        monkeypatch.delenv("VITNA_FLOAT32_FAST", raising=False)
    return Replay(model_dir, dtype, out_dir, max_tokens, kv_block=kv_block)


@pytest.mark.parametrize("mode", ["float32", "float32-fast", "bfloat16"])
@pytest.mark.parametrize("name", ["tinyA", "tinyB"])
def test_every_way_of_cutting(name, mode, sharp_dirs, tmp_path, monkeypatch):
    cfg, W = P.read_model(sharp_dirs[name])
    vocab = cfg["V"]
    rng = np.random.default_rng(5)
    reqs = _requests(name, LENGTHS[name], vocab, rng)
    plain = {rid: P.forward(cfg, W, ids) for rid, ids in reqs.items()}
    rounded = {rid: P.forward(cfg, W, ids, bf16=True) for rid, ids in reqs.items()} if mode == "bfloat16" else None
    # the pool: four live requests, each rounded up to 64 positions; pages of the configuration's own size
    live4 = sorted((-(-len(v) // 64) * 64 for v in reqs.values()), reverse=True)[:4]
    replay = _replay(sharp_dirs[name], mode, tmp_path / "out", sum(live4), TINIES[name]["page_size"], monkeypatch)
    report = {}
    alone = {}

    def check(got, what, count):
        assert len(got) == count
        a = _compare(got, plain, TOL[mode], what + " against the plain implementation")
        b = _compare(got, alone, TOL_CUT[mode], what + " against the same request whole") if alone else 0.0
        c = _compare(got, rounded, TOL_ROUNDED, what + " against the plain implementation rounding as a 16-bit engine") if rounded else 0.0
        report[what.split(":")[0]] = max(report.get(what.split(":")[0], (0, 0, 0)), (a, b, c))

    try:
        whole_rows = {}
        for rid, ids in reqs.items():
            got = replay.run(whole(rid, ids), vocab)
            check(got, f"whole: {rid}", len(ids))
            whole_rows.update(got)
        alone = {rid: np.stack([whole_rows[(rid, p)] for p in range(len(ids))]) for rid, ids in reqs.items()}
        for rid, ids in reqs.items():
            check(replay.run(tail_one_by_one(rid, ids), vocab), f"last 32 one by one: {rid}", len(ids))
        for rid, ids in reqs.items():
            check(replay.run(changing_portions(rid, ids), vocab), f"changing portions: {rid}", len(ids))
        prompt_part = {rid: max(1, len(ids) - 12) for rid, ids in reqs.items()}
        for round_ in range(2):           # twice, so that every page of the pool has held another request
            check(replay.run(mixed(reqs, prompt_part, rng), vocab), "mixed", sum(len(v) for v in reqs.values()))
    finally:
        replay.close()
    print(f"\n{name} {mode}: largest differences (against plain, against whole, against plain with 16-bit rounding) as a fraction of scale: {report}")


@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tinyA", "tinyB"])
def test_large_portions_beside_decoded_tokens(name, mode, sharp_dirs, tmp_path, monkeypatch):
    """What the scheduler does by default: a prompt portion of 65 to 200 tokens in one step with single decoded
    tokens of one to three other requests.  Such a step takes the prompt-sized kernels for its products and, in the
    same call, the decode kernel for some tokens and the prompt kernel for others.  Requests of up to 330 tokens,
    the last 40 decoded; four live at a time in a pool that is used twice over."""
    model_dir = sharp_dirs[name + "-long"]
    cfg, W = P.read_model(model_dir)
    vocab = cfg["V"]
    rng = np.random.default_rng(31)
    reqs = _requests(name, LONG_LENGTHS[name], vocab, rng)
    plain = {rid: P.forward(cfg, W, ids) for rid, ids in reqs.items()}
    rounded = {rid: P.forward(cfg, W, ids, bf16=True) for rid, ids in reqs.items()} if mode == "bfloat16" else None
    live4 = sorted((-(-len(v) // 64) * 64 for v in reqs.values()), reverse=True)[:4]
    replay = _replay(model_dir, mode, tmp_path / "out", sum(live4), TINIES[name]["page_size"], monkeypatch)
    try:
        alone = {}
        for rid, ids in reqs.items():
            got = replay.run(whole(rid, ids), vocab)
            alone[rid] = np.stack([got[(rid, p)] for p in range(len(ids))])
        a0 = _compare({(r, p): alone[r][p] for r in alone for p in range(len(alone[r]))}, plain, TOL[mode], "whole against plain")
        prompt_part = {rid: len(ids) - 40 for rid, ids in reqs.items()}
        worst = (a0, 0.0)
        for round_ in range(2):
            steps = mixed(reqs, prompt_part, rng, portions=(65, 201), one_prompt_at_a_time=True)
            sizes = [sum(len(t) for _, t, _ in entries) for entries, _ in steps]
            beside = [s for (entries, _), s in zip(steps, sizes)
                      if s > 64 and any(len(t) == 1 for _, t, _ in entries) and any(len(t) > 64 for _, t, _ in entries)]
            assert len(beside) >= 4, "the schedule was meant to put large portions beside decoded tokens"
            got = replay.run(steps, vocab)
            assert len(got) == sum(len(v) for v in reqs.values())
            worst = max(worst, (_compare(got, plain, TOL[mode], "large portions beside decodes against the plain implementation"),
                                _compare(got, alone, TOL_CUT[mode], "large portions beside decodes against the same request whole")))
            if rounded:
                r = _compare(got, rounded, TOL_ROUNDED, "large portions beside decodes against the plain implementation rounding as a 16-bit engine")
                print(f"\n{name}: against plain with 16-bit rounding: {r:.3e}")
    finally:
        replay.close()
    print(f"\n{name} {mode}: large portions, largest differences (against plain, against whole): {worst}")


def test_float32_bytes_do_not_depend_on_the_batch_or_the_pages(sharp_dirs, tmp_path, monkeypatch):
    """One request cut one way, run alone in a fresh pool; then cut the same way beside three other requests, after
    the pool has been used, so that it lies on other page ids and in other rows of the batch: the same bytes."""
    name = "tinyB"
    cfg, W = P.read_model(sharp_dirs[name])
    vocab = cfg["V"]
    rng = np.random.default_rng(77)
    ids = [int(t) for t in rng.integers(0, vocab, 120)]
    cuts = [9, 2, 40, 1, 1, 30, 1, 17, 1, 1, 1, 16]
    others = {f"o{i}": [int(t) for t in rng.integers(0, vocab, n)] for i, n in enumerate((90, 75, 130))}

    def my_steps(rid, with_others):
        at = {k: 0 for k in others}
        steps, p = [], 0
        for i, n in enumerate(cuts):
            entries = []
            if with_others:
                for j, (k, v) in enumerate(others.items()):
                    m = [5, 1, 23][(i + j) % 3]
                    m = min(m, len(v) - at[k])
                    if m > 0 and (i + j) % 4 != 3:
                        entries.append((k, v[at[k]:at[k] + m], []))
                        at[k] += m
                entries.insert(min(len(entries), i % 3), (rid, ids[p:p + n], range(n)))
            else:
                entries.append((rid, ids[p:p + n], range(n)))
            steps.append((entries, []))
            p += n
        steps[-1] = (steps[-1][0], [rid] + ([k for k in others] if with_others else []))
        return steps

    replay = _replay(sharp_dirs[name], "float32", tmp_path / "out", 4 * 192, TINIES[name]["page_size"], monkeypatch)
    try:
        a = replay.run(my_steps("alone", False), vocab)
        replay.run(whole("filler", [int(t) for t in rng.integers(0, vocab, 77)]), vocab)     # the pool has been used
        replay.run([([("held", ids[:50], [])], [])], vocab)                                   # and part of it stays held
        b = replay.run(my_steps("beside", True), vocab)
    finally:
        replay.close()
    assert len(a) == len(b) == len(ids)
    for p in range(len(ids)):
        assert np.array_equal(a[("alone", p)], b[("beside", p)]), f"position {p} differs"
    plain = P.forward(cfg, W, ids)
    assert max(np.abs(a[("alone", p)] - plain[p]).max() for p in range(len(ids))) <= 2e-5 * max(1.0, np.abs(plain).max())
