"""Trace replay on the GPU against the plain implementation: each request whole; most of it in one
step and the last 32 tokens one by one; in portions of changing size down to two tokens; and mixed,
up to four live requests with so few pages that they are used again.  In 32-bit and in bfloat16,
for both tiny configurations, through bin/trace_run as a user runs it."""
import numpy as np
import pytest

import plain_llama as P
from replay_util import Replay, changing_portions, mixed, tail_one_by_one, whole
from tiny_configs import TINIES, write_tiny

pytestmark = pytest.mark.gpu

# Largest |difference| allowed, as a fraction of max(1, largest |logit| of the plain implementation).
# Against the plain implementation: float32 is two float32 implementations that add in different
# orders; in bfloat16 the activations between kernels and the cache are rounded to 8 bits of mantissa
# (and a checkpoint stored in float32, as tinyB's, has its matrices rounded too), which with these
# sharp weights reaches a few percent of the logits' scale.
# Between two ways of cutting the same request: only the order of float32 sums may differ, which in
# bfloat16 now and then flips the rounding of an activation by one unit in the last place.
TOL = {"float32": 2e-5, "bfloat16": 8e-2}
TOL_CUT = {"float32": 2e-5, "bfloat16": 1e-2}

LENGTHS = {"tinyA": [5, 17, 33, 100, 64, 47], "tinyB": [1, 9, 40, 100, 130, 77]}


@pytest.fixture(scope="module")
def sharp_dirs(tmp_path_factory):
    """The tiny models with weights of std 0.15: attention is then far from uniform, so a wrong key,
    position or page changes the logits by much more than the tolerance."""
    root = tmp_path_factory.mktemp("sharp")
    return {name: write_tiny(str(root / name), tiny, std=0.15) for name, tiny in TINIES.items()}


def _requests(name, vocab, rng):
    return {f"{name}-{i}": [int(t) for t in rng.integers(0, vocab, n)] for i, n in enumerate(LENGTHS[name])}


def _compare(got, plain, tol, what):
    worst = 0.0
    for (rid, pos), row in got.items():
        ref = plain[rid][pos]
        worst = max(worst, float(np.abs(row - ref).max()) / max(1.0, float(np.abs(plain[rid]).max())))
    assert worst <= tol, f"{what}: largest difference {worst:.3e} of the logits' scale, allowed {tol:.1e}"
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tinyA", "tinyB"])
def test_every_way_of_cutting(name, dtype, sharp_dirs, tmp_path):
    cfg, W = P.read_model(sharp_dirs[name])
    vocab = cfg["V"]
    rng = np.random.default_rng(5)
    reqs = _requests(name, vocab, rng)
    plain = {rid: P.forward(cfg, W, ids) for rid, ids in reqs.items()}
    # the pool: four live requests, each rounded up to 64 positions
    live4 = sorted((-(-len(v) // 64) * 64 for v in reqs.values()), reverse=True)[:4]
    replay = Replay(sharp_dirs[name], dtype, tmp_path / "out", sum(live4))
    report = {}
    alone = {}

    def check(got, what, count):
        assert len(got) == count
        a = _compare(got, plain, TOL[dtype], what + " against the plain implementation")
        b = _compare(got, alone, TOL_CUT[dtype], what + " against the same request whole") if alone else 0.0
        report[what.split(":")[0]] = max(report.get(what.split(":")[0], (0, 0)), (a, b))

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
    print(f"\n{name} {dtype}: largest differences (against plain, against whole) as a fraction of scale: {report}")
