"""Each part alone against the plain function of the same name; a decoder whose schedule names a layer
twice and lets a layer read another layer's cache; and toy parts defined under tests/ (toy_archs.py), registered,
built and stepped with no change to the framework's files: a mixer with state of its own, a feed-forward with
routing and a position encoding that adds learned rows; through the step function, the Python entry point and
the replay program, with the engine's default settings."""
import json
import math

import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu


def make_ctx(model_like_specs, segments, page_size=4, dtype=torch.float32, num_pages=64):
    """A cache manager and the StepContext of one batch, made by the step function's own builder:
    segments = [(request id, first position, n tokens)].  ctx.extra["builder"] builds further batches on the same cache."""
    from vitna_anchor_b200.cache import CacheManager
    from vitna_anchor_b200.engine.context import ContextBuilder
    from vitna_anchor_b200.parts.base import Workspace
    cache = CacheManager(model_like_specs, page_size=page_size, num_pages=num_pages, max_requests=8, dtype=dtype, device="cuda")
    builder = ContextBuilder(cache, dtype, Workspace(torch.device("cuda"), 64), max_batch_tokens=64, max_segments=8,
                             max_model_len=page_size * num_pages, device="cuda")
    plan = []
    for rid, first, n in segments:
        cache.open(rid)
        if first:
            cache.reserve_step([(rid, first)]); cache.commit_step([(rid, first)])
        plan.append((rid, n))
    cache.reserve_step(plan)
    ctx, _ = builder.build([(rid, [0] * n, []) for rid, _, n in segments])
    ctx.extra["builder"] = builder
    return cache, ctx


def test_rmsnorm_part():
    from vitna_anchor_b200.parts.norms import RMSNorm
    w = 1 + 0.1 * torch.randn(50)
    x = torch.randn(7, 50) * 2
    _, ctx = make_ctx([], [("a", 0, 7)])
    y = RMSNorm(50, 1e-6, w.cuda()).forward(x.cuda(), ctx, "t")
    assert (y.cpu().numpy() - P.rms_norm(x.numpy(), w.numpy(), 1e-6)).__abs__().max() < 1e-5


def test_rotary_tables():
    from vitna_anchor_b200.parts.rotary import Rotary
    r = Rotary(48, 130000.0, 300, "cuda")
    cos, sin = P.rope_tables(np.arange(300), 48, 130000.0)
    c, s, rot = r.rotary_tables()
    assert rot == 48 and np.abs(c.cpu().numpy() - cos).max() < 1e-6 and np.abs(s.cpu().numpy() - sin).max() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from vitna_anchor_b200.parts.feed_forward import SwiGLU
    H, I, T = 40, 72, 6
    wg, wu, wd = torch.randn(I, H) * 0.3, torch.randn(I, H) * 0.3, torch.randn(H, I) * 0.3
    wg, wu, wd = (t.to(dtype).float() for t in (wg, wu, wd))
    xn = torch.randn(T, H).to(dtype).float()
    res = torch.randn(T, H)
    _, ctx = make_ctx([], [("a", 0, T)], dtype=dtype)
    part = SwiGLU(H, I, torch.cat([wg, wu]).to(dtype).cuda(), wd.to(dtype).cuda())
    out = res.clone().cuda()
    part.forward(xn.to(dtype).cuda(), ctx, out)
    want = res.numpy() + P.swiglu(xn.numpy(), wg.numpy(), wu.numpy(), wd.numpy())
    assert np.abs(out.cpu().numpy() - want).max() <= (1e-5 if dtype == torch.float32 else 3e-2) * np.abs(want).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 6])
def test_attention_part_in_two_steps(dtype, window):
    """The mixer alone: a request's first 9 positions in one step, the next 5 in another beside a second
    request; against plain projections, rotation and attention over the whole sequences."""
    from vitna_anchor_b200.parts.attention import PagedAttention
    from vitna_anchor_b200.parts.rotary import Rotary
    H, nh, nkv, hd = 40, 6, 2, 16
    rng = np.random.default_rng(0)
    rnd = lambda *s: torch.from_numpy((rng.standard_normal(s) * 0.4).astype(np.float32)).to(dtype).float()
    wq, wk, wv, wo = rnd(nh * hd, H), rnd(nkv * hd, H), rnd(nkv * hd, H), rnd(H, nh * hd)
    xa, xb = rnd(14, H) * 3, rnd(7, H) * 3
    part = PagedAttention(H, nh, nkv, hd, torch.cat([wq, wk, wv]).to(dtype).cuda(), wo.to(dtype).cuda(),
                          Rotary(hd, 10000.0, 64, "cuda"), window=window)

    def plain(x):
        T = x.shape[0]
        q = P.linear(x.numpy(), wq.numpy()).reshape(T, nh, hd); k = P.linear(x.numpy(), wk.numpy()).reshape(T, nkv, hd)
        v = P.linear(x.numpy(), wv.numpy()).reshape(T, nkv, hd)
        cos, sin = P.rope_tables(np.arange(T), hd, 10000.0)
        att = P.causal_attention(P.rope_half(q, cos, sin), P.rope_half(k, cos, sin), v, window=window or None)
        return P.linear(att, wo.numpy())
    want_a, want_b = plain(xa), plain(xb)
    cache, ctx = make_ctx([part.cache_spec()], [("a", 0, 9)], dtype=dtype)
    out1 = torch.zeros(9, H, device="cuda")
    part.forward(xa[:9].to(dtype).cuda(), ctx, ctx.caches[0], out1)
    cache.commit_step([("a", 9)])
    # second step: five more tokens of "a" beside the seven of a new request, on the same cache
    cache.open("b")
    cache.reserve_step([("a", 5), ("b", 7)])
    ctx, _ = ctx.extra["builder"].build([("a", [0] * 5, []), ("b", [0] * 7, [])])
    out2 = torch.zeros(12, H, device="cuda")
    part.forward(torch.cat([xa[9:], xb]).to(dtype).cuda(), ctx, ctx.caches[0], out2)
    got_a = torch.cat([out1, out2[:5]]).cpu().numpy()
    tol = (2e-5 if dtype == torch.float32 else 4e-2) * max(np.abs(want_a).max(), np.abs(want_b).max())
    assert np.abs(got_a - want_a).max() <= tol and np.abs(out2[5:].cpu().numpy() - want_b).max() <= tol


def _tiny_llama_weights(model_dir):
    from vitna_anchor_b200.config import read_config_json, resolve
    from vitna_anchor_b200.weights import load_weights
    cj = read_config_json(model_dir)
    arch = resolve(cj)
    cfg = arch.parse_config(cj)
    return cfg, load_weights(model_dir, arch.manifest(cfg))


def test_schedule_names_a_layer_twice_and_shares_a_cache(tiny_dirs):
    """Blocks 0, 1, 0 of tinyA run in that order, each run with a cache of its own: against the plain
    implementation told the same order.  Then a schedule whose last run reads the first run's cache
    without writing it, whole and in two steps: against the plain implementation told the same."""
    from vitna_anchor_b200.models.decoder import DecoderModel, LayerRun
    from vitna_anchor_b200.models.llama import build_llama
    from vitna_anchor_b200.engine.runner import ModelRunner, StepEntry
    cfg, weights = _tiny_llama_weights(tiny_dirs["tinyA"])
    base = build_llama(cfg, weights, torch.float32, "cuda")

    def with_schedule(schedule):
        return DecoderModel(embedding=base.embedding, blocks=base.blocks, schedule=schedule, final_norm=base.final_norm,
                            lm_head=base.lm_head, position=base.position, dtype=base.dtype, vocab_size=base.vocab_size,
                            max_positions=base.max_positions)
    ids = [5, 17, 3, 200, 41, 8, 99, 150, 7, 7, 23]
    twice = with_schedule([LayerRun(0, 0), LayerRun(1, 1), LayerRun(0, 2)])
    assert len(twice.cache_specs()) == 3
    runner = ModelRunner(twice, page_size=4, num_pages=32, max_requests=2, max_batch_tokens=32)
    runner.open("r")
    a = runner.step([StepEntry("r", ids[:6], range(6))]).cpu().numpy()
    b = runner.step([StepEntry("r", ids[6:], range(5))]).cpu().numpy()
    pc, pw = P.read_model(tiny_dirs["tinyA"])
    want = P.forward(pc, pw, ids, layer_order=[0, 1, 0])
    assert np.abs(np.concatenate([a, b]) - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
    shared = with_schedule([LayerRun(0, 0), LayerRun(1, 1), LayerRun(0, 0, write_cache=False)])
    assert len(shared.cache_specs()) == 2
    runner2 = ModelRunner(shared, page_size=4, num_pages=32, max_requests=2, max_batch_tokens=32)
    runner2.open("r")
    c = runner2.step([StepEntry("r", ids, range(len(ids)))]).cpu().numpy()
    want_shared = P.forward(pc, pw, ids, layer_order=[0, 1, 0], reads={2: 0})
    assert np.abs(want_shared - want).max() > 1e-3            # sharing the cache does change the logits
    assert np.abs(c - want_shared).max() <= 2e-5 * max(1.0, np.abs(want_shared).max())
    runner2.open("s")
    d = np.concatenate([runner2.step([StepEntry("s", ids[:4], range(4))]).cpu().numpy(),
                        runner2.step([StepEntry("s", ids[4:], range(7))]).cpu().numpy()])
    assert np.abs(d - want_shared).max() <= 2e-5 * max(1.0, np.abs(want_shared).max())
    with pytest.raises(ValueError):
        with_schedule([LayerRun(0, 0), LayerRun(1, 0)])          # two writers of one cache layer


def test_a_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    """A made-up architecture whose mixer keeps a running mean of its inputs per request in the request's
    state slot (tests/toy_archs.py; the framework's files are not touched).  With the engine's default settings:
    the model says it is not capture-safe, so nothing is captured; cut and batched in different ways, and with
    steps repeated many times, the logits are those of the plain statement; a slot that is taken again starts
    from zero; a step that fails after the mixer wrote its state leaves no trace; the state cannot be truncated."""
    import toy_archs as T
    from vitna_anchor_b200.cache import CacheError, StateSpec
    from vitna_anchor_b200.engine.loading import load_model
    from vitna_anchor_b200.engine.runner import ModelRunner, StepEntry, StepFailed
    model_dir = T.write_toy(str(tmp_path / "toy"), T.RUNNING_MEAN_CONFIG, 3, 0.3)
    model = load_model(model_dir, "float32")
    assert model.cache_specs() == [StateSpec((25,), torch.float32)] * 2
    assert not model.capture_safe
    a, b = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5, 8, 9, 7, 9, 3, 2, 3, 8, 4, 6, 2], [2, 7, 1, 8, 2, 8, 1, 8, 2, 8, 4, 5]
    want_a, want_b = T.plain_running_mean(model_dir, a), T.plain_running_mean(model_dir, b)
    tol = 2e-5 * max(1.0, np.abs(want_a).max(), np.abs(want_b).max())

    def run(cuts_a, cuts_b):
        runner = ModelRunner(model, page_size=4, num_pages=4, max_requests=2, max_batch_tokens=32)
        assert not runner.cuda_graphs
        runner.open("a"); runner.open("b")
        rows = {"a": [], "b": []}
        pa = pb = 0
        for na, nb in zip(cuts_a, cuts_b):
            entries = []
            if na: entries.append(StepEntry("a", a[pa:pa + na], range(na)))
            if nb: entries.append(StepEntry("b", b[pb:pb + nb], range(nb)))
            out = runner.step(entries).cpu().numpy()
            rows["a"].append(out[:na]); rows["b"].append(out[na:])
            pa += na; pb += nb
        runner.close("a")
        runner.open("c")                       # takes a's slot: the state must start from zero again
        c = runner.step([StepEntry("c", a, range(len(a)))]).cpu().numpy()
        return np.concatenate(rows["a"]), np.concatenate(rows["b"]), c
    a1, b1, c1 = run([22, 0], [0, 12])
    # portions, then the same counts step after step (what a captured graph would replay)
    a2, b2, c2 = run([3, 2, 5] + [1] * 12, [1, 3, 2] + [1] * 6 + [0] * 6)
    for got_a, got_b, got_c in ((a1, b1, c1), (a2, b2, c2)):
        assert np.abs(got_a - want_a).max() <= tol and np.abs(got_b - want_b).max() <= tol and np.abs(got_c - want_a).max() <= tol
    assert np.abs(a1[1:] - a1[:-1]).max() > 1e-3          # the state does change the output from token to token

    # a step that raises after the first layer's mixer wrote its state: the state is put back, and the same
    # step again gives what it gives without the failure
    runner = ModelRunner(model, page_size=4, num_pages=4, max_requests=2, max_batch_tokens=32)
    runner.open("a")
    first = runner.step([StepEntry("a", a[:6], range(6))]).cpu().numpy()
    runner.fail_after_run_once(0)
    with pytest.raises(StepFailed):
        runner.step([StepEntry("a", a[6:11], range(5))])
    assert runner.length("a") == 6
    again = runner.step([StepEntry("a", a[6:11], range(5))]).cpu().numpy()
    assert np.abs(np.concatenate([first, again]) - want_a[:11]).max() <= tol
    with pytest.raises(CacheError):
        runner.cache.truncate("a", 4)                     # a running mean cannot be taken back


def test_toy_architectures_through_the_entry_point_and_the_replay_program(tmp_path, monkeypatch):
    """The state mixer and the learned positions through Engine.generate (default settings) and through bin/trace_run
    as a child process that learns the architectures from VITNA_ANCHOR_PLUGINS: greedy tokens and logits against
    the plain statements.  The capture-safe toy is replayed from graphs; the other is never captured."""
    import toy_archs as T
    from replay_util import Replay, changing_portions, tail_one_by_one, whole
    from vitna_anchor_b200.engine.engine import Engine
    rm_dir = T.write_toy(str(tmp_path / "rm"), T.RUNNING_MEAN_CONFIG, 3, 0.3)
    lp_dir = T.write_toy(str(tmp_path / "lp"), dict(T.LEARNED_CONFIG, architectures=["ToyLearnedLM"]), 11, 0.25)
    rng = np.random.default_rng(8)

    def plain_greedy(fn, prompt, n):
        ids, rows = list(prompt), []
        for _ in range(n):
            rows.append(fn(ids)[-1]); ids.append(int(np.argmax(rows[-1])))
        return ids[len(prompt):], np.stack(rows)

    for model_dir, fn, vocab, captured in ((rm_dir, lambda ids: T.plain_running_mean(rm_dir, ids), 50, False),
                                           (lp_dir, lambda ids: T.plain_learned(lp_dir, ids, False)[0], 61, True)):
        prompts = [[int(t) for t in rng.integers(0, vocab, n)] for n in (7, 19, 3)]
        eng = Engine(model_dir, dtype="float32", kv_block=4, parallel=3, max_batch_tokens=16)
        assert eng.runner.cuda_graphs == captured
        out_file = str(tmp_path / "rows.f32")
        got = eng.generate(prompts, max_new=24, logits_out=out_file)
        want0, rows0 = plain_greedy(fn, prompts[0], 24)
        mine = np.fromfile(out_file, "<f4").reshape(24, vocab)
        assert got[0] == want0 and np.abs(mine - rows0).max() <= 2e-5 * max(1.0, np.abs(rows0).max())
        for p, g in zip(prompts[1:], got[1:]):
            assert g == plain_greedy(fn, p, 24)[0]
        assert (eng.runner.graph_replays > 10) == captured
        # the replay program, as a child process
        ids = [int(t) for t in rng.integers(0, vocab, 60)]
        want = fn(ids)
        replay = Replay(model_dir, "float32", tmp_path / f"out{int(captured)}", 128, kv_block=4, plugins="toy_archs")
        try:
            for steps in (whole("w", ids), tail_one_by_one("t", ids), changing_portions("c", ids)):
                got_rows = replay.run(steps, vocab)
                assert len(got_rows) == len(ids)
                worst = max(float(np.abs(row - want[pos]).max()) for (_, pos), row in got_rows.items())
                assert worst <= 2e-5 * max(1.0, np.abs(want).max())
        finally:
            replay.close()


def test_toy_routed_feed_forward_and_learned_positions(tmp_path):
    """A made-up architecture with two more kinds of parts defined under tests/ and nowhere in the framework: a
    position encoding that adds a learned row per position to the embeddings (the attention then rotates nothing),
    and a feed-forward with routing (a float32 router picks one of three SwiGLU experts per token and weighs it by its
    softmax probability).  Whole prompts, cut prompts and decoding, with the engine's default settings, agree with a
    plain statement of the same model."""
    import toy_archs as T
    from vitna_anchor_b200.engine.loading import load_model
    from vitna_anchor_b200.engine.runner import ModelRunner, StepEntry
    model_dir = T.write_toy(str(tmp_path / "toy"), dict(T.LEARNED_CONFIG, architectures=["ToyRoutedLM"]), 11, 0.25)
    model = load_model(model_dir, "float32")
    assert not model.capture_safe                                      # the routing reads its picks on the host
    ids = [3, 14, 15, 9, 26, 5, 35, 8, 9, 7, 9, 32, 38, 46, 26, 43, 38, 32, 7, 9, 50, 28, 8]
    want, picks = T.plain_learned(model_dir, ids, True)
    assert all(len(set(pk.tolist())) > 1 for pk in picks)              # the router does send tokens to different experts

    def run(cuts):
        runner = ModelRunner(model, page_size=4, num_pages=8, max_requests=2, max_batch_tokens=32)
        runner.open("a")
        rows, at = [], 0
        for n in cuts:
            rows.append(runner.step([StepEntry("a", ids[at:at + n], range(n))]).cpu().numpy())
            at += n
        return np.concatenate(rows)
    whole = run([len(ids)])
    cut = run([5, 2, 9, 1, 1, 1, 1, 1, 1, 1])
    scale = max(1.0, np.abs(want).max())
    assert np.abs(whole - want).max() <= 2e-5 * scale
    assert np.abs(cut - want).max() <= 2e-5 * scale
    # the same token at another position gives other logits: the learned rows are added
    runner = ModelRunner(model, page_size=4, num_pages=8, max_requests=2, max_batch_tokens=32)
    runner.open("b")
    moved = runner.step([StepEntry("b", ids[1:2], [0])]).cpu().numpy()   # token ids[1] at position 0 instead of 1
    assert np.abs(moved[0] - whole[1]).max() > 1e-3


def test_a_norm_defined_elsewhere_is_fused_if_it_says_it_is_rms_like():
    """The built-in mixer and feed-forward apply a norm in their first kernel when the norm says that it has the RMS form
    (Norm.as_rms), whatever its class; a norm of another form runs as a kernel of its own.  Both give what the plain
    functions give."""
    from vitna_anchor_b200 import ops
    from vitna_anchor_b200.parts import Norm
    from vitna_anchor_b200.parts.feed_forward import SwiGLU

    class MyRms(Norm):                       # not the framework's class, but the same formula
        def __init__(self, w, eps):
            self.w, self.eps = w, eps

        def as_rms(self):
            return self.w, self.eps

        def forward(self, x, ctx, name, rows=None):
            out = ctx.workspace.rows(name, x.shape[0] if rows is None else rows.shape[0], x.shape[1], ctx.dtype)
            return ops.rmsnorm_rows(x, self.w, self.eps, out, rows)

    class ScaleOnly(Norm):                   # y = x * w: not of the RMS form
        def __init__(self, w):
            self.w = w

        def forward(self, x, ctx, name, rows=None):
            return (x * self.w).to(ctx.dtype)

    H, I, T = 64, 96, 5
    dtype = torch.bfloat16
    rnd = lambda *s: (torch.randn(*s) * 0.3).to(dtype).float()
    wg, wu, wd = rnd(I, H), rnd(I, H), rnd(H, I)
    w = (1 + 0.1 * torch.randn(H)).float()
    x = torch.randn(T, H) * 2
    _, ctx = make_ctx([], [("a", 0, T)], dtype=dtype)
    part = SwiGLU(H, I, torch.cat([wg, wu]).to(dtype).cuda(), wd.to(dtype).cuda())
    rms, scale = MyRms(w.cuda(), 1e-5), ScaleOnly(w.cuda())
    assert part.fuses_norm(rms, ctx) and not part.fuses_norm(scale, ctx)
    fused = x.clone().cuda()
    part.forward(fused, ctx, fused, norm=rms)                                   # the norm inside the first kernel
    apart = x.clone().cuda()
    part.forward(rms.forward(apart, ctx, "t.xn"), ctx, apart)                   # the norm as a kernel of its own
    xn = torch.from_numpy(P.rms_norm(x.numpy(), w.numpy(), 1e-5)).to(dtype).float().numpy()
    want = x.numpy() + P.swiglu(xn, wg.numpy(), wu.numpy(), wd.numpy(), rnd=P.bf16_round)
    tol = 2e-2 * np.abs(want).max()
    assert np.abs(fused.cpu().numpy() - want).max() <= tol and np.abs(apart.cpu().numpy() - want).max() <= tol
    other = x.clone().cuda()
    part.forward(scale.forward(other, ctx, "t.xn"), ctx, other)
    xs = (x * w).to(dtype).float().numpy()
    want2 = x.numpy() + P.swiglu(xs, wg.numpy(), wu.numpy(), wd.numpy(), rnd=P.bf16_round)
    assert np.abs(other.cpu().numpy() - want2).max() <= 2e-2 * np.abs(want2).max()
