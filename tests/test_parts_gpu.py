"""Each part alone against the plain function of the same name; a decoder whose schedule names a layer
twice and lets a layer read another layer's cache; and toy parts defined here, registered, built and stepped
with no change to the framework's files: a mixer with state of its own, a feed-forward with routing and a
position encoding that adds learned rows."""
import json
import math

import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu


def make_ctx(model_like_specs, segments, page_size=4, dtype=torch.float32, num_pages=64):
    """A cache manager and the StepContext of one batch: segments = [(request id, first position, n tokens)]."""
    from vitna_anchor_b200.cache import CacheManager
    from vitna_anchor_b200.parts.base import GroupMeta, StepContext, Workspace
    cache = CacheManager(model_like_specs, page_size=page_size, num_pages=num_pages, max_requests=8, dtype=dtype, device="cuda")
    T = sum(n for _, _, n in segments)
    pos, seg, plan = [], [], []
    for s, (rid, first, n) in enumerate(segments):
        cache.open(rid)
        if first:
            cache.reserve_step([(rid, first)]); cache.commit_step([(rid, first)])
        plan.append((rid, n))
        pos += list(range(first, first + n)); seg += [s] * n
    cache.reserve_step(plan)
    maxb = max(len(cache.tables.get(rid).tables[0].blocks) for rid, _, _ in segments) if cache.groups else 1
    groups = []
    for g in range(len(cache.groups)):
        bt = np.zeros((len(segments), maxb), np.int32)
        sm = []
        for s, (rid, first, n) in enumerate(segments):
            blocks = cache.tables.get(rid).tables[g].blocks
            bt[s, :len(blocks)] = blocks
            sm += [blocks[p // page_size] * page_size + p % page_size for p in range(first, first + n)]
        groups.append(GroupMeta(torch.tensor(sm, dtype=torch.int32, device="cuda"), torch.from_numpy(bt).cuda(), maxb))
    starts = np.cumsum([0] + [n for _, _, n in segments]).astype(np.int32)
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device="cuda")
    ctx = StepContext(num_tokens=T, num_segments=len(segments), dtype=dtype, tokens=i32([0] * T), positions=i32(pos),
                      token_seg=i32(seg), seg_starts=i32(starts), seg_context=i32([f + n for _, f, n in segments]),
                      seg_slots=i32([cache.slot(rid) for rid, _, _ in segments]), groups=groups, caches=cache.views,
                      workspace=Workspace(torch.device("cuda"), 64), host_seg_lens=[n for _, _, n in segments],
                      host_seg_first_pos=[f for _, f, _ in segments], host_seg_slots=[cache.slot(rid) for rid, _, _ in segments],
                      max_seg_len=max(n for _, _, n in segments), max_context=max(f + n for _, f, n in segments))
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
    # second step: build its context by hand on the same cache
    from vitna_anchor_b200.parts.base import GroupMeta
    cache.open("b")
    cache.reserve_step([("a", 5), ("b", 7)])
    ps = cache.page_size
    ta, tb = cache.tables.get("a").tables[0].blocks, cache.tables.get("b").tables[0].blocks
    maxb = max(len(ta), len(tb))
    bt = np.zeros((2, maxb), np.int32); bt[0, :len(ta)] = np.maximum(ta, 0); bt[1, :len(tb)] = tb
    sm = [ta[p // ps] * ps + p % ps for p in range(9, 14)] + [tb[p // ps] * ps + p % ps for p in range(7)]
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device="cuda")
    ctx.num_tokens, ctx.num_segments = 12, 2
    ctx.positions, ctx.token_seg = i32(list(range(9, 14)) + list(range(7))), i32([0] * 5 + [1] * 7)
    ctx.groups = [GroupMeta(i32(sm), torch.from_numpy(bt).cuda(), maxb)]
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
    without writing it is built and stepped (it has no plain counterpart; it must differ from the other)."""
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
    assert np.isfinite(c).all() and np.abs(c - want).max() > 1e-3
    with pytest.raises(ValueError):
        with_schedule([LayerRun(0, 0), LayerRun(1, 0)])          # two writers of one cache layer


def test_a_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    """A made-up architecture whose mixer keeps a running mean of its inputs per request in the request's
    state slot.  Everything it needs is defined here; the framework's files are not touched."""
    from vitna_anchor_b200 import ops
    from vitna_anchor_b200.cache import StateSpec
    from vitna_anchor_b200.config import Architecture, register_architecture
    from vitna_anchor_b200.engine.loading import load_model, write_random_model
    from vitna_anchor_b200.engine.runner import ModelRunner, StepEntry
    from vitna_anchor_b200.models.decoder import DecoderModel, LayerRun
    from vitna_anchor_b200.parts import Mixer, make_part, register_part
    from vitna_anchor_b200.parts.embedding import Embedding, LMHead
    from vitna_anchor_b200.weights import WeightSpec

    class RunningMean(Mixer):
        """state = (sum of inputs so far [H], count); output_t = W (sum_t / count_t)."""

        def __init__(self, hidden, w):
            self.hidden, self.w = hidden, w

        def tensors(self):
            return [self.w]

        def cache_spec(self):
            return StateSpec((self.hidden + 1,), torch.float32)

        def forward(self, xn, ctx, cache, residual, write_cache=True):
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

    register_part("mixer", "toy_running_mean", RunningMean)

    def parse(cj):
        return dict(H=cj["hidden_size"], V=cj["vocab_size"], L=cj["num_hidden_layers"], I=cj["intermediate_size"])

    def manifest(c):
        m = [WeightSpec("embed.weight", (c["V"], c["H"])), WeightSpec("norm.weight", (c["H"],))]
        for l in range(c["L"]):
            m += [WeightSpec(f"layers.{l}.mix.weight", (c["H"], c["H"])), WeightSpec(f"layers.{l}.norm1.weight", (c["H"],)),
                  WeightSpec(f"layers.{l}.norm2.weight", (c["H"],)), WeightSpec(f"layers.{l}.gate_up.weight", (2 * c["I"], c["H"])),
                  WeightSpec(f"layers.{l}.down.weight", (c["H"], c["I"]))]
        return m

    def build(c, w, dtype, device):
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

    register_architecture(Architecture("ToyRunningMeanLM", parse, manifest, build, lambda n: "norm" in n), replace=True)
    cj = dict(architectures=["ToyRunningMeanLM"], hidden_size=24, vocab_size=50, num_hidden_layers=2, intermediate_size=40)
    write_random_model(str(tmp_path / "toy"), cj, 3, std=0.3)
    json.dump(cj, open(tmp_path / "toy" / "config.json", "w"))
    model = load_model(str(tmp_path / "toy"), "float32")
    assert model.cache_specs() == [StateSpec((25,), torch.float32)] * 2

    def run(cuts_a, cuts_b):
        runner = ModelRunner(model, page_size=4, num_pages=4, max_requests=2, max_batch_tokens=32, cuda_graphs=False)
        a, b = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3], [2, 7, 1, 8, 2, 8]
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
    a1, b1, c1 = run([10, 0], [0, 6])
    a2, b2, c2 = run([3, 2, 5], [1, 3, 2])
    assert np.abs(a1 - a2).max() < 1e-5 and np.abs(b1 - b2).max() < 1e-5
    assert np.abs(c1 - a1).max() < 1e-5 and np.abs(c2 - a1).max() < 1e-5
    assert np.abs(a1[1:] - a1[:-1]).max() > 1e-3          # the state does change the output from token to token


def test_toy_routed_feed_forward_and_learned_positions(tmp_path):
    """A made-up architecture with two more kinds of parts defined here and nowhere in the framework: a position
    encoding that adds a learned row per position to the embeddings (the attention then rotates nothing), and a
    feed-forward with routing (a float32 router picks one of three SwiGLU experts per token and weighs it by its
    softmax probability).  Whole prompts, cut prompts and decoding agree with a plain statement of the same model."""
    from vitna_anchor_b200 import ops
    from vitna_anchor_b200.config import Architecture, register_architecture
    from vitna_anchor_b200.engine.loading import load_model, write_random_model
    from vitna_anchor_b200.engine.runner import ModelRunner, StepEntry
    from vitna_anchor_b200.models.decoder import DecoderModel, LayerRun
    from vitna_anchor_b200.parts import FeedForward, PositionEncoding, make_part, register_part
    from vitna_anchor_b200.parts.embedding import Embedding, LMHead
    from vitna_anchor_b200.weights import WeightSpec

    class LearnedPositions(PositionEncoding):
        def __init__(self, table):
            self.table = table                      # float32 [max_positions, hidden]

        def tensors(self):
            return [self.table]

        def on_embeddings(self, x, ctx):
            x += self.table[ctx.positions.long()]

    class Top1Experts(FeedForward):
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

    register_part("position", "toy_learned", LearnedPositions)
    register_part("feed_forward", "toy_top1_experts", Top1Experts)
    E = 3

    def parse(cj):
        return dict(H=cj["hidden_size"], V=cj["vocab_size"], L=cj["num_hidden_layers"], I=cj["intermediate_size"],
                    nh=cj["num_attention_heads"], nkv=cj["num_key_value_heads"], hd=cj["head_dim"], P=cj["max_position_embeddings"])

    def manifest(c):
        m = [WeightSpec("embed.weight", (c["V"], c["H"])), WeightSpec("positions.weight", (c["P"], c["H"])), WeightSpec("norm.weight", (c["H"],))]
        for l in range(c["L"]):
            p = f"layers.{l}."
            m += [WeightSpec(p + "qkv.weight", ((c["nh"] + 2 * c["nkv"]) * c["hd"], c["H"])), WeightSpec(p + "o.weight", (c["H"], c["nh"] * c["hd"])),
                  WeightSpec(p + "norm1.weight", (c["H"],)), WeightSpec(p + "norm2.weight", (c["H"],)), WeightSpec(p + "router.weight", (E, c["H"]))]
            for e in range(E):
                m += [WeightSpec(p + f"experts.{e}.gate_up.weight", (2 * c["I"], c["H"])), WeightSpec(p + f"experts.{e}.down.weight", (c["H"], c["I"]))]
        return m

    def build(c, w, dtype, device):
        d = lambda n: w[n].to(device=device, dtype=dtype).contiguous()
        f = lambda n: w[n].to(device=device, dtype=torch.float32)
        position = make_part("position", "toy_learned", table=f("positions.weight"))
        blocks = []
        for l in range(c["L"]):
            p = f"layers.{l}."
            blocks.append(make_part(
                "block", "pre_norm",
                mixer_norm=make_part("norm", "rmsnorm", width=c["H"], eps=1e-5, weight=f(p + "norm1.weight")),
                mixer=make_part("mixer", "attention", hidden=c["H"], num_heads=c["nh"], num_kv_heads=c["nkv"], head_dim=c["hd"],
                                wqkv=d(p + "qkv.weight"), wo=d(p + "o.weight"), position=position),
                ffn_norm=make_part("norm", "rmsnorm", width=c["H"], eps=1e-5, weight=f(p + "norm2.weight")),
                ffn=make_part("feed_forward", "toy_top1_experts", hidden=c["H"], inter=c["I"], router=f(p + "router.weight"),
                              gate_up=[d(p + f"experts.{e}.gate_up.weight") for e in range(E)],
                              down=[d(p + f"experts.{e}.down.weight") for e in range(E)])))
        emb = Embedding(c["V"], c["H"], d("embed.weight"))
        return DecoderModel(embedding=emb, blocks=blocks, schedule=[LayerRun(l, l) for l in range(c["L"])],
                            final_norm=make_part("norm", "rmsnorm", width=c["H"], eps=1e-5, weight=f("norm.weight")),
                            lm_head=LMHead(c["V"], c["H"], emb.table), position=position, dtype=dtype, vocab_size=c["V"],
                            max_positions=c["P"])

    register_architecture(Architecture("ToyRoutedLM", parse, manifest, build, lambda n: "norm" in n), replace=True)
    cj = dict(architectures=["ToyRoutedLM"], hidden_size=40, vocab_size=61, num_hidden_layers=2, intermediate_size=24,
              num_attention_heads=4, num_key_value_heads=2, head_dim=12, max_position_embeddings=64)
    write_random_model(str(tmp_path / "toy"), cj, 11, std=0.25)
    json.dump(cj, open(tmp_path / "toy" / "config.json", "w"))
    model = load_model(str(tmp_path / "toy"), "float32")
    ids = [3, 14, 15, 9, 26, 5, 35, 8, 9, 7, 9, 32, 38, 46, 26, 43, 38, 32, 7, 9, 50, 28, 8]

    # the plain statement of this model, from the plain functions of the parts
    W = {k: v.astype(np.float32) for k, v in P.read_safetensors(str(tmp_path / "toy" / "model.safetensors")).items()}
    c = parse(cj)
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
    want = P.linear(P.rms_norm(x, W["norm.weight"], 1e-5), W["embed.weight"])
    assert all(len(set(pk.tolist())) > 1 for pk in picks)              # the router does send tokens to different experts

    def run(cuts):
        runner = ModelRunner(model, page_size=4, num_pages=8, max_requests=2, max_batch_tokens=32, cuda_graphs=False)
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
    runner = ModelRunner(model, page_size=4, num_pages=8, max_requests=2, max_batch_tokens=32, cuda_graphs=False)
    runner.open("b")
    moved = runner.step([StepEntry("b", ids[1:2], [0])]).cpu().numpy()   # token ids[1] at position 0 instead of 1
    assert np.abs(moved[0] - whole[1]).max() > 1e-3
