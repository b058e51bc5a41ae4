"""The scheduler's decisions, on the host with a cache manager that holds no tensors."""
import pytest
import torch

from vitna_anchor_b200.cache import CacheManager, KVSpec
from vitna_anchor_b200.engine.scheduler import FINISHED, Request, RequestRefused, Scheduler
from vitna_anchor_b200.sampling.params import SamplingParams


def make(pages=16, page_size=4, max_requests=4, budget=16, ctx=64):
    cache = CacheManager([KVSpec(1, 16), KVSpec(1, 16)], page_size=page_size, num_pages=pages, max_requests=max_requests,
                         dtype=torch.float32, device="cpu", allocate=False)
    return cache, Scheduler(cache, max_batch_tokens=budget, max_model_len=ctx)


def run_plan(cache, sched, plan, token=7):
    """What the engine does with a plan, without a model: reserve, commit, hand back one token per sampler."""
    cache.reserve_step([(p.request.request_id, len(p.tokens)) for p in plan])
    cache.commit_step([(p.request.request_id, len(p.tokens)) for p in plan])
    cache.check()
    return sched.update(plan, [token] * sum(p.samples for p in plan))


def test_refusals():
    cache, s = make(pages=4, ctx=32)
    with pytest.raises(RequestRefused):
        s.add(Request("e", []))
    with pytest.raises(RequestRefused):
        s.add(Request("long", [1] * 30, max_new=3))            # 33 > ctx
    with pytest.raises(RequestRefused):
        s.add(Request("big", [1] * 10, max_new=8))             # needs 17 cached positions, the pool holds 16
    s.add(Request("ok", [1] * 10, max_new=7))
    with pytest.raises(ValueError):
        s.add(Request("p", [1], sampling=SamplingParams(1.0, 0, 0.0)))


def test_budget_cuts_prompts_and_decodes_go_first():
    cache, s = make(budget=16, pages=64, ctx=128)
    a = Request("a", list(range(1, 41)), max_new=3)
    b = Request("b", list(range(1, 7)), max_new=3)
    s.add(a); s.add(b)
    p1 = s.schedule()
    assert [(p.request.request_id, len(p.tokens), p.samples) for p in p1] == [("a", 16, False)]
    run_plan(cache, s, p1)
    p2 = s.schedule()
    assert [(p.request.request_id, len(p.tokens)) for p in p2] == [("a", 16)]
    run_plan(cache, s, p2)
    p3 = s.schedule()            # a's last 8 prompt tokens, then b is admitted with what is left of the budget
    assert [(p.request.request_id, len(p.tokens), p.samples) for p in p3] == [("a", 8, True), ("b", 6, True)]
    assert p3[0].tokens == list(range(33, 41))
    run_plan(cache, s, p3)
    p4 = s.schedule()            # both decode: one token each, the one just sampled
    assert [(p.request.request_id, p.tokens, p.samples) for p in p4] == [("a", [7], True), ("b", [7], True)]
    run_plan(cache, s, p4)
    done = run_plan(cache, s, s.schedule())
    assert {r.request_id for r in done} == {"a", "b"} and all(r.finish_reason == "length" for r in done)
    assert a.output == [7, 7, 7] and not s.has_work()
    assert cache.free_pages() == [64] and cache.tables.slots.free_slots == 4


def test_decode_beside_a_prompt_portion():
    cache, s = make(budget=8, pages=64, ctx=128)
    s.add(Request("a", [1, 2, 3], max_new=10))
    run_plan(cache, s, s.schedule())
    s.add(Request("b", list(range(1, 30)), max_new=2))
    p = s.schedule()
    assert [(x.request.request_id, len(x.tokens)) for x in p] == [("a", 1), ("b", 7)]      # 1 + 7 = the budget


def test_stop_token_finishes_and_frees():
    cache, s = make()
    r = Request("a", [1, 2, 3], max_new=10, stop_ids={7})
    s.add(r)
    done = run_plan(cache, s, s.schedule(), token=7)
    assert done == [r] and r.finish_reason == "stop" and r.state == FINISHED and cache.free_pages() == [16]


def test_slots_limit_admission():
    cache, s = make(max_requests=2, pages=64, ctx=128)
    for i in range(3):
        s.add(Request(i, [1, 2], max_new=2))
    p = s.schedule()
    assert [x.request.request_id for x in p] == [0, 1] and len(s.waiting) == 1
    run_plan(cache, s, p)
    run_plan(cache, s, s.schedule())          # 0 and 1 finish
    assert [x.request.request_id for x in s.schedule()] == [2]


def test_pages_run_out_preempts_the_newest_and_it_comes_back():
    cache, s = make(pages=4, page_size=4, budget=32, ctx=64)          # 16 positions in all
    a = Request("a", [1] * 7, max_new=6)
    b = Request("b", [2] * 7, max_new=6)
    s.add(a); s.add(b)
    run_plan(cache, s, s.schedule())          # both prompts: 2 pages each, none free; each sampled one token
    assert cache.free_pages() == [0]
    run_plan(cache, s, s.schedule())          # position 7 of each still fits its second page
    p = s.schedule()                          # position 8 needs a third page: b, the newest, is preempted
    assert [x.request.request_id for x in p] == ["a"] and s.preempted_total == 1
    assert b.state == "waiting" and b.num_computed == 0 and b.output == [7, 7] and s.waiting[0] is b
    assert cache.free_pages() == [2]          # b's two pages are back
    run_plan(cache, s, p)
    steps = 0
    while s.has_work():
        plan = s.schedule()
        ids = [x.request.request_id for x in plan]
        if "b" in ids and b.num_computed == 0:
            x = plan[ids.index("b")]
            assert x.tokens == (b.prompt + b.output)[:len(x.tokens)]      # what it had generated is prompt now
        run_plan(cache, s, plan)
        steps += 1
        assert steps < 100
    assert len(a.output) == 6 and len(b.output) == 6 and b.preemptions >= 1
    assert cache.free_pages() == [4]
    cache.check()


def test_a_prompt_is_cut_where_the_free_pages_end():
    cache, s = make(pages=4, page_size=4, budget=32, ctx=64)
    a = Request("a", [1] * 6, max_new=2)
    b = Request("b", [2] * 12, max_new=2)
    s.add(a); s.add(b)
    p = s.schedule()
    assert [(x.request.request_id, len(x.tokens), x.samples) for x in p] == [("a", 6, True), ("b", 8, False)]


def test_the_metadata_buffer_holds_the_largest_legal_step():
    """The step function's metadata buffer is sized by a bound (meta_words); whatever mixture of segments a step may
    legally hold must fit it: many segments of two tokens at small limits, all tokens wanted, wide block tables."""
    import random
    from vitna_anchor_b200.engine.context import meta_words, words_used
    rng = random.Random(0)
    for max_tokens, max_segments, max_blocks, groups in [(16, 8, 4, 1), (17, 16, 64, 2), (64, 64, 2, 1), (2048, 64, 512, 1),
                                                         (130, 40, 3, 3), (5, 64, 8, 1)]:
        bound = meta_words(max_tokens, max_segments, max_blocks, groups)
        S = min(max_segments, max_tokens // 2)
        cases = [[2] * S + ([max_tokens - 2 * S] if max_tokens - 2 * S and S < max_segments else []),      # segments of two tokens
                 [1] * min(max_segments, max_tokens), [max_tokens]]
        for _ in range(200):
            lens, left = [], max_tokens
            while left and len(lens) < max_segments:
                n = rng.choice([1, 2, 3, 63, 64, 65, 127, 128, 129, left])
                n = max(1, min(n, left))
                lens.append(n); left -= n
            cases.append(lens)
        for lens in cases:
            assert words_used(lens, sum(lens), max_blocks, groups) <= bound, (max_tokens, max_segments, lens)
