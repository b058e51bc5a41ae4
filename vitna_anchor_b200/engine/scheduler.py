"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes, finishes, frees.

Every step it plans one batch for the step function: first one token for each
running request whose prompt is done (decoding is never starved), then prompt
portions in admission order with what is left of the budget, a prompt cut
wherever the budget or the free pages end; then it admits waiting requests
while a slot and pages for a first portion are free.  It only decides; the
engine runs the plan and reports the sampled tokens back.

Refused at once, never cut short: an empty prompt, and a request whose prompt
plus max_new does not fit the context or the whole pool (the reference refuses
`prompt + max_new > ctx`, engine/src/api.c:2257-2282).

When pages run out: a decoded token that cannot get a page preempts the most
recently admitted running request (possibly itself): its pages and slot go
back, and it returns to the FRONT of the queue with everything it has
generated kept; when it is admitted again its prompt and generated tokens are
recomputed as one prompt.  Logits do not depend on how work is cut, and a
request's random stream is its own, so preemption changes no output.  The
reference cannot run out (static slots, engine/src/api.c:2262-2282); its
order of service is the precedent: oldest first, decode rounds between prompt
pieces (engine/src/api.c:2185-2246).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Set

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams, SplitMix64

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


class RequestRefused(ValueError):
    pass


@dataclass
class Request:
    request_id: Hashable
    prompt: List[int]
    max_new: int = 64
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop_ids: Set[int] = field(default_factory=set)
    output: List[int] = field(default_factory=list)
    state: str = WAITING
    finish_reason: Optional[str] = None      # "length", "stop", "context", "error"
    num_computed: int = 0                    # tokens whose keys and values are cached
    preemptions: int = 0
    rng: Optional[SplitMix64] = None

    def __post_init__(self):
        if self.rng is None:
            self.rng = SplitMix64(self.sampling.seed)

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def last_token(self) -> int:
        return self.output[-1] if self.output else self.prompt[-1]

    def tokens_between(self, a: int, b: int) -> List[int]:
        """tokens[a:b] without building the whole list."""
        n = len(self.prompt)
        if b <= n:
            return self.prompt[a:b]
        if a >= n:
            return self.output[a - n:b - n]
        return self.prompt[a:] + self.output[:b - n]

    @property
    def remaining(self) -> int:
        """Tokens not yet run through the model."""
        return len(self.prompt) + len(self.output) - self.num_computed


PENDING = -1     # a token that has been sampled on the device and not yet read by the host


@dataclass
class Planned:
    request: Request
    tokens: List[int]          # the tokens this step runs for the request
    samples: bool              # the step reaches the request's last token: its logits are wanted
    start: int = 0             # index of tokens[0] among the request's tokens (prompt + output)

    def refresh(self) -> None:
        """Read the tokens again (a token that was pending when the plan was made has arrived)."""
        self.tokens = self.request.tokens_between(self.start, self.start + len(self.tokens))


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_batch_tokens: int, max_model_len: int, max_prompt_portion: int = 0):
        self.cache = cache
        self.max_batch_tokens = max_batch_tokens
        self.max_model_len = max_model_len
        self.max_prompt_portion = max_prompt_portion or max_batch_tokens
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []        # in admission order
        self.finished: List[Request] = []
        self.preempted_total = 0

    # -- admission ----------------------------------------------------------------------------
    def add(self, req: Request) -> None:
        if not req.prompt:
            raise RequestRefused("the prompt is empty")
        if req.max_new < 1:
            raise RequestRefused("max_new must be at least 1")
        total = len(req.prompt) + req.max_new
        if total > self.max_model_len:
            raise RequestRefused(f"the prompt ({len(req.prompt)} tokens) and max_new ({req.max_new}) do not fit the "
                                 f"context of {self.max_model_len} positions")
        if total - 1 > self.cache.token_capacity():
            raise RequestRefused(f"the request needs {total - 1} cached positions and the whole pool holds "
                                 f"{self.cache.token_capacity()}")
        req.sampling.validate()
        req.state = WAITING
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -- planning -----------------------------------------------------------------------------
    def _pages_for(self, req: Request, n: int) -> List[int]:
        return self.cache.tables.pages_needed(req.request_id, n)

    def _fits(self, need: Sequence[int], free: Sequence[int]) -> bool:
        return all(k <= f for k, f in zip(need, free))

    def _preempt(self, req: Request) -> None:
        self.cache.close(req.request_id)
        self.running.remove(req)
        req.state = WAITING
        req.num_computed = 0
        req.preemptions += 1
        self.preempted_total += 1
        self.waiting.appendleft(req)

    def schedule(self) -> List[Planned]:
        """The next batch.  Pages are only counted here; the step function reserves them."""
        plan: List[Planned] = []
        budget = self.max_batch_tokens
        preempted_before = self.preempted_total

        # 1. one token for each running request whose prompt is done
        while True:
            free = list(self.cache.free_pages())
            decodes, ok = [], True
            for req in self.running:
                if req.remaining != 1:
                    continue
                need = self._pages_for(req, 1)
                if not self._fits(need, free) or budget - len(decodes) < 1:
                    ok = False
                    break
                free = [f - k for f, k in zip(free, need)]
                decodes.append(req)
            if ok:
                break
            if budget - len(decodes) < 1:      # the budget, not the pages, ended the list: the rest wait a step
                break
            self._preempt(self.running[-1])    # most recently admitted; may be the one that lacked the page
        for req in decodes:
            plan.append(Planned(req, [req.last_token], True, len(req.prompt) + len(req.output) - 1))
        budget -= len(decodes)
        planned_ids = {p.request.request_id for p in plan}

        # 2. prompt portions of running requests, oldest first
        for req in self.running:
            if budget < 1:
                break
            if req.request_id in planned_ids or req.remaining < 2:
                continue
            n = self._largest_portion(req, min(req.remaining, budget, self.max_prompt_portion), free)
            if n < 1:
                continue
            need = self._pages_for(req, n)
            free = [f - k for f, k in zip(free, need)]
            toks = req.tokens_between(req.num_computed, req.num_computed + n)
            plan.append(Planned(req, toks, n == req.remaining, req.num_computed))
            budget -= n

        # 3. admit waiting requests, oldest first, while a slot and pages for a first portion are free
        # (not in a step that had to preempt: what was just taken away is not handed out again at once)
        while (self.waiting and budget >= 1 and self.cache.tables.slots.free_slots > 0
               and (self.preempted_total == preempted_before or not self.running)):
            req = self.waiting[0]
            self.cache.open(req.request_id)
            n = self._largest_portion(req, min(req.remaining, budget, self.max_prompt_portion), free)
            if n < 1:
                self.cache.close(req.request_id)
                break
            self.waiting.popleft()
            req.state = RUNNING
            self.running.append(req)
            need = self._pages_for(req, n)
            free = [f - k for f, k in zip(free, need)]
            toks = req.tokens_between(req.num_computed, req.num_computed + n)
            plan.append(Planned(req, toks, n == req.remaining, req.num_computed))
            budget -= n
        if not plan and self.has_work():
            # nothing fits although requests exist: only possible when running requests hold every page
            # and none of them decodes; give the oldest room by preempting the newest
            if len(self.running) > 1:
                self._preempt(self.running[-1])
                return self.schedule()
            raise RuntimeError("the scheduler cannot place any token; the pool is too small for the oldest request")
        return plan

    def _largest_portion(self, req: Request, want: int, free: Sequence[int]) -> int:
        """The most tokens up to `want` whose pages are free (0 if not even one)."""
        if want < 1:
            return 0
        if self._fits(self._pages_for(req, want), free):
            return want
        ps = self.cache.page_size
        rc = self.cache.tables.get(req.request_id)
        best = want
        for g, f in enumerate(free):
            have = len(rc.tables[g].blocks)
            best = min(best, (have + f) * ps - rc.length)
        return max(0, best)

    # -- results ------------------------------------------------------------------------------
    def update(self, plan: Sequence[Planned], sampled: Sequence[int]) -> List[Request]:
        """The step ran.  `sampled` has one token for each planned entry with samples=True, in order.
        Returns the requests that finished; their pages and slots are already free."""
        done: List[Request] = []
        it = iter(sampled)
        for p in plan:
            req = p.request
            req.num_computed += len(p.tokens)
            if not p.samples:
                continue
            tok = int(next(it))
            req.output.append(tok)
            if tok in req.stop_ids:
                req.finish_reason = "stop"
            elif len(req.output) >= req.max_new:
                req.finish_reason = "length"
            elif len(req.prompt) + len(req.output) > self.max_model_len:
                req.finish_reason = "context"
            if req.finish_reason:
                done.append(req)
        for req in done:
            self._finish(req)
        return done

    def fail(self, req: Request, reason: str = "error") -> None:
        """End a request whose step failed; what it generated so far is kept (cf. engine/src/api.c:1777-1782)."""
        req.finish_reason = reason
        self._finish(req)

    def _finish(self, req: Request) -> None:
        if self.cache.is_open(req.request_id):
            self.cache.close(req.request_id)
        if req in self.running:
            self.running.remove(req)
        req.state = FINISHED
        self.finished.append(req)
