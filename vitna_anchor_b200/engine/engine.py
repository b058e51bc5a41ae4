"""The Python entry point: a model folder in, generated token ids out.

Options carry the names and meanings of the reference's command line
(engine/src/main.c:211-303): model, ctx (positions the cache holds per
request, default min(model maximum, 4096), engine/src/model.c:377-378),
parallel (requests at once), max_new (default 64), temperature / top_k /
top_p / seed (greedy when temperature is 0, the default), logits_out.
Ours in addition: dtype, kv_block, num_pages, max_batch_tokens.
"""
from __future__ import annotations

import time
from typing import Dict, Hashable, Iterable, List, Optional, Sequence, Union

import numpy as np
import torch

from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .loading import load_model
from .runner import ModelRunner, StepEntry, StepFailed
from .scheduler import Planned, Request, RequestRefused, Scheduler  # noqa: F401


class Engine:
    def __init__(self, model: str, *, dtype: str = "bfloat16", ctx: Optional[int] = None, parallel: int = 8,
                 kv_block: int = 16, num_pages: Optional[int] = None, max_batch_tokens: int = 2048,
                 device: str = "cuda", cuda_graphs: bool = True):
        if str(device) not in ("cuda", "cuda:0"):
            raise ValueError(f"--device is cuda; this engine has no path for {device}")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is usable, and the engine has no CPU path")
        if not (1 <= parallel <= 64):
            raise ValueError("--parallel is between 1 and 64")        # engine/src/main.c:30
        self.model = load_model(model, dtype, "cuda")
        max_pos = self.model.max_positions
        self.ctx = min(ctx or min(max_pos, 4096), max_pos)
        self.runner = ModelRunner(self.model, page_size=kv_block, num_pages=num_pages, max_requests=parallel,
                                  max_batch_tokens=max_batch_tokens, max_model_len=self.ctx, device="cuda",
                                  cuda_graphs=cuda_graphs)
        self.scheduler = Scheduler(self.runner.cache, max_batch_tokens=max_batch_tokens, max_model_len=self.ctx)
        self.sampler = Sampler(self.model.vocab_size, parallel, "cuda")
        self._next_id = 0
        self.last_timing: Dict[str, float] = {}

    # -- requests -----------------------------------------------------------------------------
    def add_request(self, ids: Sequence[int], *, max_new: int = 64, temperature: float = 0.0, top_k: int = 0,
                    top_p: float = 1.0, seed: int = 0, stop_ids: Iterable[int] = (), request_id: Optional[Hashable] = None) -> Request:
        ids = [int(t) for t in ids]
        for t in ids:
            if not (0 <= t < self.model.vocab_size):
                raise RequestRefused(f"token id {t} is outside the vocabulary of {self.model.vocab_size}")
        if request_id is None:
            request_id = self._next_id
            self._next_id += 1
        req = Request(request_id, ids, max_new, SamplingParams(float(temperature), int(top_k), float(top_p), int(seed)),
                      set(int(s) for s in stop_ids))
        self.scheduler.add(req)
        return req

    def step(self, logits_sink=None) -> List[Request]:
        """Plan one batch, run it, sample, and hand the tokens back to the scheduler.  Returns finished requests."""
        plan = self.scheduler.schedule()
        entries = [StepEntry(p.request.request_id, p.tokens, [len(p.tokens) - 1] if p.samples else []) for p in plan]
        try:
            logits = self.runner.step(entries)
        except StepFailed:
            # the step computed nothing: its requests end with an error and keep what they had
            failed = [p.request for p in plan]
            for req in failed:
                self.scheduler.fail(req)
            return failed
        sampling = [p.request for p in plan if p.samples]
        tokens: List[int] = []
        if sampling:
            if logits_sink is not None:
                logits_sink(sampling, logits)
            tokens = self.sampler.sample(logits, [r.sampling for r in sampling], [r.rng for r in sampling])
        return self.scheduler.update(plan, tokens)

    def run(self, logits_sink=None) -> List[Request]:
        done: List[Request] = []
        while self.scheduler.has_work():
            done += self.step(logits_sink)
        return done

    # -- the one call most users make -------------------------------------------------------------
    def generate(self, ids: Union[Sequence[int], Sequence[Sequence[int]]], *, max_new: int = 64, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, seed: int = 0, stop_ids: Iterable[int] = (),
                 logits_out: Optional[str] = None) -> Union[List[int], List[List[int]]]:
        """New token ids for one prompt (a list of ids) or several (a list of lists; each gets seed + its index).
        logits_out: a file that receives each step's logits row of the FIRST prompt, float32, steps x vocab
        (engine/src/main.c:942-947)."""
        single = len(ids) > 0 and not isinstance(ids[0], (list, tuple))
        prompts = [ids] if single else list(ids)
        reqs = [self.add_request(p, max_new=max_new, temperature=temperature, top_k=top_k, top_p=top_p, seed=seed + i,
                                 stop_ids=stop_ids) for i, p in enumerate(prompts)]
        sink, out_file = None, None
        if logits_out:
            out_file = open(logits_out, "wb")
            first = reqs[0]

            def sink(sampling, logits):
                for r, req in enumerate(sampling):
                    if req is first:
                        out_file.write(np.ascontiguousarray(logits[r].cpu().numpy(), dtype="<f4").tobytes())
        t0 = time.perf_counter()
        t_first = None
        try:
            while self.scheduler.has_work():
                self.step(sink)
                if t_first is None and all(r.output for r in reqs):
                    torch.cuda.synchronize()
                    t_first = time.perf_counter()
        finally:
            if out_file:
                out_file.close()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        n_after = sum(max(0, len(r.output) - 1) for r in reqs)
        self.last_timing = {"prompt_tokens": sum(len(p) for p in prompts), "prompt_ms": ((t_first or t1) - t0) * 1e3,
                            "tokens_after_first": n_after, "decode_ms": (t1 - (t_first or t1)) * 1e3}
        for r in reqs:
            if r.finish_reason == "error":
                raise StepFailed(f"a step of request {r.request_id!r} failed after {len(r.output)} new tokens")
        outs = [list(r.output) for r in reqs]
        return outs[0] if single else outs

    def logits(self, ids: Sequence[int], piece: int = 256) -> torch.Tensor:
        """float32 logits [positions, vocab] of every position of one prompt, run in pieces of `piece` tokens
        (the reference's `logits` command, engine/src/main.c:900-937)."""
        rid = ("logits", self._next_id)
        self._next_id += 1
        self.runner.open(rid)
        rows = []
        try:
            for p in range(0, len(ids), piece):
                chunk = [int(t) for t in ids[p:p + piece]]
                rows.append(self.runner.step([StepEntry(rid, chunk, range(len(chunk)))]).clone())
        finally:
            self.runner.close(rid)
        return torch.cat(rows, dim=0)
