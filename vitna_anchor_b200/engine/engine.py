"""The Python entry point: a model folder in, generated token ids out.

Options carry the names and meanings of the reference's command line
(engine/src/main.c:211-303): model, ctx (positions the cache holds per
request, default min(model maximum, 4096), engine/src/model.c:377-378),
parallel (requests at once), max_new (default 64), temperature / top_k /
top_p / seed (greedy when temperature is 0, the default), logits_out.
Ours in addition: dtype, kv_block, num_pages, max_batch_tokens, max_prompt_portion (the most prompt tokens of
one request in a step; the reference runs a prompt in pieces of 512 between decode rounds when others are decoding,
engine/src/api.c:48-49, 2216-2224).
"""
from __future__ import annotations

import time
from typing import Dict, Hashable, Iterable, List, Optional, Sequence, Union

import numpy as np
import torch

from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .loading import load_model
from .runner import DeviceStepFailed, ModelRunner, StepEntry, StepFailed
from .scheduler import PENDING, Planned, Request, RequestRefused, Scheduler  # noqa: F401


class Engine:
    def __init__(self, model, *, dtype: str = "bfloat16", ctx: Optional[int] = None, parallel: int = 8,
                 kv_block: int = 16, num_pages: Optional[int] = None, max_batch_tokens: int = 2048,
                 max_prompt_portion: int = 0, device: str = "cuda", cuda_graphs: bool = True, pipeline: bool = True):
        if str(device) not in ("cuda", "cuda:0"):
            raise ValueError(f"--device is cuda; this engine has no path for {device}")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is usable, and the engine has no CPU path")
        if not (1 <= parallel <= 64):
            raise ValueError("--parallel is between 1 and 64")        # engine/src/main.c:30
        # a folder with config.json and model.safetensors, or a model that is already built on the device
        self.model = load_model(model, dtype, "cuda") if isinstance(model, (str, bytes)) or hasattr(model, "__fspath__") else model
        max_pos = self.model.max_positions
        self.ctx = min(ctx or min(max_pos, 4096), max_pos)
        self.runner = ModelRunner(self.model, page_size=kv_block, num_pages=num_pages, max_requests=parallel,
                                  max_batch_tokens=max_batch_tokens, max_model_len=self.ctx, device="cuda",
                                  cuda_graphs=cuda_graphs)
        if max_prompt_portion < 0:
            raise ValueError("--max-prompt-portion is 0 (no limit below the step's token budget) or a number of tokens")
        self.scheduler = Scheduler(self.runner.cache, max_batch_tokens=max_batch_tokens, max_model_len=self.ctx,
                                   max_prompt_portion=max_prompt_portion)
        self.sampler = Sampler(self.model.vocab_size, parallel, "cuda")
        self._next_id = 0
        self.last_timing: Dict[str, float] = {}
        # Decoding one step ahead of the host: the ids a step samples stay on the device and become the next step's
        # tokens there, while the host reads them a step later (see step()).
        self.pipeline = pipeline and self.runner.cuda_graphs
        self._inflight = None            # (requests, index of the pending token in each request's output, host ids, event)
        self._ids_host = [torch.empty(parallel, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._ids_turn = 0
        self._held: List[Request] = []   # finished, but their last token has not arrived yet

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
        """Plan one batch, run it, sample, and hand the tokens back to the scheduler.  Returns finished requests.

        While the batches are single decoded tokens of requests without stop ids, the host does not wait for a step's
        ids before it issues the next step: the next step takes its tokens from the sampler's device buffer
        (ModelRunner.step's token_source), the host's copy of the ids arrives a step later, and until then the
        request's output holds PENDING in that place.  A request is returned as finished only when its tokens are
        all there.  Anything else (a prompt portion in the batch, stop ids, a logits sink) first waits for what is
        pending, so the results are the same as without the overlap."""
        plan = self.scheduler.schedule()
        sampling = [p.request for p in plan if p.samples]
        pending_now = self._inflight is not None
        entries = [StepEntry(p.request.request_id, p.tokens, [len(p.tokens) - 1] if p.samples else []) for p in plan]
        can_feed = (self.pipeline and logits_sink is None and self.runner.decode_graph_takes(entries)
                    and all(not r.stop_ids for r in sampling))
        token_source = None
        if pending_now:
            if can_feed:
                reqs, _, _, _ = self._inflight
                where = {id(r): i for i, r in enumerate(reqs)}
                src = [where.get(id(p.request), -1) if p.tokens[0] == PENDING else -1 for p in plan]
                for e in entries:
                    if e.tokens[0] == PENDING:
                        e.tokens = [0]           # replaced on the device
                token_source = (self.sampler.last_ids(), src)
            else:
                try:
                    self._resolve()
                except DeviceStepFailed as e:
                    return self._device_failure(e)
                for p, e in zip(plan, entries):
                    p.refresh()
                    e.tokens = p.tokens
        try:
            logits = self.runner.step(entries, token_source)
            if token_source is not None:
                self._resolve()                  # the step before: its ids have been on their way for a whole step
            tokens: List[int] = []
            if sampling:
                if logits_sink is not None:
                    logits_sink(sampling, logits)
                if can_feed:
                    ids = self.sampler.sample_async(logits, [r.sampling for r in sampling], [r.rng for r in sampling])
                    host = self._ids_host[self._ids_turn]
                    self._ids_turn ^= 1
                    host[:len(sampling)].copy_(ids, non_blocking=True)
                    event = torch.cuda.Event()
                    event.record()
                    done = self.scheduler.update(plan, [PENDING] * len(sampling))
                    self._inflight = (sampling, [len(r.output) - 1 for r in sampling], host, event)
                    self._held += done
                    return self._release()
                tokens = self.sampler.sample(logits, [r.sampling for r in sampling], [r.rng for r in sampling])
                self.runner.check(sync=False)    # the ids have arrived, so every kernel of the step is done
        except DeviceStepFailed as e:
            return self._device_failure(e, plan)
        except StepFailed:
            # the step computed nothing: its requests end with an error and keep what they had
            failed = [p.request for p in plan]
            try:
                self._resolve()
            except DeviceStepFailed as e:
                return self._device_failure(e, plan)
            for req in failed:
                self.scheduler.fail(req)
            return failed + self._release()
        return self.scheduler.update(plan, tokens) + self._release()

    def _device_failure(self, e: DeviceStepFailed, plan=()) -> List[Request]:
        """A kernel gave up a wait: the requests of the steps that were in flight end with an error; a token that was still on its way is dropped, as the reference does not keep the
        token of a failed step (engine/src/api.c:1777-1782).  The other requests go on."""
        self._inflight = None
        hit = set(e.request_ids)
        failed = [r for r in list(self.scheduler.running) + self._held if r.request_id in hit]
        self._held = [r for r in self._held if r.request_id not in hit]
        for req in failed:
            while req.output and req.output[-1] == PENDING:
                req.output.pop()
            if req.state != "finished":
                self.scheduler.fail(req)
            else:
                req.finish_reason = "error"
        return failed + self._release()

    def _resolve(self) -> None:
        """Wait for the ids of the step in flight and put them where PENDING stands."""
        if self._inflight is None:
            return
        reqs, places, host, event = self._inflight
        event.synchronize()
        self.runner.check(sync=False)            # raises DeviceStepFailed when a kernel of that step gave up
        self._inflight = None
        for r, place, tok in zip(reqs, places, host[:len(reqs)].tolist()):
            r.output[place] = int(tok)

    def _release(self) -> List[Request]:
        """Finished requests whose tokens are all known."""
        ready = [r for r in self._held if PENDING not in r.output[-1:]]
        self._held = [r for r in self._held if PENDING in r.output[-1:]]
        return ready

    def flush(self) -> List[Request]:
        """Wait for whatever is still on its way; returns the finished requests that were held back for it
        (and those that a kernel's failure ended)."""
        try:
            self._resolve()
            self.runner.check(sync=True)
        except DeviceStepFailed as e:
            return self._device_failure(e)
        return self._release()

    def run(self, logits_sink=None) -> List[Request]:
        done: List[Request] = []
        while self.scheduler.has_work():
            done += self.step(logits_sink)
        return done + self.flush()

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
                    self.flush()
                    torch.cuda.synchronize()
                    t_first = time.perf_counter()
        finally:
            if out_file:
                out_file.close()
        self.flush()
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
            self.runner.check(sync=True)         # no logits leave before every kernel is known to have finished its waits
        finally:
            if self.runner.cache.is_open(rid):
                self.runner.close(rid)
        return torch.cat(rows, dim=0)
