"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step takes any mixture of prompt portions and single decoded tokens, cut
anywhere, runs exactly the tokens it is given as one batch, and returns
float32 logits at the places asked for.  Before anything is launched it
checks the tokens and the room, and holds pages for the new positions; if the
pools cannot give them it raises OutOfPages and nothing has changed.  A
request's length advances only when the step has been issued in full.

A step is issued, not waited for.  Kernels with bounded waits (the tcgen05 ones) report a wait that ran out
through a word the host can read; `check()` (after the caller's synchronisation, or with sync=True) and the
start of every later step read it.  When it is set, every step issued since the last clean check is undone
(lengths, pages, fixed-size states) and DeviceStepFailed names the requests: their logits were not valid.  The
reference checks every device call and turns a failure into a failed step whose position does not advance
(engine/src/model_cuda.cu:3537-3548, engine/src/model.c:868-883, engine/include/model.h:212-213).

The reference has three calls for a step (one token, engine/src/model.c:866;
a run of one sequence's tokens, model.c:982-1040; one token of each of
several sequences, model.c:1149-1172) and never mixes a prompt piece with
decode rows in one pass (engine/src/api.c:2216-2225).  Here they are one call.
"""
from __future__ import annotations

import os
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..cache.manager import CacheManager
from ..cache.pages import CacheError, OutOfPages  # noqa: F401
from ..models.decoder import DecoderModel
from ..parts.base import Workspace
from .context import ContextBuilder, MetaOverflow


class StepError(RuntimeError):
    """The step was refused before anything ran (bad token, no room, unknown request)."""


class StepFailed(RuntimeError):
    """The step failed; nothing of it is kept (cf. vitna_llama_fail_step_once, engine/src/model.c:471-493)."""


class DeviceStepFailed(StepFailed):
    """A kernel gave up a bounded wait.  `request_ids`: the requests of every step issued since the last clean
    check; they are back at the lengths they had before those steps (or closed, when that was not possible)."""

    def __init__(self, message: str, request_ids: Sequence[Hashable]):
        super().__init__(message)
        self.request_ids = list(request_ids)


@dataclass
class StepEntry:
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()      # places among `tokens` whose logits are returned


@dataclass
class _Issued:
    """A step whose kernels may still be running."""
    before: List[Tuple[Hashable, int]]     # (request, its length before the step)
    states: object                         # what CacheManager.save_states returned, or None
    event: torch.cuda.Event


GRAPH_LOGIT_ROWS = 64      # steps with up to this many wanted rows may run from a captured graph


class ModelRunner:
    def __init__(self, model: DecoderModel, *, page_size: int = 16, num_pages: Optional[int] = None,
                 max_requests: int = 64, max_batch_tokens: int = 2048, max_model_len: Optional[int] = None,
                 device="cuda", cache_tokens: Optional[int] = None, cuda_graphs: bool = True):
        self.model = model
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise StepError("the engine runs on a CUDA device only; there is no CPU path")
        self.max_model_len = min(max_model_len or model.max_positions, model.max_positions)
        self.max_batch_tokens = max_batch_tokens
        self.page_size = page_size
        if num_pages is None:
            tokens = cache_tokens if cache_tokens is not None else self.max_model_len * max_requests
            num_pages = -(-tokens // page_size)
        self.cache = CacheManager(model.cache_specs(), page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                                  dtype=model.dtype, device=self.device)
        self.max_blocks = -(-self.max_model_len // page_size)
        self.workspace = Workspace(self.device, max_batch_tokens, max_requests, self.max_model_len)
        self.max_segments = max_requests
        self.builder = ContextBuilder(self.cache, model.dtype, self.workspace, max_batch_tokens=max_batch_tokens,
                                      max_segments=max_requests, max_model_len=self.max_model_len, device=self.device)
        self._meta_dev = self.builder.meta_dev
        self._fail_at: Optional[int] = None
        self._fail_after_run: Optional[int] = None
        env = os.environ.get("VITNA_TEST_FAIL_STEP")
        if env is not None:
            self._fail_at = int(env) if env.strip() else 0
        self.steps_run = 0
        # A model is run from captured graphs only if every part of it says that a capture replays it faithfully.
        self.cuda_graphs = bool(cuda_graphs) and model.capture_safe
        self._decode_graphs: "OrderedDict[tuple, tuple]" = OrderedDict()    # (batch bucket, context bucket) -> (graph, kernels)
        self._mixed_graphs: Dict[tuple, tuple] = {}                          # the counts of a mixed step -> (graph, logits, kernels)
        self._seen_shapes: Dict[tuple, int] = {}
        self.graph_mixed_steps = True            # steps with prompt portions are captured too, once their counts repeat
        self.max_decode_graphs = 32              # least recently used goes first
        self.max_mixed_graphs = 48
        self._graph_logits: Optional[torch.Tensor] = None      # [GRAPH_LOGIT_ROWS, vocab]: where every graph leaves its logits
        self._src_dev = None
        self._src_host = None
        self.graph_replays = 0
        self._issued: List[_Issued] = []

    # -- requests ---------------------------------------------------------------------------
    def open(self, request_id: Hashable) -> int:
        return self.cache.open(request_id)

    def close(self, request_id: Hashable) -> None:
        self.cache.close(request_id)

    def length(self, request_id: Hashable) -> int:
        return self.cache.length(request_id)

    def fail_step_once(self, position: int = 0) -> None:
        """The next step that would compute `position` of any request raises StepFailed instead."""
        self._fail_at = position

    def fail_after_run_once(self, run: int) -> None:
        """For tests: the next step raises StepFailed on the host after run `run` of the model's schedule has been
        issued (its kernels may have written caches and states; the step must leave no trace of that)."""
        self._fail_after_run = run

    def decode_graph_takes(self, entries: Sequence[StepEntry]) -> bool:
        """Whether the batch is single tokens, each wanted: the decode graph's case."""
        return (self.cuda_graphs and len(entries) <= GRAPH_LOGIT_ROWS
                and all(len(e.tokens) == 1 and len(e.want) == 1 for e in entries))

    # -- device errors ------------------------------------------------------------------------
    def check(self, sync: bool = True) -> None:
        """Whether a kernel of the steps issued so far gave up a wait.  sync=True waits for them first (call it with
        sync=False right after a synchronisation of your own).  Clean: returns.  Otherwise every step issued
        since the last clean check is undone and DeviceStepFailed is raised."""
        if sync:
            torch.cuda.current_stream(self.device).synchronize()
        code = ops.device_error_code()
        if code == 0:
            if sync:
                self._issued.clear()
            else:
                while self._issued and self._issued[0].event.query():
                    if ops.device_error_code() != 0:       # set between the two reads: handled below
                        return self.check(sync=True)
                    self._issued.pop(0)
            return
        if not sync:
            torch.cuda.current_stream(self.device).synchronize()
        try:
            ops.check_device_errors()                       # clears the word
        except ops.KernelGaveUp as e:
            message = str(e)
        undone = self._undo_issued()
        raise DeviceStepFailed(f"{message}; {len(undone)} request(s) were put back to where they were before", undone)

    def _undo_issued(self) -> List[Hashable]:
        """Put every request of the issued steps back to its length before the oldest of them."""
        first_len: Dict[Hashable, int] = {}
        for item in self._issued:
            for rid, n in item.before:
                first_len.setdefault(rid, n)
        for item in reversed(self._issued):                 # the oldest snapshot of a slot is restored last
            if item.states is not None:
                self.cache.restore_states(item.states)
        self._issued.clear()
        for rid, n in first_len.items():
            if not self.cache.is_open(rid):
                continue
            try:
                if self.cache.length(rid) > n:
                    self.cache.rewind(rid, n)
            except CacheError:
                self.cache.close(rid)                       # a window has given pages back: nothing to return to
        return list(first_len)

    # -- the step ---------------------------------------------------------------------------
    def _validate(self, entries: Sequence[StepEntry]) -> Tuple[int, int]:
        if not entries:
            raise StepError("a step needs at least one entry")
        if len(entries) > self.max_segments:
            raise StepError(f"{len(entries)} entries in a step; the limit is {self.max_segments}")
        seen = set()
        T = R = 0
        V = self.model.vocab_size
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} is in the step twice")
            seen.add(e.request_id)
            if not self.cache.is_open(e.request_id):
                raise StepError(f"request {e.request_id!r} is not open")
            n = len(e.tokens)
            if n < 1:
                raise StepError(f"request {e.request_id!r} brings no token")
            for t in e.tokens:
                if not (0 <= int(t) < V):
                    raise StepError(f"token {t} of request {e.request_id!r} is outside the vocabulary of {V}")
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise StepError(f"request {e.request_id!r} wants place {w} of {n} tokens")
            if self.cache.length(e.request_id) + n > self.max_model_len:
                raise StepError(f"request {e.request_id!r} would pass the context of {self.max_model_len} positions")
            T += n
            R += len(e.want)
        if T > self.max_batch_tokens:
            raise StepError(f"{T} tokens in a step; the limit is {self.max_batch_tokens}")
        return T, R

    def step(self, entries: Sequence[StepEntry], token_source: Optional[Tuple[torch.Tensor, Sequence[int]]] = None) -> Optional[torch.Tensor]:
        """Run the batch.  Returns float32 logits [wanted places, vocab] on the device, in the order of the
        entries and of each entry's `want`, or None when nothing is wanted.

        The result is valid until the next step() of this runner: steps that are replayed from a captured graph
        all leave their logits in the same buffer.  Copy what is to be kept (Engine.logits does).

        token_source = (ids, src): only for a batch of single tokens that goes through the decode graph; entry i
        with src[i] >= 0 takes its token from the device tensor ids[src[i]] (what an earlier step's sampling left
        there) instead of from entries[i].tokens, so the host need not wait for that step."""
        self.check(sync=False)                # a wait that ran out in an earlier step ends here, before anything new is issued
        T, R = self._validate(entries)
        plan = [(e.request_id, len(e.tokens)) for e in entries]
        if self._fail_at is not None:
            for e in entries:
                lo = self.cache.length(e.request_id)
                if lo <= self._fail_at < lo + len(e.tokens):
                    self._fail_at = None
                    raise StepFailed(f"the step that computes position {lo} failed as the test asked")
        before = [(e.request_id, self.cache.length(e.request_id)) for e in entries]
        self.cache.reserve_step(plan)         # OutOfPages leaves everything as it was
        states = None
        try:
            states = self.cache.save_states([e.request_id for e in entries])
            if self._fail_after_run is not None:
                logits = self._eager_step(entries)
            elif self.decode_graph_takes(entries):
                logits = self._decode_step(entries, token_source)
            elif token_source is not None:
                raise StepError("tokens can be taken from the device only by a batch of single tokens")
            elif self.cuda_graphs and self.graph_mixed_steps and R <= GRAPH_LOGIT_ROWS:
                logits = self._graphed_step(entries, T, R)
            else:
                logits = self._eager_step(entries)
        except BaseException as exc:
            self.cache.rollback_step(plan)
            if states is not None:
                self.cache.restore_states(states)
            if isinstance(exc, MetaOverflow):
                raise StepError(str(exc)) from None
            raise
        self.cache.commit_step(plan)
        self.steps_run += 1
        event = torch.cuda.Event()
        event.record()
        self._issued.append(_Issued(before, states, event))
        return logits

    def _eager_step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        ctx, rows = self.builder.build([(e.request_id, e.tokens, e.want) for e in entries])
        if self._fail_after_run is not None:
            fail_at, self._fail_after_run = self._fail_after_run, None

            def after_run(i: int) -> None:
                if i == fail_at:
                    raise StepFailed(f"the step failed after run {i} of the schedule as the test asked")
            ctx.after_run = after_run
        return self.model.forward(ctx, rows)

    # -- replaying captured graphs ----------------------------------------------------------------
    def _logits_buffer(self) -> torch.Tensor:
        if self._graph_logits is None:
            self._graph_logits = torch.empty((GRAPH_LOGIT_ROWS, self.model.vocab_size), dtype=torch.float32, device=self.device)
        return self._graph_logits

    def _capture(self, ctx, rows, n_rows: int):
        """Capture the step's launches (the step has just run eagerly, so every workspace buffer exists)."""
        out = self._logits_buffer()[:n_rows] if n_rows else None
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with torch.cuda.graph(graph):
            self.model.forward(ctx, rows, out=out)
        kernels = ops.launch_count() - before
        ops.add_launches(-kernels)            # capture does not run the kernels
        return graph, kernels

    @staticmethod
    def context_bucket(longest: int, limit: int) -> int:
        """The bound on positions a decode graph is captured for: steps of 512 up to 4,096, of 1,024 up to 8,192,
        of 2,048 beyond, so that a long context does not mean hundreds of graphs."""
        step = 512 if longest <= 4096 else 1024 if longest <= 8192 else 2048
        return min(limit, -(-longest // step) * step)

    def _decode_step(self, entries: Sequence[StepEntry], token_source=None) -> torch.Tensor:
        S = len(entries)
        B = 1
        while B < S:
            B *= 2
        B = min(B, self.max_segments, GRAPH_LOGIT_ROWS)
        # the longest context, rounded up, bounds the grid of the decode attention: a graph per batch bucket and
        # context bucket, so that a short context does not launch the blocks of a long one.  The first batch of a
        # bucket runs eagerly and is then captured (a stall of about two steps, once per bucket).
        longest = max(self.cache.tables.get(e.request_id).length for e in entries) + 1
        reach = self.context_bucket(longest, self.max_model_len)
        key = (B, reach)
        held = self._decode_graphs.get(key)
        ctx, rows = self.builder.build_decode([e.request_id for e in entries], [e.tokens[0] for e in entries], B,
                                              views=held is None, reach=reach)
        if token_source is not None:
            ids, src = token_source
            if self._src_dev is None:
                self._src_dev = torch.empty(self.max_segments, dtype=torch.int32, device=self.device)
                self._src_host = [torch.empty(self.max_segments, dtype=torch.int32).pin_memory() for _ in range(4)]
            host = self._src_host[self.builder.turn]
            host[:B] = -1
            host[:S] = torch.as_tensor(list(src), dtype=torch.int32)
            self._src_dev[:B].copy_(host[:B], non_blocking=True)
            ops.take_tokens(self._meta_dev[:B], ids, self._src_dev[:B])      # the tokens are the first B words of the metadata
        out = self._logits_buffer()[:B]
        if held is None:
            self.model.forward(ctx, rows, out=out)
            graph, kernels = self._capture(ctx, rows, B)
            self._decode_graphs[key] = (graph, kernels)
            while len(self._decode_graphs) > self.max_decode_graphs:
                self._decode_graphs.popitem(last=False)
            return out[:S]
        self._decode_graphs.move_to_end(key)
        graph, kernels = held
        graph.replay()
        ops.add_launches(kernels)
        self.graph_replays += 1
        return out[:S]

    def _graphed_step(self, entries: Sequence[StepEntry], T: int, R: int) -> Optional[torch.Tensor]:
        """A step with prompt portions.  Issuing its few hundred launches from the host takes longer than the GPU
        needs for them, so once the same counts come a second time the step's launches are captured and from then
        on replayed.  Everything that differs between two such steps (tokens, positions, slots, block tables, which
        rows are wanted) is in the metadata buffer, at places that depend on the counts alone; a part that reads
        anything else of a batch must say so (Part.capture_safe)."""
        lens = [len(e.tokens) for e in entries]
        n_dec = sum(1 for n in lens if n == 1)
        n_tiles = sum(-(-n // 64) for n in lens if n > 1)
        n_big = sum(-(-n // 128) for n in lens if n > 1)
        key = ("mixed", T, len(entries), R, n_dec, n_tiles, n_big)
        ctx, rows = self.builder.build([(e.request_id, e.tokens, e.want) for e in entries], fixed_blocks=self.max_blocks,
                                       for_graph=True)
        out = self._logits_buffer()[:R] if R else None
        held = self._mixed_graphs.get(key)
        if held is not None:
            graph, kernels = held
            graph.replay()
            ops.add_launches(kernels)
            self.graph_replays += 1
            return out
        logits = self.model.forward(ctx, rows, out=out)
        seen = self._seen_shapes.get(key, 0) + 1
        self._seen_shapes[key] = seen
        if seen >= 2 and len(self._mixed_graphs) < self.max_mixed_graphs:
            self._mixed_graphs[key] = self._capture(ctx, rows, R)
        return logits
