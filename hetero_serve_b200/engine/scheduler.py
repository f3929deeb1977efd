"""The continuous-batching scheduler above the step function.

In the manner of the reference's per-device worker (heteroserve/worker/worker.py):

* requests are admitted in arrival order; admission reserves pages for the whole
  prompt after a prefix match (worker.py:378-416, heteroserve/kv/blocks.py:168-201);
* prompts are cut into portions of at most ``max_prefill_tokens`` (worker.py:599-657);
* every running request decodes one token per step, at most ``max_batch`` of them
  (worker.py:586-589, 659-703);
* a request finishes after ``max_new_tokens``, at an end-of-sequence token if
  ``stop_at_eos`` (worker.py:714-715), or when it reaches the context limit; its full
  pages are published for reuse and everything it holds is given back (worker.py:721-764);
* when pages run out while decoding, the NEWEST running request is preempted by
  recomputation: its pages are given back, its tokens kept, and it is prefilled again
  later (worker.py:738-757).

Two policies compose a step.  ``prefill_first`` is the reference's: while any prompt is
unfinished, a step is one portion of the oldest such prompt; otherwise a step decodes
(worker.py:580-591).  ``mixed`` puts the decoded tokens of all running requests and, in
what is left of the token budget, portions of waiting prompts into the same step.

What happens when pages run out — decided here:

1. at admission: the request waits (and blocks those behind it, keeping arrival order)
   until pages for its whole prompt are obtainable; a prompt that could never fit the
   pool is refused when it is submitted;
2. while decoding: preempt the newest running request and try again; a request that
   preempts itself sits the step out.  A request that has outgrown the whole pool on its
   own (nothing else is live and it still cannot be admitted) ends with the tokens it
   has, ``finish_reason == "out_of_pages"``.  A preempted request goes to the FRONT of the
   waiting queue, keeps its sampled tokens, and is prefilled again over prompt + outputs
   (all but the last token, which decoding feeds).  Because the random draw of a token
   depends only on (seed, position), a preempted request continues exactly as it would
   have.

Pipelining (``pipeline=True``).  ``step_fn`` may return, instead of a list of tokens, an object
whose ``tokens_host()`` yields them later.  The scheduler then launches step i+1 BEFORE it reads
step i's tokens: a request whose latest token is still on its way decodes with
``FROM_DEVICE`` (the step reads the token from device memory), so the host's work and the
transfer hide behind the device's.  What needs the token itself waits for it: a request that
reaches ``max_new_tokens`` or the context limit with the token in flight sits the next step
out (its end is known by counting); an end-of-sequence token is seen one step late, and the
request's part in the step launched meanwhile is discarded (its pages were still its own when
that step was launched, and whoever gets them next is ordered behind it on the stream);
preemption first waits for the tokens in flight, since a preempted request is prefilled again
over all of its tokens.
"""

from __future__ import annotations

import itertools
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Hashable, Sequence

from ..cache import CacheManager, OutOfPages
from .step import FROM_DEVICE, StepEntry


class SeqState:                     # heteroserve/worker/protocol.py:38-42
    WAITING = "waiting"             # queued; nothing resident
    PREFILL = "prefill"             # admitted; prompt partly resident
    RUNNING = "running"             # generating
    DONE = "done"


class RequestRefused(ValueError):
    """A request that can never run: empty, too long, or larger than the whole pool."""


_ids = itertools.count()


@dataclass
class Request:
    """What a caller submits (heteroserve/sched/router.py:36-44, worker.py:53-61)."""

    prompt_ids: Sequence[int]
    max_new_tokens: int = 32
    temperature: float = 0.0
    top_k: int = 0
    seed: int = 0
    stop_at_eos: bool = True
    req_id: Hashable = field(default_factory=lambda: f"req-{next(_ids)}")


@dataclass
class SequenceState:
    """A request inside the scheduler (heteroserve/worker/worker.py:53-87)."""

    request: Request
    output_ids: list[int] = field(default_factory=list)
    n_kv: int = 0                       # positions resident in the cache
    state: str = SeqState.WAITING
    admitted: bool = False
    cached_prefix_tokens: int = 0
    prefill_tokens_computed: int = 0
    preemptions: int = 0
    finish_reason: str = ""
    pending: int = 0                    # tokens sampled for it that the host has not read yet
    t_submit: float = 0.0
    t_admit: float = 0.0
    t_first_token: float = 0.0
    t_done: float = 0.0

    @property
    def req_id(self):
        return self.request.req_id

    @property
    def ctx(self) -> list[int]:
        return list(self.request.prompt_ids) + self.output_ids

    @property
    def prefill_target(self) -> int:
        """How far prefill must reach before decoding takes over (worker.py:79-83)."""
        n = len(self.request.prompt_ids) + len(self.output_ids)
        return n - 1 if self.output_ids else n


@dataclass
class Planned:
    """One entry of a planned step."""

    seq: SequenceState
    start: int
    tokens: list[int]
    samples: bool           # the last of these tokens yields a new token


@dataclass
class SchedulerStats:
    steps: int = 0
    prefill_steps: int = 0
    decode_steps: int = 0
    mixed_steps: int = 0
    tokens_generated: int = 0
    tokens_prefilled: int = 0
    tokens_saved_by_cache: int = 0
    preemptions: int = 0
    finished: int = 0


class Scheduler:
    """Decides what each step runs.  ``step_fn(entries)`` runs a batch through the step
    function with device sampling and returns one token per entry that wanted one, in entry
    order — as a list, or as an object whose ``tokens_host()`` returns that list when asked
    (see "Pipelining" above); the scheduler owns everything around it."""

    def __init__(self, manager: CacheManager, step_fn: Callable[[list[StepEntry]], object],
                 *, max_batch: int, max_prefill_tokens: int, max_ctx: int,
                 eos_token_id: int | None, policy: str = "prefill_first",
                 vocab_size: int | None = None, clock: Callable[[], float] = time.perf_counter,
                 pipeline: bool = False):
        if policy not in ("prefill_first", "mixed"):
            raise ValueError(f"unknown policy {policy!r}")
        self.manager = manager
        self.step_fn = step_fn
        self.max_batch = max_batch
        self.max_prefill_tokens = max_prefill_tokens
        self.max_ctx = max_ctx
        self.eos_token_id = eos_token_id
        self.policy = policy
        self.vocab_size = vocab_size
        self.clock = clock
        self.waiting: deque[SequenceState] = deque()
        self.active: list[SequenceState] = []          # admitted, in admission order
        self.finished: list[SequenceState] = []
        self.stats = SchedulerStats()
        self.pipeline = bool(pipeline)
        self._inflight: tuple[list[Planned], object] | None = None   # launched, tokens unread
        self._late_done: list[SequenceState] = []     # finished while a plan was being made

    # -- submission -----------------------------------------------------------
    def add(self, request: Request) -> SequenceState:
        n = len(request.prompt_ids)
        if n == 0:
            raise RequestRefused("the prompt is empty")
        if n >= self.max_ctx:
            raise RequestRefused(f"the prompt has {n} tokens; with one generated token it "
                                 f"would exceed the context limit of {self.max_ctx}")
        if request.max_new_tokens <= 0:
            raise RequestRefused("max_new_tokens must be positive")
        if self.vocab_size is not None:
            bad = [t for t in request.prompt_ids if not 0 <= t < self.vocab_size]
            if bad:
                raise RequestRefused(f"token id {bad[0]} is outside [0, {self.vocab_size})")
        for pool in self.manager.pools:
            if self.manager.pages_for(n + 1) > pool.num_pages:
                raise RequestRefused(
                    f"the prompt needs {self.manager.pages_for(n + 1)} pages, the pool has "
                    f"{pool.num_pages}")
        seq = SequenceState(request=request, t_submit=self.clock())
        self.waiting.append(seq)
        return seq

    def has_work(self) -> bool:
        return bool(self.waiting or self.active or self._inflight is not None)

    # -- admission --------------------------------------------------------------
    def _admit(self) -> None:
        """Admit from the front of the queue while a state slot and the pages of the whole
        prompt (after the prefix match) can be had.  The head blocks those behind it."""
        mgr = self.manager
        while self.waiting:
            seq = self.waiting[0]
            if mgr.free_slots() == 0:
                return
            ctx = seq.ctx
            target = seq.prefill_target
            opened = mgr.open(seq.req_id, ctx[:target] if target else None)
            try:
                mgr.reserve(seq.req_id, max(target, 1))
            except OutOfPages:
                mgr.close(seq.req_id)
                # correct the counters the failed attempt touched
                mgr.hit_tokens -= opened.cached_tokens
                mgr.miss_tokens -= (target - opened.cached_tokens) if target else 0
                return
            self.waiting.popleft()
            seq.admitted = True
            seq.n_kv = min(opened.cached_tokens, target)
            if not seq.preemptions:
                seq.cached_prefix_tokens = seq.n_kv
                seq.t_admit = self.clock()
            self.stats.tokens_saved_by_cache += seq.n_kv
            seq.state = SeqState.PREFILL if seq.n_kv < target else SeqState.RUNNING
            self.active.append(seq)

    # -- planning ----------------------------------------------------------------
    def plan(self) -> list[Planned]:
        """Choose the entries of the next step (reserving pages; may preempt)."""
        self._admit()
        prefilling = [s for s in self.active if s.state == SeqState.PREFILL]
        planned: list[Planned] = []
        budget = self.max_prefill_tokens
        if self.policy == "prefill_first":
            if prefilling:
                return [self._portion(prefilling[0], budget)]
            return self._decodes()
        planned = self._decodes()
        budget -= len(planned)
        for seq in prefilling:
            if budget <= 0:
                break
            if seq.state != SeqState.PREFILL:      # preempted meanwhile
                continue
            p = self._portion(seq, budget)
            planned.append(p)
            budget -= len(p.tokens)
        return planned

    def _portion(self, seq: SequenceState, budget: int) -> Planned:
        if seq.prefill_tokens_computed == 0 and self.manager.prefix_cache:
            # nothing of it has run yet: pages published since its admission (by requests
            # admitted together with it) may cover more of its prompt by now
            before = seq.n_kv
            got = min(self.manager.rematch(seq.req_id, seq.ctx[:seq.prefill_target]),
                      seq.prefill_target)
            if got > before:
                seq.n_kv = got
                if not seq.preemptions:
                    seq.cached_prefix_tokens = got
                self.stats.tokens_saved_by_cache += got - before
        start = seq.n_kv
        end = min(start + budget, seq.prefill_target)
        toks = seq.ctx[start:end]
        # pages for the whole prompt were reserved at admission
        samples = end >= seq.prefill_target and not seq.output_ids
        return Planned(seq, start, toks, samples)

    def _decodes(self) -> list[Planned]:
        mgr = self.manager
        planned: list[Planned] = []
        running = [s for s in self.active if s.state == SeqState.RUNNING][: self.max_batch]
        for seq in running:
            if seq.pending and self._ends_by_count(seq, seq.pending):
                continue                            # its token in flight is its last
            while seq.state == SeqState.RUNNING:    # else: preempted, or ended while we waited
                try:
                    mgr.reserve(seq.req_id, seq.n_kv + 1)
                    tok = FROM_DEVICE if seq.pending else seq.ctx[seq.n_kv]
                    planned.append(Planned(seq, seq.n_kv, [tok], True))
                    break
                except OutOfPages:
                    victim = self._preempt_newest()
                    if victim is seq or victim is None:
                        break
                    planned = [p for p in planned if p.seq is not victim]
        return planned

    def _ends_by_count(self, seq: SequenceState, extra: int) -> bool:
        """Would ``extra`` more tokens end the request whatever they are?"""
        n = len(seq.output_ids) + extra
        return (n >= seq.request.max_new_tokens
                or len(seq.request.prompt_ids) + n >= self.max_ctx)

    def _preempt_newest(self) -> SequenceState | None:
        """Recompute-preemption of the newest running request (worker.py:738-757)."""
        if self._inflight is not None:
            # a preempted request is prefilled again over all its tokens: have them first
            self._late_done.extend(self._resolve())
        running = [s for s in self.active if s.state == SeqState.RUNNING]
        if not running:
            return None
        victim = running[-1]
        self.manager.publish(victim.req_id, victim.ctx[: victim.n_kv])
        self.manager.close(victim.req_id)
        self.active.remove(victim)
        victim.n_kv = 0
        victim.admitted = False
        victim.state = SeqState.WAITING
        victim.preemptions += 1
        self.stats.preemptions += 1
        self.waiting.appendleft(victim)
        return victim

    # -- running a step -------------------------------------------------------------
    def step(self) -> list[SequenceState]:
        """Plan and launch one step; returns the requests whose end became known in it.  With
        ``pipeline`` the tokens of the step launched here are read in the NEXT call."""
        planned = self.plan()
        done, self._late_done = self._late_done, []
        # requests that ended while the plan waited for tokens in flight have left it
        planned = [p for p in planned
                   if p.seq.state in (SeqState.PREFILL, SeqState.RUNNING)]
        if not planned:
            if self._inflight is not None:
                done.extend(self._resolve())
                return done
            if self.waiting and not self.active:
                head = self.waiting[0]
                if head.output_ids:
                    # it outgrew the whole pool while generating: end it with what it has
                    self.waiting.popleft()
                    head.state, head.finish_reason = SeqState.DONE, "out_of_pages"
                    head.t_done = self.clock()
                    self.finished.append(head)
                    self.stats.finished += 1
                    return done + [head]
                raise RequestRefused(
                    f"request {head.req_id!r} cannot be admitted although nothing else is "
                    f"running: the pool is too small for it")
            return done
        entries = []
        for p in planned:
            r = p.seq.request
            entries.append(StepEntry(
                p.seq.req_id, p.tokens, want=[len(p.tokens) - 1] if p.samples else (),
                temperature=r.temperature, top_k=r.top_k, seed=r.seed))
        result = self.step_fn(entries)
        n_dec = sum(1 for p in planned if len(p.tokens) == 1 and p.seq.state == SeqState.RUNNING)
        for p in planned:
            seq = p.seq
            was_prefill = seq.state == SeqState.PREFILL
            seq.n_kv = p.start + len(p.tokens)
            if was_prefill:
                seq.prefill_tokens_computed += len(p.tokens)
                self.stats.tokens_prefilled += len(p.tokens)
                if seq.n_kv >= seq.prefill_target:
                    # publish the finished prompt so that others can share it (worker.py:635-645)
                    self.manager.publish(seq.req_id, seq.ctx[: seq.n_kv])
                    seq.state = SeqState.RUNNING
            if p.samples:
                seq.pending += 1
        self.stats.steps += 1
        if n_dec == len(planned):
            self.stats.decode_steps += 1
        elif n_dec == 0:
            self.stats.prefill_steps += 1
        else:
            self.stats.mixed_steps += 1
        earlier, self._inflight = self._inflight, (planned, result)
        if earlier is not None:
            done.extend(self._read(earlier))
        if not self.pipeline:
            done.extend(self._resolve())
        return done

    def _resolve(self) -> list[SequenceState]:
        """Read the tokens of the step in flight, if any."""
        inflight, self._inflight = self._inflight, None
        return self._read(inflight) if inflight is not None else []

    def _read(self, inflight) -> list[SequenceState]:
        planned, result = inflight
        tokens = result.tokens_host() if hasattr(result, "tokens_host") else result
        it = iter(tokens)
        done: list[SequenceState] = []
        now = self.clock()
        for p in planned:
            if not p.samples:
                continue
            tok = int(next(it))
            seq = p.seq
            if seq.state == SeqState.DONE:
                continue            # ended (or aborted) while this step was in flight
            seq.pending -= 1
            seq.output_ids.append(tok)
            self.stats.tokens_generated += 1
            if not seq.t_first_token:
                seq.t_first_token = now
            if self._finished(seq, tok):
                self._finish(seq, now)
                done.append(seq)
        return done

    def _finished(self, seq: SequenceState, tok: int) -> bool:
        r = seq.request
        if len(seq.output_ids) >= r.max_new_tokens:
            seq.finish_reason = "max_new_tokens"
        elif r.stop_at_eos and self.eos_token_id is not None and tok == self.eos_token_id:
            seq.finish_reason = "eos"
        elif len(r.prompt_ids) + len(seq.output_ids) >= self.max_ctx:
            seq.finish_reason = "max_ctx"
        return bool(seq.finish_reason)

    def _finish(self, seq: SequenceState, now: float) -> None:
        seq.state = SeqState.DONE
        seq.t_done = now
        # what was generated becomes reusable too (worker.py:720-721)
        self.manager.publish(seq.req_id, seq.ctx[: seq.n_kv])
        self.manager.close(seq.req_id)
        self.active.remove(seq)
        self.finished.append(seq)
        self.stats.finished += 1

    def abort(self, req_id) -> bool:
        """Drop a request wherever it is; what it holds is given back."""
        for seq in list(self.active):
            if seq.req_id == req_id:
                self.manager.close(req_id)
                self.active.remove(seq)
                seq.state, seq.finish_reason = SeqState.DONE, "aborted"
                return True
        for seq in list(self.waiting):
            if seq.req_id == req_id:
                self.waiting.remove(seq)
                seq.state, seq.finish_reason = SeqState.DONE, "aborted"
                return True
        return False

    def state_message(self) -> dict:
        """Counters in the manner of the worker's state message (worker.py:786-812)."""
        s = self.stats
        return {
            "kv": self.manager.snapshot(),
            "queued": len(self.waiting) + sum(1 for q in self.active if q.state == SeqState.PREFILL),
            "running": sum(1 for q in self.active if q.state == SeqState.RUNNING),
            "steps": s.steps, "prefill_steps": s.prefill_steps, "decode_steps": s.decode_steps,
            "mixed_steps": s.mixed_steps, "tokens_generated": s.tokens_generated,
            "tokens_prefilled": s.tokens_prefilled,
            "tokens_saved_by_cache": s.tokens_saved_by_cache, "preemptions": s.preemptions,
            "finished": s.finished,
        }
