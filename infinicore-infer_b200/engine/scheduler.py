"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees; and decides what happens when pages run out.

It is host-side logic over the cache manager's bookkeeping and needs no GPU: ``schedule()``
returns the step to run, the caller runs it (``Engine.step``) and reports the sampled tokens
back with ``complete()``.

Policy of one step, in this order (rows are laid out in the same order):
  1. every running request that is decoding contributes its one pending token;
  2. the rest of the token budget goes to prompt portions of at most ``chunk_size`` tokens,
     oldest request first; a portion may be as small as what is left of the budget;
  3. waiting requests are admitted, oldest first, while a request slot is free, fewer than
     ``max_batch`` run, budget is left and the pages of their first portion can be had.
When pages run out: a portion shrinks to the pages that are free, or waits a step; if the
decoding requests themselves cannot all get a page, the YOUNGEST running request is preempted
by recomputation: its pages and slot are freed, it goes to the front of the waiting queue with
prompt + generated tokens as its new prompt, and the tokens it sampled are kept.  A request
that cannot run even alone in an empty cache finishes with reason ``length``.

The reference's counterpart: ``InferTask`` (scripts/infer_task.py:1-36), ``KVCachePool``
(scripts/kvcache_pool.py:8-90) and the worker loop (scripts/launch_server.py:134-159), which
admit a request when a whole-context cache is free and run every new prompt whole.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from ..cache import CacheManager

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
    """A request and its progress.  ``tokens`` = prompt + generated; ``computed`` of them are in
    the cache; the rest is pending (many while the prompt is read, exactly one while decoding)."""
    id: object
    prompt: Sequence[int]
    max_new_tokens: int = 16
    temperature: float = 0.0
    topk: int = 0
    topp: float = 1.0
    seed: int = 0
    eos_token_ids: Tuple[int, ...] = ()
    # progress
    generated: List[int] = field(default_factory=list)
    computed: int = 0
    status: str = WAITING
    finish_reason: Optional[str] = None
    preemptions: int = 0
    arrival: int = -1

    @property
    def tokens(self) -> List[int]:
        return list(self.prompt) + self.generated

    @property
    def pending(self) -> int:
        return len(self.prompt) + len(self.generated) - self.computed

    @property
    def decoding(self) -> bool:
        return self.status == RUNNING and self.pending == 1 and len(self.generated) > 0


@dataclass
class Scheduled:
    request: Request
    tokens: List[int]
    samples: bool          # the portion ends the pending tokens: a new token is sampled from its last row


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch: int = 64, max_tokens_per_step: int = 2048,
                 chunk_size: int = 512, max_positions: Optional[int] = None):
        if chunk_size < 1 or max_tokens_per_step < 1 or max_batch < 1:
            raise ValueError("limits must be positive")
        self.cache = cache
        self.max_batch = max_batch
        self.max_tokens_per_step = max_tokens_per_step
        self.chunk_size = chunk_size
        self.max_positions = max_positions or cache.max_positions
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self._arrivals = 0
        self._preempted = False
        self.counters = {"steps": 0, "tokens": 0, "preemptions": 0, "admitted": 0, "finished": 0,
                         "shrunk_portions": 0}

    # ---- entering ----------------------------------------------------------------------------
    def add(self, req: Request) -> None:
        if not len(req.prompt):
            raise ValueError(f"request {req.id!r} has an empty prompt")
        if req.arrival < 0:
            req.arrival = self._arrivals
            self._arrivals += 1
        req.status = WAITING
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- page arithmetic (all groups) -----------------------------------------------------------
    def _free_pages(self) -> List[int]:
        return [g.pool.available for g in self.cache.groups]

    def _fits(self, req: Request, new_len: int, free: List[int]) -> bool:
        return all(n <= f for n, f in zip(self.cache.pages_needed(req.id, new_len), free))

    def _take(self, req: Request, new_len: int, free: List[int]) -> None:
        for i, n in enumerate(self.cache.pages_needed(req.id, new_len)):
            free[i] -= n

    def _largest_fit(self, req: Request, want: int, free: List[int]) -> int:
        """The most tokens (<= want) of req's pending ones whose pages are free."""
        lo, hi = 0, want
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if self._fits(req, req.computed + mid, free):
                lo = mid
            else:
                hi = mid - 1
        return lo

    # ---- one step ---------------------------------------------------------------------------------
    def schedule(self) -> List[Scheduled]:
        """Decide the next step.  Preempts and finishes requests as needed; returns the entries in
        row order (decoding requests first).  An empty list means nothing can run."""
        self._preempted = False
        while True:
            plan = self._plan()
            if plan is not None:
                return plan

    def _plan(self) -> Optional[List[Scheduled]]:
        free = self._free_pages()
        budget = self.max_tokens_per_step
        out: List[Scheduled] = []
        # 1. decoding requests
        decoders = [r for r in self.running if r.decoding]
        for r in decoders:
            if not self._fits(r, r.computed + 1, free):
                self._preempt_youngest()
                return None                       # plan again with the pages that came back
            self._take(r, r.computed + 1, free)
            out.append(Scheduled(r, [r.tokens[r.computed]], True))
            budget -= 1
        # 2. portions of running prompts, oldest first
        for r in sorted((r for r in self.running if not r.decoding), key=lambda r: r.arrival):
            if budget <= 0:
                break
            n = min(self.chunk_size, budget, r.pending)
            fit = self._largest_fit(r, n, free)
            if fit < n:
                self.counters["shrunk_portions"] += 1
            if fit == 0:
                continue
            self._take(r, r.computed + fit, free)
            toks = r.tokens[r.computed: r.computed + fit]
            out.append(Scheduled(r, toks, fit == r.pending))
            budget -= fit
        # 3. admissions (none in a step that had to preempt: the pages that came back are the decoders')
        while (self.waiting and budget > 0 and len(self.running) < self.max_batch and not self._preempted
               and self.cache.slots.available > len([s for s in out if not self.cache.is_live(s.request.id)])):
            r = self.waiting[0]
            total = len(r.prompt) + len(r.generated)
            if total > self.max_positions or not self._can_ever_fit(r):
                self.waiting.popleft()
                self._finish(r, "length")
                continue
            n = min(self.chunk_size, budget, r.pending)
            if not self._fits(r, r.computed + n, free):
                break                             # wait until the whole first portion fits; keep the queue's order
            fit = n
            self.waiting.popleft()
            r.status = RUNNING
            self.running.append(r)
            self.counters["admitted"] += 1
            self._take(r, r.computed + fit, free)
            out.append(Scheduled(r, r.tokens[r.computed: r.computed + fit], fit == r.pending))
            budget -= fit
        if not out and self.running:
            # running requests exist but none can move: free pages by preempting the youngest;
            # a lone request that still cannot move can never finish
            if len(self.running) == 1:
                self._finish(self.running[0], "length")
            else:
                self._preempt_youngest()
            return None
        return out

    def _can_ever_fit(self, r: Request) -> bool:
        """Could the request's next token ever be computed, alone in an empty cache?"""
        total = len(r.prompt) + len(r.generated)
        return all(g.need.most_pages_alone(total, self.chunk_size, self.cache.page_size) <= g.pool.capacity
                   for g in self.cache.groups)

    def _preempt_youngest(self) -> None:
        victim = max(self.running, key=lambda r: r.arrival)
        self._preempted = True
        if len(self.running) == 1:
            self._finish(victim, "length")
            return
        self.running.remove(victim)
        if self.cache.is_live(victim.id):
            self.cache.release(victim.id)
        victim.computed = 0
        victim.status = WAITING
        victim.preemptions += 1
        self.counters["preemptions"] += 1
        self.waiting.appendleft(victim)

    def _finish(self, r: Request, reason: str) -> None:
        if r in self.running:
            self.running.remove(r)
        if self.cache.is_live(r.id):
            self.cache.release(r.id)
        r.status, r.finish_reason = FINISHED, reason
        self.finished.append(r)
        self.counters["finished"] += 1

    # ---- after the step ------------------------------------------------------------------------------
    def complete(self, plan: Sequence[Scheduled], sampled: Sequence[Optional[int]]) -> List[Request]:
        """Report a step's result: ``sampled[i]`` is the new token of ``plan[i]`` (ignored unless
        ``plan[i].samples``).  Returns the requests that finished."""
        done = []
        self.counters["steps"] += 1
        for s, tok in zip(plan, sampled):
            r = s.request
            r.computed += len(s.tokens)
            self.counters["tokens"] += len(s.tokens)
            if not s.samples:
                continue
            r.generated.append(int(tok))
            if int(tok) in r.eos_token_ids:
                self._finish(r, "stop"); done.append(r)
            elif len(r.generated) >= r.max_new_tokens:
                self._finish(r, "length"); done.append(r)
            elif r.computed + 1 > self.max_positions:
                self._finish(r, "length"); done.append(r)
        return done

    def cancel(self, req_id) -> bool:
        for r in list(self.running) + list(self.waiting):
            if r.id == req_id:
                if r in self.waiting:
                    self.waiting.remove(r)
                self._finish(r, "cancel")
                return True
        return False
