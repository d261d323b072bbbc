"""The step function: a batch of (request, its next tokens) in, logits at the wanted rows out.

One call runs exactly the tokens it is given, as one batch, against the cache that earlier
calls left: portions of prompts beside single decoded tokens, cut anywhere.  The reference's
counterpart is ``inferBatch`` / ``forwardBatch`` with ``tokens, req_lens, req_pos``
(include/infinicore_infer/models/jiuge.h:89-110, src/models/jiuge/jiuge.cpp:114-298); here a
request's position is what the cache holds of it, logits come back for the rows asked for,
and errors are exceptions raised before anything ran.

A step whose entries all carry one token is a decode step: it runs as a CUDA graph captured
once per (batch-size bucket, context bucket), with the batch padded by rows that read and write the null page.
"""
from __future__ import annotations

import gc
import os

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, OutOfPages
from ..config import read_config
from ..kernels import host as host_rules
from ..parts import Model, ProgramRunner, Runtime, StepContext, cache_needs, model_manifest
from ..weights import FileWeights, check_manifest


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places (indices into ``tokens``)
    whose logits are wanted."""
    req_id: object
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


class StepError(ValueError):
    """A step that cannot run as given (bad token, context overflow, unknown place)."""


class Engine:
    """A model, its cache and the step function over them."""

    def __init__(self, spec, weights, dtype: torch.dtype = torch.bfloat16, device="cuda:0",
                 cache_tokens: int = 4096, page_size: int = 16, max_requests: int = 64,
                 max_step_tokens: int = 8192, use_graphs: bool = True, native_runner: bool = True,
                 strict_weights: bool = False, context_buckets: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("the engine runs on a CUDA device only; there is no CPU path")
        self.spec = spec
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.runtime = Runtime(dtype, self.device)
        manifest = model_manifest(spec)
        check_manifest(manifest, weights.shapes(), where=getattr(weights, "model_dir", ""), strict=strict_weights)
        weights.plan(manifest)
        self.model = Model(spec, weights, self.runtime)
        weights.close()
        num_pages = (cache_tokens + page_size - 1) // page_size
        self.cache = CacheManager(cache_needs(spec), num_pages, page_size, max_requests,
                                  spec.max_positions, dtype=dtype, device=self.device)
        self.max_requests = max_requests
        self.max_step_tokens = max_step_tokens
        self.use_graphs = use_graphs and self.model.graph_safe
        # The model as launch records (parts/program.py) and the buffers that a step replays them over.  With
        # ``native_runner=False`` (or JK_NO_RUNNER=1) every record is a call of its own, so that no record shares work
        # with its neighbours: the unfused way of running the same program.
        self.program = self.model.plan(self.cache.views, page_size, self.cache.max_blocks)
        one_by_one = not native_runner or os.environ.get("JK_NO_RUNNER") == "1"
        self.runner = ProgramRunner(self.program, max_step_tokens, one_by_one=one_by_one)
        # what the mixers ask every step to carry (work lists), after the arrays that every model needs
        self._list_owners = list(self.program.list_owners)
        self._layouts: Dict[tuple, tuple] = {}
        cap = self._layout(max_step_tokens, max_requests)[0].total
        self._meta_dev = torch.zeros(cap, dtype=torch.int32, device=self.device)
        self._meta_host = [torch.zeros(cap, dtype=torch.int32, pin_memory=True) for _ in range(3)]
        self._meta_events: List[Optional[torch.cuda.Event]] = [None] * 3
        self._meta_turn = 0
        self._table_scratch = [np.zeros((max_requests, self.cache.max_blocks), dtype=np.int32) for _ in self.cache.groups]
        self._graphs: Dict[tuple, object] = {}
        # Captured decode steps are kept per (batch bucket, context bucket): how the decode attention cuts a row's keys
        # follows the live requests' lengths, not the model's longest context.
        self.context_buckets = context_buckets
        self.steps_run = 0
        self.tokens_run = 0
        self.kernel_launches = 0      # this package's kernels launched by steps (replayed graphs included)
        # A decode step that was asked to may prepare the step after it while the device still runs (see _stage_next).
        self._staged: Optional[tuple] = None
        self._may_stage = os.environ.get("JK_NO_STAGE") != "1"
        self.staged_steps = 0         # steps that ran from what the step before them had prepared

    # ---- construction -------------------------------------------------------------------------
    @classmethod
    def from_folder(cls, model_dir: str, dtype: torch.dtype = torch.bfloat16, device="cuda:0",
                    max_tokens: Optional[int] = None, **kw) -> "Engine":
        """Load ``config.json`` and the safetensors of a folder; the architecture's registry
        entry decides the configuration class."""
        config = read_config(model_dir, max_tokens=max_tokens)
        weights = FileWeights(model_dir, dtype, device)
        eng = cls(config.model_spec(), weights, dtype=dtype, device=device, **kw)
        eng.config = config
        return eng

    # ---- requests -----------------------------------------------------------------------------
    def begin(self, req_id) -> None:
        self.cache.admit(req_id)

    def end(self, req_id) -> None:
        self.cache.release(req_id)

    def check(self) -> None:
        """Raise if a kernel of an earlier step gave up a bounded wait (reads one word; synchronises)."""
        from .. import kernels
        kernels.check_gemm_status(self.device)

    def position(self, req_id) -> int:
        return self.cache.length(req_id) if self.cache.is_live(req_id) else 0

    # ---- the step -------------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], stage_next: bool = False) -> torch.Tensor:
        """Run the entries as one batch; return float32 logits ``[wanted, vocab]`` on the device,
        in the order of the entries and of their ``want``.  ``stage_next``: the caller expects to come back with one
        more token for each of these requests (a decode loop); the step may then prepare that step before it returns."""
        entries = [e for e in entries if len(e.tokens)]
        staged, self._staged = self._staged, None
        if staged is not None:
            if entries and self._staged_fits(staged, entries):
                return self._run_staged(staged, entries, stage_next)
            self._drop_staged(staged)
        if not entries:
            return torch.empty(0, self.spec.vocab_size, dtype=torch.float32, device=self.device)
        self._validate(entries)
        starts = [self.position(e.req_id) for e in entries]
        new_len = {e.req_id: s + len(e.tokens) for e, s in zip(entries, starts)}
        if not self.cache.can_reserve(new_len):          # checked for the whole step before anything changes
            raise OutOfPages(sum(sum(self.cache.pages_needed(r, n)) for r, n in new_len.items()),
                             min(g.pool.available for g in self.cache.groups), "step")
        for e in entries:
            if not self.cache.is_live(e.req_id):
                self.cache.admit(e.req_id)
        for r, n in new_len.items():
            self.cache.reserve(r, n)

        decode = self.use_graphs and all(len(e.tokens) == 1 for e in entries)
        if decode:
            logits = self._run_decode_graph(entries, starts)
        else:
            ctx = self._upload(entries, starts, len(entries), sum(len(e.tokens) for e in entries))
            logits = self._forward(ctx)
            self.kernel_launches += self.runner.launches
        for r, n in new_len.items():
            self.cache.commit(r, n)
        self.steps_run += 1
        self.tokens_run += sum(len(e.tokens) for e in entries)
        if decode and stage_next:
            self._stage_next([e.req_id for e in entries], [s + 1 for s in starts])
        return logits

    # ---- the step after a decode step, prepared while the device runs this one --------------------------------
    # Between two decode steps of the same requests the device idles while the host validates, takes pages, packs the
    # metadata and launches.  All of that but the token ids is known one step early: after a decode step's graph is
    # launched, the next step's pages are taken and its metadata packed into a pinned buffer of its own.  If the next
    # call brings exactly one token for each of the same requests, only the ids are written, the buffer copied and the
    # graph replayed; if it brings anything else, the pages taken ahead go back before the step is planned.
    def _stage_next(self, reqs: List[object], starts: List[int]) -> None:
        if not self._may_stage or any(s + 1 > self.spec.max_positions for s in starts):
            return
        B = len(reqs)
        bucket = self._bucket(B)
        if bucket > self.max_requests:
            bucket = B
        key = (bucket, self._context_of(starts, [1] * B))
        new_len = {r: s + 1 for r, s in zip(reqs, starts)}
        if key not in self._graphs or not self.cache.can_reserve(new_len):
            return
        for r, n in new_len.items():
            self.cache.reserve(r, n)
        lay, turn = self._pack([StepEntry(r, [0], [0]) for r in reqs], starts, B, B, pad_to=bucket, copy=False)
        self._staged = (tuple(reqs), list(starts), new_len, key, lay, turn)

    def _staged_fits(self, staged, entries) -> bool:
        reqs, starts = staged[0], staged[1]
        return len(entries) == len(reqs) and all(
            e.req_id == r and len(e.tokens) == 1 and self.cache.is_live(r) and self.cache.length(r) == s
            for e, r, s in zip(entries, reqs, starts))

    def _drop_staged(self, staged) -> None:
        for r in staged[0]:
            if self.cache.is_live(r):
                self.cache.truncate(r, self.cache.length(r))

    def _run_staged(self, staged, entries, stage_next: bool) -> torch.Tensor:
        reqs, starts, new_len, key, lay, turn = staged
        B = len(entries)
        tokens = [e.tokens[0] for e in entries]
        if min(tokens) < 0 or max(tokens) >= self.spec.vocab_size or any(w != 0 for e in entries for w in e.want):
            self._drop_staged(staged)
            self._validate(entries)           # says what is wrong with them
            raise StepError("a wanted place is not among a request's tokens")
        host = self._meta_host[turn].numpy()
        host[lay.tokens: lay.tokens + B] = tokens
        self._meta_dev[:lay.total].copy_(self._meta_host[turn][:lay.total], non_blocking=True)
        if self._meta_events[turn] is None:
            self._meta_events[turn] = torch.cuda.Event()
        self._meta_events[turn].record()
        graph, out, launches = self._graphs[key]
        graph.replay()
        self.kernel_launches += launches
        for r, n in new_len.items():
            self.cache.commit(r, n)
        self.steps_run += 1
        self.staged_steps += 1
        self.tokens_run += B
        logits = self._graph_rows(out, entries)
        if stage_next:
            self._stage_next(list(reqs), [s + 1 for s in starts])
        return logits

    def _forward(self, ctx: StepContext) -> torch.Tensor:
        return self.runner.forward(ctx, self.spec.vocab_size)

    # ---- checks that run before anything touches the device ------------------------------------
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        seen = set()
        total = 0
        for e in entries:
            if e.req_id in seen:
                raise StepError(f"request {e.req_id!r} appears twice in one step")
            seen.add(e.req_id)
            n = len(e.tokens)
            total += n
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= self.spec.vocab_size:
                raise StepError(f"request {e.req_id!r}: token id {lo if lo < 0 else hi} is outside "
                                f"the vocabulary of {self.spec.vocab_size}")
            if self.position(e.req_id) + n > self.spec.max_positions:
                raise StepError(f"request {e.req_id!r}: position {self.position(e.req_id) + n} exceeds "
                                f"the model's {self.spec.max_positions}")
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"request {e.req_id!r}: wanted place {w} is not among its {n} tokens")
        if total > self.max_step_tokens:
            raise StepError(f"{total} tokens in one step exceed the engine's {self.max_step_tokens}")
        new = sum(1 for e in entries if not self.cache.is_live(e.req_id))
        if new > self.cache.slots.available:
            raise StepError(f"{new} new requests but {self.cache.slots.available} request slots free")

    # ---- host -> device metadata ------------------------------------------------------------------
    def _layout(self, T: int, B: int):
        """The layout of a step of T rows and B requests, with the place of every work list in its extra words."""
        key = (T, B)
        made = self._layouts.get(key)
        if made is None:
            places, extra = [], 0
            for owner in self._list_owners:
                for name, words in owner.step_list_capacity(T, B).items():
                    places.append((owner, name, extra, words))
                    extra += (words + 3) // 4 * 4
            lay = host_rules.StepLayout(T, B, len(self.cache.groups), self.cache.max_blocks, extra)
            made = self._layouts[key] = (lay, places)
        return made

    def _pack(self, entries, starts, B: int, T: int, pad_to: Optional[int] = None, copy: bool = True):
        """Fill a pinned buffer with the step's metadata (``jk::pack_step`` and the mixers' work lists) and copy it in
        one piece.  ``pad_to``: batch size of a captured decode step; missing entries become rows that use slot 0
        and the null page at position 0, and every row is a wanted row."""
        nB, nT = pad_to or B, pad_to or T
        lay, places = self._layout(nT, nB)
        turn = self._meta_turn
        self._meta_turn = (turn + 1) % len(self._meta_host)
        if self._meta_events[turn] is not None:
            self._meta_events[turn].synchronize()
        host = self._meta_host[turn].numpy()
        tokens: List[int] = []
        want: List[int] = []
        lens = []
        for e in entries:
            n = len(e.tokens)
            want.extend(len(tokens) + w for w in e.want)
            tokens.extend(e.tokens)
            lens.append(n)
        n_want = len(want)
        if pad_to:
            want = list(range(nT))
        reqs = [e.req_id for e in entries]
        slots = self.cache.slot_ids(reqs)
        tables = []
        for gi in range(len(self.cache.groups)):
            rows = self._table_scratch[gi][:B]
            self.cache.block_table_rows(gi, reqs, rows)
            tables.append(rows)
        host_rules.pack_step(host, lay, B, tokens, lens, starts, slots, want, tables)
        counts = {}
        for owner in self._list_owners:
            arrays = {name: host[lay.extra + off: lay.extra + off + max(words, 1)] for o, name, off, words in places if o is owner}
            for name, got in owner.fill_step_lists(B, nB, lens, starts, arrays).items():
                counts[f"{owner.__name__}.{name}"] = got
        if not copy:
            return lay, turn
        self._meta_dev[:lay.total].copy_(self._meta_host[turn][:lay.total], non_blocking=True)
        if self._meta_events[turn] is None:
            self._meta_events[turn] = torch.cuda.Event()
        self._meta_events[turn].record()
        return lay, places, counts, lens, slots, (n_want if not pad_to else nT), len(want)

    def _context_of(self, starts, lens) -> int:
        if not self.context_buckets:
            return 0
        longest = max((s + n for s, n in zip(starts, lens)), default=1)
        return host_rules.context_bucket(longest, self.spec.max_positions)

    def _upload(self, entries, starts, B: int, T: int, pad_to: Optional[int] = None, context: Optional[int] = None) -> StepContext:
        """Pack and copy the step's metadata; return views of the device copy."""
        lay, places, counts, lens, slots, n_want, n_rows_wanted = self._pack(entries, starts, B, T, pad_to)
        m, mb = self._meta_dev, self.cache.max_blocks
        sl = lambda off, n: m[off: off + n]
        ctx = StepContext(
            ntok=lay.T, nreq=lay.B,
            tokens=sl(lay.tokens, lay.T), positions=sl(lay.positions, lay.T),
            row_req=sl(lay.row_req, lay.T), req_start=sl(lay.req_start, lay.B + 1),
            req_pos=sl(lay.req_pos, lay.B), slot_ids=sl(lay.slot_ids, lay.B),
            block_tables=[sl(off, lay.B * mb).view(lay.B, mb) for off in lay.tables],
            want_rows=sl(lay.want_rows, n_rows_wanted), n_want=n_want)
        ctx.context = self._context_of(starts, lens) if context is None else context
        for owner, name, off, words in places:
            count, identity = counts[f"{owner.__name__}.{name}"]
            ctx.lists[f"{owner.__name__}.{name}"] = (None if identity else sl(lay.extra + off, max(count, 1)), count)
        row, req_start = 0, [0]
        for n in lens:
            row += n
            req_start.append(row)
        for _ in range(lay.B - B):
            row += 1
            req_start.append(row)
        ctx.host_req_start = req_start
        ctx.host_req_pos = list(starts) + [0] * (lay.B - B)
        ctx.host_slot_ids = list(slots) + [0] * (lay.B - B)
        return ctx

    # ---- decode steps as CUDA graphs -----------------------------------------------------------------
    @staticmethod
    def _bucket(n: int) -> int:
        b = 1
        while b < n:
            b *= 2
        return b

    def _run_decode_graph(self, entries, starts) -> torch.Tensor:
        B = len(entries)
        bucket = self._bucket(B)
        if bucket > self.max_requests:
            bucket = B
        context = self._context_of(starts, [1] * B)
        key = (bucket, context)
        rec = self._graphs.get(key)
        if rec is None:
            # Warm up (library handles, lazy module loads) on a batch of padding rows only: they touch
            # the null page and slot 0, so a mixer whose state update is not idempotent sees the real
            # step exactly once, at the replay below.
            dummy = self._upload([], [], 0, 0, pad_to=bucket, context=context)
            dummy.decode_only = True
            self._forward(dummy)
            torch.cuda.synchronize()
            ctx = self._upload(entries, starts, B, B, pad_to=bucket, context=context)
            ctx.decode_only = True
            graph = torch.cuda.CUDAGraph()
            # no garbage collection while capturing: an unreachable engine's graphs, destroyed by the collector
            # in the middle of this capture, would invalidate it
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph):
                    out = self._forward(ctx)
            finally:
                if gc_was_on:
                    gc.enable()
            rec = (graph, out, self.runner.launches)
            self._graphs[key] = rec
        else:
            self._pack(entries, starts, B, B, pad_to=bucket)      # the same buffer contents; the views are the capture's
        graph, out, launches = rec
        graph.replay()
        self.kernel_launches += launches
        return self._graph_rows(out, entries)

    def _graph_rows(self, out: torch.Tensor, entries) -> torch.Tensor:
        # `out` is the captured graph's own buffer, which the next replay overwrites: the caller gets a copy
        B = len(entries)
        if all(len(e.want) == 1 for e in entries):
            return out[:B].clone()
        rows = []
        for i, e in enumerate(entries):
            rows.extend([i] * len(e.want))
        if not rows:
            return out[:0]
        return out[torch.tensor(rows, device=self.device)]
