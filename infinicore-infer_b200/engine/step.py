"""The step function: a batch of (request, its next tokens) in, logits at the wanted rows out.

One call runs exactly the tokens it is given, as one batch, against the cache that earlier
calls left: portions of prompts beside single decoded tokens, cut anywhere.  The reference's
counterpart is ``inferBatch`` / ``forwardBatch`` with ``tokens, req_lens, req_pos``
(include/infinicore_infer/models/jiuge.h:89-110, src/models/jiuge/jiuge.cpp:114-298); here a
request's position is what the cache holds of it, logits come back for the rows asked for,
and errors are exceptions raised before anything ran.

A step whose entries all carry one token is a decode step: it runs as a CUDA graph captured
once per batch-size bucket, with the batch padded by rows that read and write the null page.
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
from ..parts import SHORT_ROWS, TILE_ROWS, Model, Runtime, StepContext, cache_needs, model_manifest
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


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class _Layout:
    """Offsets (in int32 elements) of a step's arrays inside the metadata buffer."""

    def __init__(self, T: int, B: int, n_groups: int, max_blocks: int):
        self.T, self.B = T, B
        o = 0
        self.tokens = o; o += _align(T)
        self.positions = o; o += _align(T)
        self.row_req = o; o += _align(T)
        self.want_rows = o; o += _align(T)
        self.req_start = o; o += _align(B + 1)
        self.req_pos = o; o += _align(B)
        self.slot_ids = o; o += _align(B)
        self.short_rows = o; o += _align(T)
        self.tiles = o; o += _align(2 * (T // TILE_ROWS + B))
        self.tables = []
        for _ in range(n_groups):
            self.tables.append(o); o += _align(B * max_blocks)
        self.total = o


class Engine:
    """A model, its cache and the step function over them."""

    def __init__(self, spec, weights, dtype: torch.dtype = torch.bfloat16, device="cuda:0",
                 cache_tokens: int = 4096, page_size: int = 16, max_requests: int = 64,
                 max_step_tokens: int = 8192, use_graphs: bool = True, native_runner: bool = True,
                 strict_weights: bool = False):
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
        n_groups, mb = len(self.cache.groups), self.cache.max_blocks
        cap = _Layout(max_step_tokens, max_requests, n_groups, mb).total
        self._meta_dev = torch.zeros(cap, dtype=torch.int32, device=self.device)
        self._meta_host = [torch.zeros(cap, dtype=torch.int32, pin_memory=True) for _ in range(3)]
        self._meta_events: List[Optional[torch.cuda.Event]] = [None] * 3
        self._meta_turn = 0
        self._decode_templates: Dict[int, tuple] = {}
        self._graphs: Dict[int, object] = {}
        self.steps_run = 0
        self.tokens_run = 0
        self.kernel_launches = 0      # this package's kernels launched by steps (replayed graphs included)
        # the standard stack is issued from native code (csrc/runner.cu); other models through the parts
        self.runner = None
        if native_runner and os.environ.get("JK_NO_RUNNER") != "1":
            from .runner import NativeRunner
            self.runner = NativeRunner.build(self)

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
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the entries as one batch; return float32 logits ``[wanted, vocab]`` on the device,
        in the order of the entries and of their ``want``."""
        entries = [e for e in entries if len(e.tokens)]
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
            from .. import kernels
            ctx = self._upload(entries, starts, len(entries), sum(len(e.tokens) for e in entries))
            before = kernels.launch_count
            logits = self._forward(ctx)
            self.kernel_launches += kernels.launch_count - before
        for r, n in new_len.items():
            self.cache.commit(r, n)
        self.steps_run += 1
        self.tokens_run += sum(len(e.tokens) for e in entries)
        return logits

    def _forward(self, ctx: StepContext) -> torch.Tensor:
        if self.runner is not None:
            from .. import kernels
            logits = self.runner.forward(ctx)
            kernels.launch_count += self.runner.launches
            return logits
        return self.model.forward(ctx, self.cache.views)

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
    def _upload(self, entries, starts, B: int, T: int, pad_to: Optional[int] = None) -> StepContext:
        """Fill the pinned buffer, copy it in one piece, return views of the device copy.

        ``pad_to``: batch size of a captured decode step; missing entries become rows that use
        slot 0 and the null page at position 0.
        """
        nB = pad_to or B
        nT = pad_to or T
        lay = _Layout(nT, nB, len(self.cache.groups), self.cache.max_blocks)
        turn = self._meta_turn
        self._meta_turn = (turn + 1) % len(self._meta_host)
        if self._meta_events[turn] is not None:
            self._meta_events[turn].synchronize()
        host = self._meta_host[turn].numpy()
        host[:lay.total] = 0
        row = 0
        want_rows: List[int] = []
        req_start = [0]
        for i, (e, s) in enumerate(zip(entries, starts)):
            n = len(e.tokens)
            host[lay.tokens + row: lay.tokens + row + n] = np.asarray(e.tokens, dtype=np.int32)
            host[lay.positions + row: lay.positions + row + n] = np.arange(s, s + n, dtype=np.int32)
            host[lay.row_req + row: lay.row_req + row + n] = i
            want_rows.extend(row + w for w in e.want)
            row += n
            req_start.append(row)
        for i in range(B, nB):           # padding rows of a captured step
            host[lay.row_req + row] = i
            row += 1
            req_start.append(row)
        short_rows: List[int] = []
        tile_list: List[tuple] = []
        for i in range(nB):
            r0, r1 = req_start[i], req_start[i + 1]
            if r1 - r0 <= SHORT_ROWS:
                short_rows.extend(range(r0, r1))
            else:
                for t0 in range(r0, r1, TILE_ROWS):
                    tile_list.append((starts[i] + (t0 - r0), i, t0))
        # the attention kernels start tiles in the order of the list: those that see the most keys first
        tile_list.sort(key=lambda t: -t[0])
        tiles: List[int] = [v for t in tile_list for v in t[1:]]
        host[lay.short_rows: lay.short_rows + len(short_rows)] = short_rows
        host[lay.tiles: lay.tiles + len(tiles)] = tiles
        n_want = len(want_rows)
        if pad_to:                       # a captured step computes logits for every row
            want_rows = list(range(nT))
        host[lay.want_rows: lay.want_rows + len(want_rows)] = want_rows
        host[lay.req_start: lay.req_start + nB + 1] = req_start
        host[lay.req_pos: lay.req_pos + B] = starts
        reqs = [e.req_id for e in entries]
        slots = self.cache.slot_ids(reqs)
        host[lay.slot_ids: lay.slot_ids + B] = slots
        mb = self.cache.max_blocks
        for gi, off in enumerate(lay.tables):
            self.cache.block_table_rows(gi, reqs, host[off: off + nB * mb].reshape(nB, mb))
        self._copy_meta(turn, lay.total)
        ctx = self._context(lay, len(want_rows))
        ctx.host_req_start = req_start
        ctx.host_req_pos = list(starts) + [0] * (nB - B)
        ctx.host_slot_ids = list(slots) + [0] * (nB - B)
        ctx.n_want = n_want if not pad_to else nT
        ctx.n_short, ctx.n_tiles = len(short_rows), len(tiles) // 2
        ctx.short_rows = None if ctx.n_short == nT else self._meta_dev[lay.short_rows: lay.short_rows + ctx.n_short]
        ctx.tiles = self._meta_dev[lay.tiles: lay.tiles + len(tiles)]
        return ctx

    def _copy_meta(self, turn: int, words: int) -> None:
        self._meta_dev[:words].copy_(self._meta_host[turn][:words], non_blocking=True)
        if self._meta_events[turn] is None:
            self._meta_events[turn] = torch.cuda.Event()
        self._meta_events[turn].record()

    def _upload_decode_replay(self, entries, starts, bucket: int) -> None:
        """The upload of a captured decode step that is only replayed: the same buffer contents as
        ``_upload(..., pad_to=bucket)`` gives, without the device views that only a capture needs.
        What does not change from step to step comes from a template made once per bucket."""
        B = len(entries)
        made = self._decode_templates.get(bucket)
        if made is None:
            lay = _Layout(bucket, bucket, len(self.cache.groups), self.cache.max_blocks)
            t = np.zeros(lay.total, dtype=np.int32)
            t[lay.row_req: lay.row_req + bucket] = np.arange(bucket)
            t[lay.req_start: lay.req_start + bucket + 1] = np.arange(bucket + 1)
            t[lay.short_rows: lay.short_rows + bucket] = np.arange(bucket)
            t[lay.want_rows: lay.want_rows + bucket] = np.arange(bucket)
            made = self._decode_templates[bucket] = (lay, t)
        lay, template = made
        turn = self._meta_turn
        self._meta_turn = (turn + 1) % len(self._meta_host)
        if self._meta_events[turn] is not None:
            self._meta_events[turn].synchronize()
        host = self._meta_host[turn].numpy()
        host[:lay.total] = template
        host[lay.tokens: lay.tokens + B] = [e.tokens[0] for e in entries]
        host[lay.positions: lay.positions + B] = starts
        host[lay.req_pos: lay.req_pos + B] = starts
        reqs = [e.req_id for e in entries]
        host[lay.slot_ids: lay.slot_ids + B] = self.cache.slot_ids(reqs)
        mb = self.cache.max_blocks
        for gi, off in enumerate(lay.tables):
            self.cache.block_table_rows(gi, reqs, host[off: off + bucket * mb].reshape(bucket, mb))
        self._copy_meta(turn, lay.total)

    def _context(self, lay: _Layout, n_want: int) -> StepContext:
        m, mb = self._meta_dev, self.cache.max_blocks
        sl = lambda off, n: m[off: off + n]
        return StepContext(
            ntok=lay.T, nreq=lay.B,
            tokens=sl(lay.tokens, lay.T), positions=sl(lay.positions, lay.T),
            row_req=sl(lay.row_req, lay.T), req_start=sl(lay.req_start, lay.B + 1),
            req_pos=sl(lay.req_pos, lay.B), slot_ids=sl(lay.slot_ids, lay.B),
            block_tables=[sl(off, lay.B * mb).view(lay.B, mb) for off in lay.tables],
            want_rows=sl(lay.want_rows, n_want), n_want=n_want)

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
        rec = self._graphs.get(bucket)
        if rec is None:
            # Warm up (library handles, lazy module loads) on a batch of padding rows only: they touch
            # the null page and slot 0, so a mixer whose state update is not idempotent sees the real
            # step exactly once, at the replay below.
            dummy = self._upload([], [], 0, 0, pad_to=bucket)
            dummy.decode_only = True
            self._forward(dummy)
            torch.cuda.synchronize()
        if rec is not None:
            self._upload_decode_replay(entries, starts, bucket)
        else:
            ctx = self._upload(entries, starts, B, B, pad_to=bucket)
            ctx.decode_only = True
            from .. import kernels
            graph = torch.cuda.CUDAGraph()
            before = kernels.launch_count
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
            rec = (graph, out, kernels.launch_count - before)
            self._graphs[bucket] = rec
        graph, out, launches = rec
        graph.replay()
        self.kernel_launches += launches
        # `out` is the captured graph's own buffer, which the next replay overwrites: the caller gets a copy
        if all(len(e.want) == 1 for e in entries):
            return out[:B].clone()
        rows = []
        for i, e in enumerate(entries):
            rows.extend([i] * len(e.want))
        if not rows:
            return out[:0]
        return out[torch.tensor(rows, device=self.device)]
