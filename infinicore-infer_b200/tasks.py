"""Request objects with the reference's names and meanings: InferTask, KVCache, KVCachePool.

A user of the reference's Python side (scripts/infer_task.py, scripts/kvcache_pool.py) finds
the same three classes here with the same constructor arguments, attributes and methods, so
code that drives ``batch_infer_one_round`` carries over.  What stands behind them differs: a
``KVCache`` is a handle on one request of the paged cache manager (pages are taken as the
request grows and given back when the handle is dropped or goes back to a shorter prefix),
not a whole-context tensor per layer.
"""
from __future__ import annotations

import threading
from typing import List, Optional, Sequence, Tuple


class KVCache:
    """A cache handle plus a host-side record of the token ids it holds (for prefix reuse)."""

    def __init__(self, model):
        self._kvcache = model.create_kv_cache()
        self.tokens: List[int] = [0] * model.max_context_len()

    def data(self):
        return self._kvcache

    def drop(self, model) -> None:
        model.drop_kv_cache(self._kvcache)

    def update_tokens(self, tokens: Sequence[int], pos: int) -> None:
        """Record that ``tokens`` now sit at positions pos, pos+1, ... (what overflows is cut)."""
        room = len(self.tokens) - pos
        fit = list(tokens[:max(room, 0)])
        self.tokens[pos:pos + len(fit)] = fit


class InferTask:
    """One request between rounds: the tokens to feed next and where they start.

    After a round, ``next(token)`` records the fed tokens in the cache handle, moves ``pos``
    past them and decides: ``finish_reason`` becomes "stop" if the token is an end token (or
    None), "length" if ``pos`` has reached ``max_tokens`` (a bound on the absolute position,
    prompt included, as in scripts/infer_task.py:31-34), else ``tokens`` becomes ``[token]``.
    """

    def __init__(self, id, tokens, max_tokens, temperature, topk, topp, end_tokens):
        self.id = id
        self.tokens = tokens
        self.max_tokens = max_tokens
        self.temperature, self.topk, self.topp = temperature, topk, topp
        self.end_tokens = end_tokens
        self.finish_reason: Optional[str] = None
        self.pos = 0
        self._kv_cache: Optional[KVCache] = None

    def bind_kvcache(self, kv_cache: KVCache, pos: int = 0) -> None:
        """Attach a cache that already holds the first ``pos`` tokens of this task."""
        self._kv_cache, self.pos = kv_cache, pos
        self.tokens = self.tokens[pos:]

    def release_kvcache(self) -> Optional[KVCache]:
        kv, self._kv_cache = self._kv_cache, None
        return kv

    def kvcache(self) -> Optional[KVCache]:
        return self._kv_cache

    def next(self, out_token) -> None:
        fed = self.tokens
        self._kv_cache.update_tokens(fed, self.pos)
        self.pos += len(fed)
        if out_token is None or out_token in self.end_tokens:
            self.finish_reason = "stop"
            return
        if self.pos >= self.max_tokens:
            self.finish_reason = "length"
            return
        self.tokens = [out_token]


def common_prefix(a: Sequence[int], b: Sequence[int]) -> int:
    n = 0
    for x, y in zip(a, b):
        if x != y:
            break
        n += 1
    return n


class KVCachePool:
    """At most ``max_caches`` handles, made on demand and kept for reuse.

    ``acquire_sync(task)`` binds a handle to the task: a new one while fewer than
    ``max_caches`` exist, else the free one whose recorded tokens share the longest prefix
    with the task's prompt, bound at ``min(prefix, len(prompt) - 1)`` so that at least one
    token is left to feed (scripts/kvcache_pool.py:35-42, :58-76); with none free it waits.
    """

    def __init__(self, model, max_caches: int = 32):
        self.model = model
        self.max_caches = max_caches
        self.num_caches = 0
        self._available: List[KVCache] = []
        self._cond = threading.Condition()
        self._shutdown = False

    def find_most_matching_cache(self, tokens: Sequence[int]) -> Tuple[int, int]:
        best = max(range(len(self._available)),
                   key=lambda i: (common_prefix(tokens, self._available[i].tokens), -i), default=0)
        match = common_prefix(tokens, self._available[best].tokens) if self._available else 0
        return min(match, len(tokens) - 1), best

    def acquire_sync(self, infer_task: InferTask):
        with self._cond:
            while True:
                if self._shutdown:
                    raise RuntimeError("KVCachePool is shutting down; cannot acquire new cache.")
                if self._available:
                    match, index = self.find_most_matching_cache(infer_task.tokens)
                    return infer_task.bind_kvcache(self._available.pop(index), match)
                if self.num_caches < self.max_caches:
                    self.num_caches += 1
                    return infer_task.bind_kvcache(KVCache(self.model), 0)
                self._cond.wait()

    def release_sync(self, infer_task: InferTask) -> None:
        with self._cond:
            self._available.append(infer_task.release_kvcache())
            self._cond.notify()

    def finalize(self) -> None:
        """Wait until every handle is back, then drop them all."""
        with self._cond:
            self._shutdown = True
            while len(self._available) < self.num_caches:
                self._cond.wait()
            for kv in self._available:
                kv.drop(self.model)
            self._available.clear()
            self.max_caches = self.num_caches = 0
