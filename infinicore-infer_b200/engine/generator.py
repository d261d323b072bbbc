"""Generation: the scheduler, the step function and the sampler in one loop.

``Generator.step()`` asks the scheduler for the next batch, runs it through ``Engine.step``,
samples a token for every request whose pending tokens were all consumed, and reports the
tokens back.  The reference's loop of this kind is the server's worker
(scripts/launch_server.py:134-159) and ``generate`` (scripts/jiuge.py:539-586).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

from ..sampling import Sampler, SamplingParams
from .scheduler import Request, Scheduled, Scheduler
from .step import Engine, StepEntry


class Generator:
    def __init__(self, engine: Engine, max_batch: Optional[int] = None, max_tokens_per_step: Optional[int] = None,
                 chunk_size: int = 512):
        self.engine = engine
        self.scheduler = Scheduler(engine.cache, max_batch=max_batch or engine.max_requests,
                                   max_tokens_per_step=min(max_tokens_per_step or engine.max_step_tokens,
                                                           engine.max_step_tokens),
                                   chunk_size=chunk_size, max_positions=engine.spec.max_positions)
        self.sampler = Sampler(engine.device)
        self._next_id = 0

    def submit(self, prompt: Sequence[int], max_new_tokens: int = 16, temperature: float = 0.0, topk: int = 0,
               topp: float = 1.0, seed: int = 0, eos_token_ids: Optional[Sequence[int]] = None,
               req_id=None) -> Request:
        if req_id is None:
            req_id = f"g{self._next_id}"
            self._next_id += 1
        eos = tuple(self.engine.spec.eos_token_ids) if eos_token_ids is None else tuple(eos_token_ids)
        req = Request(id=req_id, prompt=list(prompt), max_new_tokens=max_new_tokens, temperature=temperature,
                      topk=topk, topp=topp, seed=seed, eos_token_ids=eos)
        self.scheduler.add(req)
        return req

    def step(self) -> List[Tuple[Request, int]]:
        """Run one scheduled step; return (request, new token) for every token produced."""
        plan = self.scheduler.schedule()
        if not plan:
            return []
        entries = [StepEntry(s.request.id, s.tokens, [len(s.tokens) - 1] if s.samples else [])
                   for s in plan]
        # a step of single tokens is most often followed by the same requests' next tokens: the engine may prepare that
        # step while the device runs this one (what it takes ahead is what these requests, who come first, would take
        # next anyway, and goes back if another step comes)
        logits = self.engine.step(entries, stage_next=all(len(s.tokens) == 1 for s in plan))
        samplers = [s for s in plan if s.samples]
        params = [SamplingParams(s.request.temperature, s.request.topk, s.request.topp, s.request.seed)
                  for s in samplers]
        # the uniform of a new token depends on the request's seed and the token's absolute position
        new = self.sampler.sample(logits, params, [len(s.request.prompt) + len(s.request.generated) for s in samplers])
        self.engine.check()
        it = iter(new)
        sampled = [next(it) if s.samples else None for s in plan]
        self.scheduler.complete(plan, sampled)
        return [(s.request, t) for s, t in zip(plan, sampled) if s.samples]

    def run(self) -> None:
        while self.scheduler.has_work():
            self.step()

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16, **sampling) -> List[List[int]]:
        reqs = [self.submit(p, max_new_tokens=max_new_tokens, **sampling) for p in prompts]
        self.run()
        return [r.generated for r in reqs]
