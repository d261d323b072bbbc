"""Sampling the next token of each request from float32 logits on the device.

Options are the reference's per-request arrays (include/infinicore_infer/models/jiuge.h:85-87):
``temperature`` (0 = greedy), ``topk`` (1 = greedy; 0 or >= vocabulary = no cut), ``topp``
(1 = no cut).  The reference draws one uniform per request from a generator it reseeds from
the operating system at every step (src/models/jiuge/jiuge.cpp:279-284), so its runs cannot be
repeated; here the uniform for the token at absolute position i of a request is a hash of (seed, i) alone: the
same request samples the same tokens whatever else is in the batch and however its prompt
was cut.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import torch

from ..kernels.host import uniform_for      # noqa: F401  (seed, absolute position) -> [0, 1): one rule, written in csrc/host_rules.h


@dataclass
class SamplingParams:
    temperature: float = 0.0
    topk: int = 0
    topp: float = 1.0
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.topk == 1


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], indices: Sequence[int]) -> List[int]:
        """One token per row of ``logits``; ``indices[i]`` is the absolute position the new token
        of row i's request will take (the second argument of ``uniform_for``)."""
        from .. import kernels
        n = logits.shape[0]
        if n == 0:
            return []
        if len(params) != n or len(indices) != n:
            raise ValueError("one SamplingParams and one index per row of logits")
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        if all(p.greedy for p in params):
            kernels.argmax(logits, out)
        else:
            host = torch.tensor(
                [[p.temperature, float(p.topk), p.topp, uniform_for(p.seed, i)] for p, i in zip(params, indices)],
                dtype=torch.float32).t().contiguous()
            dev = host.to(self.device)
            kernels.sample(logits, dev[0], dev[1].to(torch.int32), dev[2], dev[3], out)
        return out.tolist()
