"""Sampling parameters and the per-batch sampler that drives the device kernels.

Options and their meaning are the reference's (`app_params`, application/llama/llama.cpp:20-41;
`Model::init`, include/model.h:38-39; algorithm `llama_sample_top_p_top_k`, src/utils.cpp:31-115):
temperature, top_k, top_p, repeat_penalty over the last `repeat_last_n` tokens (prompt
included, src/core/model_imp.cpp:25-28,72-73), seed.  Differences: temperature 0 means greedy
(the reference would divide by zero); random numbers come from a counter-based generator keyed
by (seed, request number, step), so a sequence's draws do not depend on what else is in its
batch (the reference has one `std::mt19937` for its one sequence).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..kernels import ops


@dataclass
class SamplingParams:
    temp: float = 0.0             # 0 = greedy
    top_k: int = 0                # 0 = off
    top_p: float = 1.0            # 1 = off
    repeat_penalty: float = 1.0   # 1 = off
    repeat_last_n: int = 64
    seed: int = 0

    def validate(self):
        if self.temp < 0:
            raise ValueError("temp must be >= 0")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        if self.repeat_penalty <= 0:
            raise ValueError("repeat_penalty must be > 0")
        if self.top_k < 0 or self.repeat_last_n < 0:
            raise ValueError("top_k and repeat_last_n must be >= 0")

    @property
    def greedy(self) -> bool:
        return self.temp == 0.0


def uniform_for(seed: int, request: int, step: int) -> float:
    """A float32 uniform number in [0, 1) from (seed, request, step): splitmix64 of the mixed key."""
    m = (1 << 64) - 1
    x = (seed * 0x9E3779B97F4A7C15 + request * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB
         + 0x2545F4914F6CDD1D) & m
    for _ in range(2):
        x = (x + 0x9E3779B97F4A7C15) & m
        z = x
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
        x = z ^ (z >> 31)
    return float(np.float32((x >> 40) / float(1 << 24)))


class Sampler:
    """Chooses one token per row of logits.  `histories[i]` is the list of tokens (prompt and
    generated) of row i's sequence, `requests[i]` its request number, `steps[i]` how many tokens
    it has generated so far."""

    def __init__(self, params: SamplingParams):
        params.validate()
        self.params = params

    def choose(self, logits: torch.Tensor, requests: Sequence[int], steps: Sequence[int],
               histories: Optional[Sequence[List[int]]] = None) -> torch.Tensor:
        p = self.params
        if p.greedy and p.repeat_penalty == 1.0:
            return ops.argmax(logits)
        B = logits.shape[0]
        last = None
        if p.repeat_penalty != 1.0 and p.repeat_last_n > 0 and histories is not None:
            arr = np.full((B, p.repeat_last_n), -1, dtype=np.int32)
            for i, h in enumerate(histories):
                tail = h[-p.repeat_last_n:]
                arr[i, :len(tail)] = tail
            last = torch.from_numpy(arr).to(logits.device)
        if p.greedy:
            # greedy with a repetition penalty: the penalised maximum; top_k = 1 keeps exactly it
            u = torch.zeros(B, dtype=torch.float32, device=logits.device)
            return ops.sample(logits, u, 1.0, 1, 1.0, p.repeat_penalty, last)
        u = torch.tensor([uniform_for(p.seed, r, s) for r, s in zip(requests, steps)],
                         dtype=torch.float32).to(logits.device)
        return ops.sample(logits, u, p.temp, p.top_k, p.top_p, p.repeat_penalty, last)
