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
    it has generated so far.

    For the repetition penalty the sampler needs each sequence's last `repeat_last_n` tokens.  A
    loop that has them on the host passes `histories` with every call.  A loop that keeps the
    sampled tokens on the device (`generate_pipelined`) passes the prompts as `histories` with the
    first call of a batch (all `steps` 0) and None afterwards: the sampler then keeps the windows
    on the device itself, one row per request, and writes every token it samples into them (the
    sequences of a batch advance together, so the oldest entry of every row is at the same place)."""

    def __init__(self, params: SamplingParams):
        params.validate()
        self.params = params
        self._window = None          # int32 [requests of the batch, repeat_last_n] on the device
        self._row_of = {}            # request -> its row of the window
        self._u_ring, self._u_next = [None] * 4, 0     # pinned staging for the uniform numbers

    def _uniforms(self, requests, steps, device):
        """The step's uniform numbers on the device, through pinned memory and a copy that does not
        make the host wait for the work already queued (a copy from pageable memory would)."""
        n = len(requests)
        slot = self._u_next
        self._u_next = (slot + 1) % len(self._u_ring)
        buf = self._u_ring[slot]
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 64), dtype=torch.float32, pin_memory=(device.type == "cuda"))
            self._u_ring[slot] = buf
        view = buf.numpy()
        for i, (r, st) in enumerate(zip(requests, steps)):
            view[i] = uniform_for(self.params.seed, r, st)
        return buf[:n].to(device, non_blocking=True)

    def _wants_history(self) -> bool:
        return self.params.repeat_penalty != 1.0 and self.params.repeat_last_n > 0

    def _start_windows(self, requests, histories, device):
        n = self.params.repeat_last_n
        arr = np.full((len(requests), n), -1, dtype=np.int32)
        for i, h in enumerate(histories):
            tail = list(h[-n:])
            if tail:
                arr[i, n - len(tail):] = tail          # oldest first: entry 0 is the first to be replaced
        self._window = torch.from_numpy(arr).to(device)
        self._row_of = {r: i for i, r in enumerate(requests)}

    def choose(self, logits: torch.Tensor, requests: Sequence[int], steps: Sequence[int],
               histories: Optional[Sequence[List[int]]] = None) -> torch.Tensor:
        p = self.params
        if p.greedy and p.repeat_penalty == 1.0:
            return ops.argmax(logits)
        B = logits.shape[0]
        last, on_device, rows = None, False, None
        if self._wants_history():
            if histories is not None and all(s == 0 for s in steps) and len(set(steps)) <= 1:
                # (also what a host-side loop passes at its first step: the windows then simply
                # mirror what it keeps passing)
                self._start_windows(requests, histories, logits.device)
            if histories is not None:
                arr = np.full((B, p.repeat_last_n), -1, dtype=np.int32)
                for i, h in enumerate(histories):
                    tail = h[-p.repeat_last_n:]
                    arr[i, :len(tail)] = tail
                last = torch.from_numpy(arr).to(logits.device)
            elif self._window is not None and all(r in self._row_of for r in requests):
                idx = [self._row_of[r] for r in requests]
                rows = None if idx == list(range(self._window.shape[0])) else torch.tensor(idx, device=logits.device)
                last = self._window if rows is None else self._window[rows]
                on_device = True
        if p.greedy:
            # greedy with a repetition penalty: the penalised maximum; top_k = 1 keeps exactly it
            u = torch.zeros(B, dtype=torch.float32, device=logits.device)
            toks = ops.sample(logits, u, 1.0, 1, 1.0, p.repeat_penalty, last)
        else:
            u = self._uniforms(requests, steps, logits.device)
            toks = ops.sample(logits, u, p.temp, p.top_k, p.top_p, p.repeat_penalty, last)
        if self._wants_history() and self._window is not None and (on_device or histories is not None) \
                and all(r in self._row_of for r in requests):
            # the new token takes the place of the window's oldest entry
            col = int(steps[0]) % p.repeat_last_n
            if rows is None and len(requests) == self._window.shape[0]:
                self._window[:, col] = toks
            else:
                idx = rows if rows is not None else torch.tensor([self._row_of[r] for r in requests],
                                                                 device=logits.device)
                self._window[idx, col] = toks
        return toks
