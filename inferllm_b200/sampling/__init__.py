"""Sampling as Python sees it: the parameters, the counter-based uniform numbers and a face of the
device sampler (`sampling/sampler.h`)."""
from __future__ import annotations

import ctypes
import json
from dataclasses import asdict, dataclass
from typing import List, Optional, Sequence

from .. import binding as _b


@dataclass
class SamplingParams:
    temp: float = 0.0             # 0 = greedy
    top_k: int = 0                # 0 = off
    top_p: float = 1.0            # 1 = off
    repeat_penalty: float = 1.0   # 1 = off
    repeat_last_n: int = 64
    seed: int = 0

    def validate(self):
        _b.check(_b.lib().illm_sampling_params_validate(json.dumps(asdict(self)).encode()))

    @property
    def greedy(self) -> bool:
        return self.temp == 0.0


def uniform_for(seed: int, request: int, step: int) -> float:
    """A float32 uniform number in [0, 1) from (seed, request, step)."""
    return float(_b.lib().illm_uniform_for(seed, request, step))


class Sampler:
    """Chooses one token per row of float32 logits on the device (a torch tensor [B, V]); returns an
    int32 torch tensor [B].  See `sampling/sampler.h` for `histories`."""

    def __init__(self, engine, params: SamplingParams):
        params.validate()
        self.params = params
        self._engine = engine
        out = ctypes.c_void_p()
        _b.check(_b.lib().illm_sampler_create(engine._ptr, json.dumps(asdict(params)).encode(), ctypes.byref(out)))
        self._ptr = out
        engine._adopt(self)

    def _free(self) -> None:
        # (the sampler's buffers live on the engine's device: once the engine is gone they are gone too,
        # and the library's object must not be touched any more)
        engine = getattr(self, "_engine", None)
        if getattr(self, "_ptr", None) and _b._lib is not None and engine is not None and engine._ptr:
            _b._lib.illm_sampler_free(self._ptr)
        self._ptr = None

    def __del__(self):
        self._free()

    def choose(self, logits, requests: Sequence[int], steps: Sequence[int], histories: Optional[Sequence[List[int]]] = None):
        import torch
        B, V = logits.shape
        lens = hist = None
        if histories is not None:
            lens = _b.ints(len(h) for h in histories)
            hist = _b.ints(t for h in histories for t in h)
        if not self._ptr:
            raise _b.EngineError("the sampler's engine is gone")
        out = ctypes.c_void_p()
        self._engine.order(0)           # the sampler works on the engine's stream: it waits for the logits
        _b.check(_b.lib().illm_sampler_choose(self._ptr, logits.data_ptr(), B, V, _b.ints(requests), _b.ints(steps), lens, hist,
                                              ctypes.byref(out)))
        self._engine.order(1)
        toks = torch.empty(B, dtype=torch.int32, device=logits.device)
        self._engine._copy(toks.data_ptr(), out.value, 4 * B)
        return toks
