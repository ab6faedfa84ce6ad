"""The programming entry point, in the manner of the reference's `inferllm::Model`
(include/model.h:14-59): a `ModelConfig`, then `load`, `init`, `prefill`, `decode`,
`decode_iter`, `get_remain_token`, `reset_token`, `decode_summary`, with the same names and
meanings.  Differences that the scope of this library brings: prompts are lists of token ids
(there is no tokenizer here), the model folder holds config.json and safetensors, the model
class is chosen by config.json unless `model_name` names a registered one, and `generate`
adds batches of requests on top of the reference's single conversation.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import List, Optional, Sequence

from ..sampling import Sampler, SamplingParams
from .generate import GenerationResult, generate, generate_pipelined
from .step import Engine, EngineError, EngineOptions, StepItem


@dataclass
class ModelConfig:
    """Fields of the reference's ModelConfig (include/model.h:14-23).  `compt_type`:
    "bfloat16" or "float32"; `device_type` must be "gpu"; `nr_thread` and `enable_mmap` are
    accepted and have no effect (no CPU threads compute here, and weight files are always
    memory-mapped); `nr_ctx` is the longest sequence; `device_id` the GPU ordinal.
    `max_tokens` (not in the reference) sizes the cache for batches; default `nr_ctx`."""

    compt_type: str = "bfloat16"
    device_type: str = "gpu"
    nr_thread: int = 1
    nr_ctx: int = 2048
    device_id: int = 0
    enable_mmap: bool = True
    max_tokens: Optional[int] = None
    max_batch: Optional[int] = None


class Model:
    def __init__(self, config: ModelConfig, model_name: Optional[str] = None):
        if config.device_type.lower() not in ("gpu", "cuda"):
            raise EngineError(f"device_type '{config.device_type}' is not supported: this library "
                              "runs on one CUDA GPU only")
        self.config = config
        self.model_name = model_name
        self.engine: Optional[Engine] = None
        self.sampling = SamplingParams()
        self.end_token: Optional[int] = None
        self.end_tokens: List[int] = []
        self._slot: Optional[int] = None
        self._history: List[int] = []
        self._n_generated = 0
        self._pre_token: Optional[int] = None
        self._decode_s = 0.0
        self._decode_tokens = 0

    # ---- load / init

    def _options(self) -> EngineOptions:
        c = self.config
        return EngineOptions(dtype=c.compt_type, device_id=c.device_id,
                             max_tokens=c.max_tokens or c.nr_ctx, max_seq_len=c.nr_ctx,
                             max_batch=c.max_batch)

    def load(self, model_path: str) -> None:
        """Load config.json and the safetensors weights of a model folder."""
        self.engine = Engine.from_folder(model_path, self._options(), self.model_name)
        self._take_end_tokens()

    def load_random(self, config, seed: int = 0) -> None:
        """Random weights for a typed configuration, made on the device."""
        self.engine = Engine.from_config(config, self._options(), seed)
        self._take_end_tokens()

    def _take_end_tokens(self) -> None:
        """The configuration's end tokens: `end_token` is the first (the single number the
        reference's `init` takes), `end_tokens` all of them (config.json may list several)."""
        self.end_tokens = [int(t) for t in self.engine.model.spec.eos_token_ids]
        self.end_token = self.end_tokens[0] if self.end_tokens else None

    def init(self, top_k: int, top_p: float, temp: float, repeat_penalty: float,
             repeat_last_n: int, seed: int, end_token: int) -> None:
        """Sampling parameters of the conversation (include/model.h:38-39)."""
        if seed < 0:
            seed = int(time.time())
        self.sampling = SamplingParams(temp=temp, top_k=top_k, top_p=top_p,
                                       repeat_penalty=repeat_penalty, repeat_last_n=repeat_last_n,
                                       seed=seed)
        self.sampling.validate()
        self.end_token = end_token

    # ---- the single conversation of the reference's API

    def get_remain_token(self) -> int:
        used = self.engine.sequence_length(self._slot) if self._slot is not None else 0
        return self.engine.cache.max_seq_len - used

    def reset_token(self) -> None:
        if self._slot is not None:
            self.engine.end_sequence(self._slot)
        self._slot = None
        self._history = []
        self._n_generated = 0
        self._pre_token = None

    def prefill(self, prompt: Sequence[int]) -> None:
        """Run a prompt into the cache without producing a token (src/core/model_imp.cpp:22-34)."""
        if self._slot is None:
            self._slot = self.engine.new_sequence()
        self.engine.step([StepItem(self._slot, list(prompt), [])])
        self._history.extend(int(t) for t in prompt)

    def decode(self, user_input: Sequence[int]) -> int:
        """Run further input tokens and return the first answer token (:37-52)."""
        if self._slot is None:
            self._slot = self.engine.new_sequence()
        toks = list(user_input)
        logits = self.engine.step([StepItem(self._slot, toks, [len(toks) - 1])])
        self._history.extend(int(t) for t in toks)
        return self._sample(logits)

    def decode_iter(self) -> int:
        """Feed the previous answer token and return the next one (:55-64); timed."""
        if self._pre_token is None:
            raise EngineError("decode_iter needs a previous token: call decode first")
        t0 = time.perf_counter()
        logits = self.engine.step([StepItem(self._slot, [self._pre_token], [0])])
        tok = self._sample(logits)
        self._decode_s += time.perf_counter() - t0
        self._decode_tokens += 1
        return tok

    def _sample(self, logits) -> int:
        tok = int(Sampler(self.sampling).choose(logits, [0], [self._n_generated],
                                                [self._history]).tolist()[0])
        self._n_generated += 1
        self._history.append(tok)
        self._pre_token = tok
        return tok

    def decode_summary(self) -> str:
        """Totals in the reference's wording (src/core/model_imp.cpp:133-142)."""
        per = self._decode_s * 1e3 / self._decode_tokens if self._decode_tokens else 0.0
        rate = self._decode_tokens / self._decode_s if self._decode_s > 0 else 0.0
        return (f"Run Model Summary:\nTotal Model Compute Time:   {self._decode_s:.3f}s\n"
                f"Total Model Compute Token:  {self._decode_tokens}\n"
                f"Average Token Compute Time: {per:.3f}ms\n"
                f"Average Token Generation Speed: {rate:.3f}token/s\n")

    def warm_up(self, prompt_tokens: int = 0, batch_sizes: Sequence[int] = ()) -> None:
        """Before the first request: run what costs extra the first time (see `Engine.warm_up`)."""
        self.engine.warm_up(prompt_tokens, batch_sizes)

    # ---- batches of requests

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 128,
                 stop_ids: Optional[Sequence[int]] = None, on_token=None) -> GenerationResult:
        """Generate for many requests.  `stop_ids` default to the end token given to `init`; where
        that is one of the configuration's end tokens (or `init` was given none), to all of them:
        the reference ends a turn on its one end token (application/llama/llama.cpp:237), a
        config.json may name several."""
        if stop_ids is None:
            if self.end_token is None or self.end_token in self.end_tokens:
                stop_ids = list(self.end_tokens)
            else:
                stop_ids = [self.end_token]
        sampler = Sampler(self.sampling)
        # the loop that keeps the host one step behind the device; the sampler keeps the windows of
        # last tokens for the repetition penalty on the device
        res = generate_pipelined(self.engine, prompts, sampler.choose, max_new_tokens, stop_ids, on_token)
        self.engine.check_device_errors()
        return res
