"""The generation loop above the step function.

Requests (lists of token ids) are cut into batches that fit the cache; each batch starts
together: all prompts in one step, then one token per live sequence and step.  A sequence
ends at a stop token (which is kept in its output), at `max_new_tokens`, or when it has
filled the longest sequence the cache allows; it leaves the batch at once and its slot and
pages go back to the pools, where the next batch finds them.

The reference's loop is the command line's `while (get_remain_token() > 0) decode_iter`
(application/llama/llama.cpp:222-244) for its one sequence, ending a turn on token 2 (:237) and
the run when the context is full (`n_ctx - m_past`, src/core/model_imp.h:93); its timing sums
the wall time of the decode calls only (src/core/model_imp.cpp:56-59,133-142), as here.

The loop only needs `new_sequence`, `end_sequence`, `step` and `limits` of its backend and a
`choose` function, so its decisions are tested on the CPU with stand-ins for both.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from .step import Limits, StepItem


@dataclass
class GenerationResult:
    tokens: List[List[int]]                    # generated ids per request (stop token included)
    finish: List[str]                          # "stop" | "length" | "context"
    batches: List[List[int]]                   # which requests ran together
    prefill_tokens: int = 0
    prefill_s: float = 0.0
    decode_tokens: int = 0
    decode_s: float = 0.0
    decode_steps: int = 0
    step_s: List[float] = field(default_factory=list)    # wall time of every decode step, in order

    def summary(self) -> str:
        pf = self.prefill_tokens / self.prefill_s if self.prefill_s > 0 else 0.0
        dc = self.decode_tokens / self.decode_s if self.decode_s > 0 else 0.0
        return (f"prefill: {self.prefill_tokens} tokens in {self.prefill_s * 1e3:.1f} ms "
                f"({pf:.1f} tok/s); decode: {self.decode_tokens} tokens in {self.decode_steps} steps, "
                f"{self.decode_s * 1e3:.1f} ms ({dc:.1f} tok/s)")


class RequestTooLong(ValueError):
    pass


def plan_batches(prompt_lens: Sequence[int], max_new_tokens: int, limits: Limits) -> List[List[int]]:
    """Cut the requests, in order, into batches: at most `max_batch` sequences, and pages for
    every sequence's worst case (prompt + new tokens, capped by the longest sequence), so that
    a batch that has started never runs out of cache."""
    batches, cur, cur_pages = [], [], 0
    for i, n in enumerate(prompt_lens):
        if n <= 0:
            raise RequestTooLong(f"request {i}: the prompt is empty")
        if n > limits.max_seq_len:
            raise RequestTooLong(f"request {i}: prompt of {n} tokens exceeds the longest sequence "
                                 f"({limits.max_seq_len})")
        worst = min(n + max_new_tokens, limits.max_seq_len)
        pages = -(-worst // limits.page_size)
        if pages > limits.num_pages:
            raise RequestTooLong(f"request {i}: {worst} tokens need {pages} pages, the cache has "
                                 f"{limits.num_pages}")
        if cur and (len(cur) >= limits.max_batch or cur_pages + pages > limits.num_pages):
            batches.append(cur)
            cur, cur_pages = [], 0
        cur.append(i)
        cur_pages += pages
    if cur:
        batches.append(cur)
    return batches


def generate(backend, prompts: Sequence[Sequence[int]], choose: Callable, max_new_tokens: int,
             stop_ids: Sequence[int] = (), on_token: Optional[Callable] = None,
             clock: Callable = time.perf_counter) -> GenerationResult:
    """`choose(logits, requests, steps, histories)` returns one token per row of logits (any
    sequence of ints, or a tensor with `.tolist()`).  `on_token(request, token)` is called for
    every generated token."""
    limits: Limits = backend.limits()
    stop = set(int(s) for s in stop_ids)
    n = len(prompts)
    res = GenerationResult([[] for _ in range(n)], [""] * n,
                           plan_batches([len(p) for p in prompts], max_new_tokens, limits))
    if max_new_tokens <= 0:
        res.finish = ["length"] * n
        return res
    for batch in res.batches:
        slots = {r: backend.new_sequence() for r in batch}
        hist = {r: list(prompts[r]) for r in batch}
        live = _longest_first(batch, prompts)
        try:
            t0 = clock()
            logits = backend.step([StepItem(slots[r], list(prompts[r]), [len(prompts[r]) - 1])
                                   for r in live])
            toks = _as_list(choose(logits, live, [0] * len(live), [hist[r] for r in live]))
            res.prefill_s += clock() - t0
            res.prefill_tokens += sum(len(prompts[r]) for r in live)
            first = True
            while True:
                nxt = []
                for r, tok in zip(live, toks):
                    res.tokens[r].append(tok)
                    hist[r].append(tok)
                    if on_token:
                        on_token(r, tok)
                    if tok in stop:
                        res.finish[r] = "stop"
                    elif len(res.tokens[r]) >= max_new_tokens:
                        res.finish[r] = "length"
                    elif len(hist[r]) > limits.max_seq_len:
                        # the new token itself no longer fits the cache
                        res.finish[r] = "context"
                    else:
                        nxt.append(r)
                        continue
                    backend.end_sequence(slots.pop(r))
                if not first:
                    res.step_s.append(clock() - t0)
                    res.decode_s += res.step_s[-1]
                    res.decode_tokens += len(live)
                    res.decode_steps += 1
                first = False
                live = nxt
                if not live:
                    break
                t0 = clock()
                logits = backend.step([StepItem(slots[r], [hist[r][-1]], [0]) for r in live])
                toks = _as_list(choose(logits, live, [len(res.tokens[r]) for r in live],
                                       [hist[r] for r in live]))
        finally:
            for s in slots.values():
                backend.end_sequence(s)
    return res


def generate_pipelined(backend, prompts: Sequence[Sequence[int]], choose: Callable, max_new_tokens: int,
                       stop_ids: Sequence[int] = (), on_token: Optional[Callable] = None,
                       clock: Callable = time.perf_counter) -> GenerationResult:
    """The same loop with the host one step behind the device.  The sampled tokens stay on the
    device and feed the next step directly (`backend.step(..., device_ids=...)`); the host reads
    them only afterwards, while that next step already runs, so its own work (bookkeeping, packing
    and launching a step) no longer adds to the time per token.  A sequence that turns out to have
    sampled a stop token has then already been run one step too far: that step's result for it is
    dropped and its slot is freed, which changes nothing for the others (a sequence's logits do
    not depend on the rest of its batch).  `choose` gets the prompts as histories with the first
    call of a batch and None afterwards: a sampler that needs the last tokens (repetition penalty)
    keeps them itself from there (`sampling.Sampler` does, on the device)."""
    limits: Limits = backend.limits()
    stop = set(int(s) for s in stop_ids)
    n = len(prompts)
    res = GenerationResult([[] for _ in range(n)], [""] * n,
                           plan_batches([len(p) for p in prompts], max_new_tokens, limits))
    if max_new_tokens <= 0:
        res.finish = ["length"] * n
        return res
    for batch in res.batches:
        slots = {r: backend.new_sequence() for r in batch}
        n_fed = {r: len(prompts[r]) for r in batch}          # tokens of r that the cache holds
        try:
            t0 = clock()
            order = _longest_first(batch, prompts)
            logits = backend.step([StepItem(slots[r], list(prompts[r]), [len(prompts[r]) - 1]) for r in order])
            # (the prompts go with the first call: a sampler that penalises repetitions starts its
            # windows of last tokens from them and keeps them on the device from then on)
            pending, pending_toks = order, choose(logits, order, [0] * len(order),
                                                  [list(prompts[r]) for r in order])
            # the copy of the tokens to the host starts behind the sampling and is waited for by
            # itself, not by the stream (which by then holds the next step); `pending_sel` picks the
            # sequences that are still pending out of what was copied
            pending_read, pending_sel = _start_read(backend, pending_toks), None
            first = True
            while pending:
                # who goes on if the token just sampled is no stop token: decided by counts alone
                n_tok = {r: len(res.tokens[r]) + 1 for r in pending}
                cont = [r for r in pending if n_tok[r] < max_new_tokens and n_fed[r] + 1 <= limits.max_seq_len]
                nxt_toks = None
                if cont:
                    idx = [pending.index(r) for r in cont]
                    feed = pending_toks if len(cont) == len(pending) else pending_toks[idx]
                    logits = backend.step([StepItem(slots[r], [0], [0]) for r in cont], device_ids=feed)
                    for r in cont:
                        n_fed[r] += 1
                    nxt_toks = choose(logits, cont, [n_tok[r] for r in cont], None)
                nxt_read = _start_read(backend, nxt_toks) if nxt_toks is not None else None
                if pending_read is not None:                  # waits for the sampling before the step above
                    toks = pending_read()
                    toks = toks if pending_sel is None else [toks[i] for i in pending_sel]
                else:
                    toks = _as_list(pending_toks)
                now = clock()
                if first:
                    res.prefill_s += now - t0
                    res.prefill_tokens += sum(len(prompts[r]) for r in batch)
                    first = False
                else:
                    res.step_s.append(now - t0)
                    res.decode_s += now - t0
                    res.decode_tokens += len(pending)
                    res.decode_steps += 1
                t0 = now
                stopped = set()
                for r, tok in zip(pending, toks):
                    res.tokens[r].append(tok)
                    if on_token:
                        on_token(r, tok)
                    if tok in stop:
                        res.finish[r] = "stop"
                        stopped.add(r)
                    elif len(res.tokens[r]) >= max_new_tokens:
                        res.finish[r] = "length"
                    elif r not in cont:
                        res.finish[r] = "context"
                    else:
                        continue
                    backend.end_sequence(slots.pop(r))
                nxt_sel = None
                if stopped & set(cont):
                    keep = [i for i, r in enumerate(cont) if r not in stopped]
                    nxt_toks = nxt_toks[keep] if keep else None
                    nxt_sel = keep
                    cont = [cont[i] for i in keep]
                pending, pending_toks, pending_read, pending_sel = cont, nxt_toks, nxt_read, nxt_sel
        finally:
            for s in slots.values():
                backend.end_sequence(s)
    return res


def _longest_first(batch, prompts):
    """The requests of a batch in the order in which they are stepped: the longest prompt first
    (all grow by one token per step, so the order holds).  The attention kernels hand out their
    blocks in the order of the step's sequences, and the blocks with the most keys should start
    first; results are kept by request, so nothing else depends on the order."""
    return sorted(batch, key=lambda r: -len(prompts[r]))


def _start_read(backend, toks):
    """Begin the device-to-host copy of sampled tokens if the backend can do that apart from its
    stream (`read_tokens_async(toks)` returns a function that waits for that copy alone and gives
    the list); None otherwise."""
    f = getattr(backend, "read_tokens_async", None)
    return f(toks) if f is not None and toks is not None else None


def _as_list(toks):
    return [int(t) for t in (toks.tolist() if hasattr(toks, "tolist") else toks)]
