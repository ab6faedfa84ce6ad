"""The engine: a model, its cache, and the one step function that everything else drives.

`Engine.step(items)` runs the tokens it is given, as one batch, from the cache that earlier
steps left, and returns the float32 logits at the wanted places.  A step may hold prompts of
unequal lengths (all their tokens at once), single next tokens, or both; a sequence's start
position is the cache's own record of its length.  The generation loop, the command line, the
Python entry point and `bin/trace_run` all go through this function.

The reference's counterpart is `Graph::execute(tokens, logits, nr_past, prefill)`
(src/core/graph.cpp:166-197): one sequence, the caller passes the past length, logits of the
last token only or none at all.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheError, SequenceCache
from ..kernels import ops
from ..parts.base import Runtime
from ..registry import config_from_folder, get_architecture
from ..weights import init_random_weights, load_model_weights

PROMPT_BUCKET = 64                # tokens; also the rows the library's products are rounded up to
PROMPT_GRAPH_MAX_TOKENS = 1024    # longer prompts keep the GPU busy longer than the host needs to issue them

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32}


class EngineError(RuntimeError):
    pass


@dataclass
class EngineOptions:
    dtype: str = "bfloat16"        # "bfloat16": serving kernels; "float32": everything in true 32-bit
    device_id: int = 0
    max_tokens: Optional[int] = 4096    # tokens that live sequences may hold together (sizes the cache);
                                        # None: what `mem_fraction` of the memory left beside the weights holds
    mem_fraction: float = 0.9
    max_seq_len: Optional[int] = None   # longest sequence; default the model's max positions
    max_batch: Optional[int] = None     # slots; default max_tokens / page_size
    page_size: int = 64
    cuda_graphs: bool = True       # replay one-token-per-sequence steps from captured CUDA graphs
    gemm: str = "auto"             # bfloat16 products: "auto" | "tc" | "library" (see kernels.ops.set_gemm_backend)
    poison_freed_pages: bool = False    # fill pages that go back to the pool with NaN (a check, not for serving)


@dataclass
class Limits:
    max_batch: int      # sequences that can be live together (slots)
    num_pages: int      # pages of the cache
    page_size: int
    max_seq_len: int


@dataclass
class StepItem:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)  # places among `tokens` whose logits are asked for


class StepContext:
    """Device-side description of one step, shared by all parts.

    ids, token_pos, token_seq : int32 [T]   token id, absolute position, index of its sequence
    want_rows : int32 [K]   rows (among the T tokens) whose logits are wanted
    slots, seq_lens, cu_q : int32 [B], [B], [B+1]   slot, length after the step, token offsets
    """

    def __init__(self, engine, plan, ids_host, want_rows_host, into=None):
        """`into`: a device buffer of an earlier step of the same shape to fill again (the
        static input of a captured graph); None uploads into a fresh buffer."""
        cache = engine.cache
        B = len(plan.slots)
        q = np.asarray(plan.q_lens, dtype=np.int32)
        past = np.asarray(plan.past, dtype=np.int32)
        T = int(q.sum())
        if T == B:                       # one token per sequence: no arithmetic needed
            cu = np.arange(B + 1, dtype=np.int32)
            token_seq, token_pos = cu[:-1], past
        else:
            cu = np.zeros(B + 1, dtype=np.int32)
            np.cumsum(q, out=cu[1:])
            token_seq = np.repeat(np.arange(B, dtype=np.int32), q)
            token_pos = np.arange(T, dtype=np.int32) - np.repeat(cu[:-1], q) + np.repeat(past, q)
        parts = [np.asarray(ids_host, dtype=np.int32), token_pos, token_seq,
                 np.asarray(want_rows_host, dtype=np.int32), np.asarray(plan.slots, dtype=np.int32),
                 past + q, cu] + [t.reshape(-1) for t in plan.tables]
        offs, total = [], 0
        for p in parts:
            offs.append(total)
            total += (p.size + 3) // 4 * 4  # keep every array 16-byte aligned
        buf = engine._upload(parts, offs, total, into)
        self.buffer = buf

        def view(i):
            return buf[offs[i]:offs[i] + parts[i].size]

        self.T, self.B = T, B
        self.ids, self.token_pos, self.token_seq = view(0), view(1), view(2)
        self.want_rows, self.slots, self.seq_lens, self.cu_q = view(3), view(4), view(5), view(6)
        self.tables = [view(7 + i).view(B, cache.width) for i in range(len(plan.tables))]
        self.q_lens, self.past = list(plan.q_lens), list(plan.past)
        self.max_q = int(q.max())
        self.max_len = int((past + q).max())
        self.is_decode = self.max_q == 1
        self.max_seq_len = cache.max_seq_len
        self.err = engine.err
        self._cache = cache

    def cache_view(self, entry: int, writes: bool = True):
        if entry not in self._cache.where:
            return None
        kind, gi = self._cache.group_of(entry)
        if kind == "kv":
            view = self._cache.kv_view(entry, self.tables[gi])
            view.writes = writes
            return view
        return self._cache.state_view(entry, self.slots)


class Engine:
    def __init__(self, config, options: EngineOptions):
        if options.dtype not in _DTYPES:
            raise EngineError(f"dtype '{options.dtype}' is not supported (bfloat16 or float32)")
        self.config = config
        self.options = options
        self.rt = self._make_runtime(options)
        dev = self.rt.device
        self.model = get_architecture(config.architecture).build_model(config, self.rt)
        spec = self.model.spec
        self.vocab_size = spec.vocab_size
        max_seq = min(options.max_seq_len or spec.max_positions, spec.max_positions)
        ps = options.page_size
        max_tokens = options.max_tokens
        if max_tokens is None:
            max_tokens = self._tokens_that_fit(options.mem_fraction)
        num_pages = max(1, -(-max_tokens // ps))
        num_slots = options.max_batch or num_pages
        self.cache = SequenceCache(self.model.cache_requests(), num_slots, num_pages, ps, max_seq,
                                   self.rt, poison_freed_pages=options.poison_freed_pages)
        if options.poison_freed_pages:          # pages that no sequence has held yet are as foreign as freed ones
            for g in self.cache.paged:
                g.k.fill_(float("nan"))
                g.v.fill_(float("nan"))
        self.err = torch.zeros(1, dtype=torch.int32, device=dev)
        self._stages = [(None, None, None)] * 4    # (pinned tensor, its numpy view, copy-done event)
        self._tok_bufs, self._tok_next = [None] * 4, 0   # pinned buffers for sampled tokens on their way to the host
        self._stage_next = 0
        self._graphs = {}
        self._pad_safe = None          # whether single prompts may be padded and replayed (asked once)
        self._graphs_backend = None    # `kernels.ops.gemm_backend()` when the graphs were captured
        self._graph_pool = None
        self.loaded = False

    def _tokens_that_fit(self, fraction: float) -> int:
        """How many tokens of cache fit into `fraction` of the device memory that is free now and not
        needed for the weights (which are loaded after the cache is made)."""
        from ..parts.base import PagedKV
        elem = 4 if self.rt.is_f32 else 2
        weights = 0
        for decl in self.model.tensor_decls().values():
            n = 1
            for d in decl.shape:
                n *= int(d)
            weights += n * elem
        per_token = sum(2 * r.n_kv_heads * r.head_dim * elem for r in self.model.cache_requests().values()
                        if isinstance(r, PagedKV))
        free, _ = torch.cuda.mem_get_info(self.rt.device)
        room = int((free - weights) * fraction)
        if per_token == 0:
            return self.options.page_size
        if room < per_token * self.options.page_size:
            raise EngineError(f"the weights ({weights / 2**30:.1f} GiB) leave no room for a cache on this device "
                              f"({free / 2**30:.1f} GiB free)")
        return room // per_token

    def _make_runtime(self, options: EngineOptions) -> Runtime:
        if not torch.cuda.is_available():
            raise EngineError("inferllm_b200 needs a CUDA device: there is no CPU path")
        from ..kernels.lib import load
        load()  # fail here, loudly, if the kernels cannot be built or loaded
        ops.set_gemm_backend(options.gemm)
        dev = torch.device("cuda", options.device_id)
        torch.cuda.set_device(dev)
        return Runtime(dev, _DTYPES[options.dtype], options.page_size)

    # ---- construction

    @classmethod
    def from_folder(cls, folder: str, options: EngineOptions, model_name: Optional[str] = None):
        eng = cls(config_from_folder(folder, model_name), options)
        load_model_weights(eng.model, folder)
        eng.loaded = True
        return eng

    @classmethod
    def from_config(cls, config, options: EngineOptions, seed: int = 0):
        """Random weights made on the device, without a file."""
        eng = cls(config, options)
        init_random_weights(eng.model, seed)
        eng.loaded = True
        return eng

    # ---- sequences

    def new_sequence(self) -> int:
        return self.cache.alloc_slot()

    def end_sequence(self, slot: int) -> None:
        self.cache.free_slot(slot)

    def sequence_length(self, slot: int) -> int:
        return self.cache.seq_len[slot]

    def limits(self) -> Limits:
        c = self.cache
        return Limits(c.num_slots, c.num_pages, c.page_size, c.max_seq_len)

    # ---- the step

    def _upload(self, parts, offs, total: int, into=None) -> torch.Tensor:
        """One asynchronous copy for all of a step's index arrays, from a small ring of pinned
        staging buffers: the host may prepare the next steps while the GPU still runs this one,
        and waits only when it comes back to a buffer whose copy has not left yet."""
        slot = self._stage_next
        self._stage_next = (slot + 1) % len(self._stages)
        stage, stage_np, busy = self._stages[slot]
        if busy is not None:
            busy.synchronize()
        if stage is None or stage.numel() < total:
            stage = torch.empty(max(total, 4096), dtype=torch.int32, pin_memory=True)
            stage_np = stage.numpy()      # the same pinned memory, for cheap fills
        for o, p in zip(offs, parts):
            stage_np[o:o + p.size] = p
        buf = into if into is not None else torch.empty(total, dtype=torch.int32, device=self.rt.device)
        buf.copy_(stage[:total], non_blocking=True)
        self.last_upload_bytes = 4 * total
        busy = torch.cuda.Event()
        busy.record()
        self._stages[slot] = (stage, stage_np, busy)
        return buf

    def step(self, items: Sequence[StepItem], device_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run one step; returns float32 logits [number of wanted places, vocab] on the device,
        in the order of the items and of each item's `want`.

        `device_ids` (int32 tensor on the device, one id per item) gives the tokens of a
        one-token-per-sequence step without a round trip through the host, e.g. straight from the
        sampling kernel; the items' `tokens` are then placeholders of length one."""
        if not self.loaded:
            raise EngineError("the model has no weights yet")
        if not items:
            raise EngineError("a step needs at least one sequence")
        if ops.gemm_backend() != self._graphs_backend:
            # the choice of product kernels is process-wide and part of what a graph captured
            self._graphs, self._graphs_backend = {}, ops.gemm_backend()
        ids, want_rows, off = [], [], 0
        for it in items:
            n = len(it.tokens)
            if n == 0:
                raise EngineError(f"slot {it.slot}: a step must bring at least one token")
            for t in it.tokens:
                if not 0 <= int(t) < self.vocab_size:
                    raise EngineError(f"slot {it.slot}: token id {t} is outside the vocabulary "
                                      f"[0, {self.vocab_size})")
            for w in it.want:
                if not 0 <= int(w) < n:
                    raise EngineError(f"slot {it.slot}: wanted place {w} is outside its {n} tokens")
                want_rows.append(off + int(w))
            ids.extend(int(t) for t in it.tokens)
            off += n
        if device_ids is not None and (len(ids) != len(items) or device_ids.numel() != len(items)
                                       or device_ids.dtype != torch.int32):
            raise EngineError("device_ids needs one int32 id per item and items of one token each")
        if (self.options.cuda_graphs and len(items) == 1 and 1 < len(ids) <= PROMPT_GRAPH_MAX_TOKENS
                and self._pads_prompts()):
            logits = self._prompt_step_graphed(items[0].slot, ids, want_rows)
            if logits is not None:
                return logits
        plan = self.cache.plan_step([it.slot for it in items], [len(it.tokens) for it in items])
        if self.options.cuda_graphs and len(ids) == len(items) and self.model.graph_safe():
            logits = self._decode_step_graphed(plan, ids, want_rows, device_ids)
        else:
            ctx = StepContext(self, plan, ids, want_rows)
            if device_ids is not None:
                ctx.ids.copy_(device_ids)
            logits = self.model.forward(ctx)
        self.cache.commit_step(plan)
        return logits

    def _pads_prompts(self) -> bool:
        if self._pad_safe is None:
            self._pad_safe = bool(self.model.pad_safe())
        return self._pad_safe

    def _prompt_step_graphed(self, slot: int, ids, want_rows) -> Optional[torch.Tensor]:
        """A single prompt (or a further piece of one sequence) of up to 1,024 tokens: the host needs
        longer to issue the step's launches than the GPU to run them, so the step is padded to whole
        buckets of 64 tokens, with tokens behind the real ones that no real token sees (what they
        leave in the sequence's pages lies behind its length and is overwritten by the tokens that
        follow), and the launches of a bucket are captured in a CUDA graph the second time it is
        seen.  Only where the padding needs no page that the step would not need anyway and stays
        within the longest sequence; None otherwise (the caller then runs the step as it is).  The
        logits of the real tokens do not depend on the padding beyond rounding, and in float32 not
        at all."""
        c = self.cache
        T = len(ids)
        padded = -(-T // PROMPT_BUCKET) * PROMPT_BUCKET
        past = c.seq_len[slot] if c.slots.is_held(slot) else 0
        if not c.slots.is_held(slot) or past + padded > c.max_seq_len:
            return None
        if any(g.ledger.pages_needed(slot, past + padded) != g.ledger.pages_needed(slot, past + T) for g in c.paged):
            return None
        plan = c.plan_step([slot], [padded])
        ids = list(ids) + [0] * (padded - T)
        key = ("prompt", padded, len(want_rows))
        entry = self._graphs.get(key)
        if entry is None or entry == "seen":
            ctx = StepContext(self, plan, ids, want_rows)
            if entry is None:
                self._graphs[key] = "seen"
                out = self.model.forward(ctx)
            else:
                if len(self._graphs) > 64:
                    self._graphs = {k: v for k, v in self._graphs.items() if v == "seen"}
                torch.cuda.current_stream().synchronize()
                graph = torch.cuda.CUDAGraph()
                before = ops.launch_count()
                with torch.cuda.graph(graph, pool=self._graph_pool):
                    out = self.model.forward(ctx)
                launches = ops.launch_count() - before
                if self._graph_pool is None:
                    self._graph_pool = graph.pool()
                self._graphs[key] = (graph, ctx, out, launches)
                graph.replay()
                out = out.clone()
        else:
            graph, ctx, out, launches = entry
            StepContext(self, plan, ids, want_rows, into=ctx.buffer)
            graph.replay()
            ops.count_launches(launches)
            out = out.clone()
        plan.q_lens = [T]               # the sequence grows by its real tokens only
        c.commit_step(plan)
        return out

    def _decode_step_graphed(self, plan, ids, want_rows, device_ids=None) -> torch.Tensor:
        """One token per sequence: the launches of such a step are the same every time (all that
        changes lies in device memory), so the step is captured in a CUDA graph the second time
        a batch size is seen and replayed from then on.  The logits of a replayed step are
        copied out of the graph's own output buffer, so they stay valid."""
        key = (len(ids), tuple(want_rows))
        entry = self._graphs.get(key)
        if entry is None:
            self._graphs[key] = "seen"
            ctx = StepContext(self, plan, ids, want_rows)
            if device_ids is not None:
                ctx.ids.copy_(device_ids)
            return self.model.forward(ctx)
        if entry == "seen":
            if len(self._graphs) > 64:
                self._graphs = {k: v for k, v in self._graphs.items() if v == "seen"}
            ctx = StepContext(self, plan, ids, want_rows)
            if device_ids is not None:
                ctx.ids.copy_(device_ids)
            torch.cuda.current_stream().synchronize()
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                out = self.model.forward(ctx)
            launches = ops.launch_count() - before
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            self._graphs[key] = (graph, ctx, out, launches)
            graph.replay()
            return out.clone()
        graph, ctx, out, launches = entry
        StepContext(self, plan, ids, want_rows, into=ctx.buffer)
        if device_ids is not None:
            ctx.ids.copy_(device_ids)
        graph.replay()
        ops.count_launches(launches)
        return out.clone()

    def read_tokens_async(self, toks: torch.Tensor):
        """Start copying sampled token ids (int32, on the device) to pinned host memory behind
        what the stream holds now; the returned function waits for that copy alone, not for work
        queued later, and gives the ids as a list."""
        n = int(toks.numel())
        slot = self._tok_next
        self._tok_next = (slot + 1) % len(self._tok_bufs)
        buf = self._tok_bufs[slot]
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 256), dtype=torch.int32, pin_memory=True)
            self._tok_bufs[slot] = buf
        buf[:n].copy_(toks.reshape(-1), non_blocking=True)
        done = torch.cuda.Event()
        done.record()

        def result():
            done.synchronize()
            return buf[:n].tolist()
        return result

    def warm_up(self, prompt_tokens: int = 0, batch_sizes: Sequence[int] = ()) -> None:
        """Pay what is paid once, before the first request: prompt steps for every bucket of 64
        tokens up to `prompt_tokens` (the library chooses its kernels per shape of a product, about
        10 ms each at 7B size; the second step of a bucket of up to 1,024 tokens captures its CUDA
        graph), and for every batch size three one-token steps, of which the second captures the
        graph that later steps of that size replay.  Uses free slots and pages
        only and gives them back; sizes that do not fit the cache are left out."""
        lim = self.limits()
        longest = min(int(prompt_tokens), lim.max_seq_len, lim.num_pages * lim.page_size)
        for n in range(ops.LIBRARY_ROW_BUCKET, longest + 1, ops.LIBRARY_ROW_BUCKET):
            try:
                for _ in range(2 if n <= PROMPT_GRAPH_MAX_TOKENS else 1):     # the second sight of a bucket captures its graph
                    slot = self.new_sequence()
                    try:
                        self.step([StepItem(slot, [0] * n, [n - 1])])
                    finally:
                        self.end_sequence(slot)
            except CacheError:              # live sequences hold the pages: no larger size fits either
                break
        for b in batch_sizes:
            if b < 1 or b > lim.max_batch or b > lim.num_pages or self.cache.slots.n_free < b:
                continue
            slots = [self.new_sequence() for _ in range(b)]
            try:
                self.step([StepItem(s, [0], [0]) for s in slots])
                for _ in range(3):
                    self.step([StepItem(s, [0], [0]) for s in slots])
            finally:
                for s in slots:
                    self.end_sequence(s)
        torch.cuda.current_stream().synchronize()

    def check_device_errors(self) -> None:
        """Read the kernels' error word (synchronises)."""
        code = int(self.err.item())
        tc = ops.tc_error_word(self.rt.device)
        tc_code = int(tc.item())
        if tc_code:
            tc.zero_()
            family = {4: "a wait inside the tensor-core matrix product (gemm_tc, gemm_tc2) timed out",
                      5: "a wait inside the tensor-core prompt attention (attention_prefill_tc) timed out",
                      6: "a tensor-core kernel found its shared memory misaligned and did not run",
                      7: "a wait inside the decode attention (attention_decode_ring) timed out"}
            raise EngineError(family.get(tc_code, f"a tensor-core kernel reported error {tc_code}")
                              + ": the step's results are not valid")
        if code:
            self.err.zero_()
            what = {1: "a token id outside the embedding table", 2: "a cache write to a page that "
                    "the sequence does not hold", 3: "a position beyond the position table"}
            raise EngineError("a kernel reported " + what.get(code, f"error {code}"))
