"""The cache of a model: a slot per sequence, paged keys and values per group of layers,
and per-sequence state of fixed size.

Layers ask for storage through their mixer's `cache_request()`: `PagedKV(n_kv_heads,
head_dim, window)` or `FixedState(shape, dtype)`.  Cache entries (one per writing entry of
the model's schedule) with equal requests form a group; every group has storage, a page
pool and page tables of its own, so groups with different needs (all keys, a window of
them, another head size) live side by side.  Device storage of a paged group:
`k, v : [entries, pages, kv heads, page_size, head_dim]` in the runtime's dtype; of a state
group: `[entries, slots, *shape]`.

Life of a sequence: `alloc_slot()` (state zeroed) -> `plan_step()` / `commit_step()` once per
step (pages are reserved before the step runs and the length advances after it) ->
`free_slot()` (pages and slot go back to the pools for the next sequence).

The reference's counterpart is `KvStorage` (src/core/kvstorage.h:9-54): one sequence, one
contiguous float32 tensor per layer, length checked against the caller's `nr_past`
(src/core/op.cpp:349-351).  Here the length is the cache's own and the caller passes none.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np

from ..parts.base import FixedState, PagedKV
from .pools import CacheError, CacheFull, IndexPool, PageLedger


@dataclass
class KVView:
    """What an attention mixer sees of its cache entry during one step."""

    k: object               # [pages, kv heads, page_size, head_dim]
    v: object
    block_table: object     # int32 [B, width] on the device, rows in the order of the step's sequences
    page_size: int
    window: Optional[int]
    writes: bool = True


@dataclass
class StateView:
    """What a mixer with fixed-size state sees: its storage [slots, *shape] and the slots of
    the step's sequences (int32 [B] on the device)."""

    state: object
    slots: object


class _PagedGroup:
    def __init__(self, request: PagedKV, entries: List[int], num_pages, page_size, num_slots):
        self.request = request
        self.entries = entries
        self.ledger = PageLedger(num_pages, page_size, num_slots, request.window)
        self.k = self.v = None

    def allocate(self, runtime):
        import torch
        r = self.request
        shape = (len(self.entries), self.ledger.pool.n, r.n_kv_heads, self.ledger.page_size, r.head_dim)
        self.k = torch.zeros(shape, dtype=runtime.dtype, device=runtime.device)
        self.v = torch.zeros(shape, dtype=runtime.dtype, device=runtime.device)

    def bytes(self, elem_size):
        r = self.request
        return 2 * len(self.entries) * self.ledger.pool.n * r.n_kv_heads * self.ledger.page_size * r.head_dim * elem_size


class _StateGroup:
    def __init__(self, request: FixedState, entries: List[int], num_slots):
        self.request = request
        self.entries = entries
        self.num_slots = num_slots
        self.state = None

    def allocate(self, runtime):
        import torch
        self.state = torch.zeros((len(self.entries), self.num_slots, *self.request.shape),
                                 dtype=self.request.dtype, device=runtime.device)


@dataclass
class StepPlan:
    slots: List[int]
    q_lens: List[int]
    past: List[int]                    # length of each sequence before the step
    tables: List[np.ndarray]           # per paged group: int32 [B, width]


class SequenceCache:
    def __init__(self, requests: Dict[int, object], num_slots: int, num_pages: int, page_size: int,
                 max_seq_len: int, runtime=None, poison_freed_pages: bool = False):
        """`requests`: cache entry number -> PagedKV | FixedState | None.  `runtime=None` keeps
        the cache host-only (bookkeeping without device storage).  `poison_freed_pages`: pages that
        go back to the pool are filled with NaN on the device, so that a kernel that reads a page
        its sequence does not hold shows it."""
        self.poison_freed_pages = bool(poison_freed_pages)
        if num_slots <= 0 or num_pages <= 0 or page_size <= 0:
            raise CacheError("num_slots, num_pages and page_size must be positive")
        self.num_slots, self.num_pages, self.page_size = int(num_slots), int(num_pages), int(page_size)
        self.max_seq_len = int(max_seq_len)
        self.width = -(-self.max_seq_len // self.page_size)  # columns of a page table
        self.slots = IndexPool(num_slots, "slot")
        self.seq_len = [0] * num_slots
        self.paged: List[_PagedGroup] = []
        self.states: List[_StateGroup] = []
        self.where: Dict[int, tuple] = {}  # entry -> ("kv"|"state", group index, index in group)
        by_req: Dict[object, object] = {}
        for entry in sorted(requests):
            req = requests[entry]
            if req is None:
                continue
            if isinstance(req, PagedKV):
                g = by_req.get(req)
                if g is None:
                    g = by_req[req] = _PagedGroup(req, [], num_pages, page_size, num_slots)
                    self.paged.append(g)
                self.where[entry] = ("kv", self.paged.index(g), len(g.entries))
            elif isinstance(req, FixedState):
                g = by_req.get(req)
                if g is None:
                    g = by_req[req] = _StateGroup(req, [], num_slots)
                    self.states.append(g)
                self.where[entry] = ("state", self.states.index(g), len(g.entries))
            else:
                raise CacheError(f"cache entry {entry}: unknown kind of request {req!r}")
            g.entries.append(entry)
        self.runtime = runtime
        if runtime is not None:
            self._check_fits(runtime)
            for g in self.paged + self.states:
                g.allocate(runtime)

    def _check_fits(self, runtime) -> None:
        """Refuse a cache that the device cannot hold, in words, before any allocation."""
        import torch
        if runtime.device.type != "cuda":
            return
        elem = torch.empty((), dtype=runtime.dtype).element_size()
        need = sum(g.bytes(elem) for g in self.paged)
        free, _ = torch.cuda.mem_get_info(runtime.device)
        free += torch.cuda.memory_reserved(runtime.device) - torch.cuda.memory_allocated(runtime.device)
        if need > free:
            tokens = max((g.ledger.pool.n * g.ledger.page_size for g in self.paged), default=0)
            raise CacheError(f"a cache for {tokens} tokens needs {need / 2**30:.1f} GiB, the device has "
                             f"{free / 2**30:.1f} GiB free: ask for fewer tokens (max_tokens)")

    # ---- slots

    def alloc_slot(self) -> int:
        (slot,) = self.slots.alloc(1)
        self.seq_len[slot] = 0
        for g in self.states:
            if g.state is not None:
                g.state[:, slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} freed twice (or never handed out)")
        for g in self.paged:
            self._poison(g, g.ledger.release_all(slot))
        self.seq_len[slot] = 0
        self.slots.free([slot])

    def _poison(self, group, pages) -> None:
        if self.poison_freed_pages and pages and group.k is not None:
            import torch

            from ..kernels import ops
            ops.poison_pages(group.k, group.v, torch.tensor(sorted(pages), dtype=torch.int32, device=group.k.device))

    def reset(self) -> None:
        for slot in range(self.num_slots):
            if self.slots.is_held(slot):
                self.free_slot(slot)

    # ---- steps

    def plan_step(self, slots: Sequence[int], q_lens: Sequence[int]) -> StepPlan:
        """Reserve pages for a step that appends q_lens[i] tokens to slots[i]; all or nothing."""
        if len(slots) != len(q_lens) or not slots:
            raise CacheError("a step needs as many lengths as slots, and at least one")
        if len(set(slots)) != len(slots):
            raise CacheError("a slot appears twice in one step")
        for s, q in zip(slots, q_lens):
            if not self.slots.is_held(s):
                raise CacheError(f"slot {s} is not live")
            if q <= 0:
                raise CacheError(f"slot {s}: a step must bring at least one token")
            if self.seq_len[s] + q > self.max_seq_len:
                raise CacheError(f"slot {s}: {self.seq_len[s]} + {q} tokens exceed the maximum "
                                 f"sequence length {self.max_seq_len}")
        for g in self.paged:
            need = sum(g.ledger.pages_needed(s, self.seq_len[s] + q) for s, q in zip(slots, q_lens))
            if need > g.ledger.pool.n_free:
                raise CacheFull(f"the step needs {need} more pages, {g.ledger.pool.n_free} of "
                                f"{g.ledger.pool.n} are free")
        tables = []
        for g in self.paged:
            tab = np.empty((len(slots), self.width), dtype=np.int32)
            for i, (s, q) in enumerate(zip(slots, q_lens)):
                g.ledger.reserve(s, self.seq_len[s] + q)
                g.ledger.row(s, self.width, tab[i])
            tables.append(tab)
        return StepPlan(list(slots), list(q_lens), [self.seq_len[s] for s in slots], tables)

    def commit_step(self, plan: StepPlan) -> None:
        for s, q in zip(plan.slots, plan.q_lens):
            self.seq_len[s] += q
            for g in self.paged:
                self._poison(g, g.ledger.release_outside_window(s, self.seq_len[s]))

    # ---- views

    def kv_view(self, entry: int, table_dev, group_index_out=None) -> KVView:
        kind, gi, ei = self.where[entry]
        if kind != "kv":
            raise CacheError(f"cache entry {entry} holds fixed state, not keys and values")
        g = self.paged[gi]
        return KVView(g.k[ei], g.v[ei], table_dev, self.page_size, g.request.window)

    def group_of(self, entry: int):
        return self.where[entry][:2]

    def state_view(self, entry: int, slots_dev) -> StateView:
        kind, gi, ei = self.where[entry]
        if kind != "state":
            raise CacheError(f"cache entry {entry} holds keys and values, not fixed state")
        return StateView(self.states[gi].state[ei], slots_dev)

    # ---- checks and figures

    def check(self) -> None:
        self.slots.check()
        for g in self.paged:
            g.ledger.check()
            for slot in range(self.num_slots):
                if not self.slots.is_held(slot) and g.ledger.pages[slot]:
                    raise CacheError(f"free slot {slot} still holds pages")

    def pages_free(self) -> List[int]:
        return [g.ledger.pool.n_free for g in self.paged]

    def storage_bytes(self, elem_size: int) -> int:
        return sum(g.bytes(elem_size) for g in self.paged)
