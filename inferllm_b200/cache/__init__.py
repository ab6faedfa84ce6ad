"""The cache's bookkeeping as Python sees it (for tests and for looking into an engine's cache): the
pools, ledgers and the sequence cache are the C++ core's (`cache/cache.h`); nothing here touches a
device."""
from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .. import binding as _b
from ..binding import CacheError, CacheFull   # noqa: F401


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every position (or of the last `window` positions) of a sequence."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def to_json(self):
        return {"kind": "kv", "n_kv_heads": self.n_kv_heads, "head_dim": self.head_dim, "window": self.window}


@dataclass(frozen=True)
class FixedState:
    """State of a fixed size per sequence, zeroed when a slot is handed out."""

    shape: Tuple[int, ...]
    dtype: str = "float32"

    def to_json(self):
        return {"kind": "state", "shape": list(self.shape), "dtype": str(self.dtype).replace("torch.", "")}


class IndexPool:
    def __init__(self, n: int, what: str, _ptr=None, _owner=None):
        self._owner = _owner
        if _ptr is None:
            out = ctypes.c_void_p()
            _b.check(_b.lib().illm_pool_create(n, what.encode(), ctypes.byref(out)))
            _ptr = out
        self._ptr = _ptr
        self.n = n

    def __del__(self):
        if self._owner is None and self._ptr and _b._lib is not None:
            _b._lib.illm_pool_free_handle(self._ptr)

    def _stats(self):
        a, b = ctypes.c_int(), ctypes.c_int()
        _b.lib().illm_pool_stats(self._ptr, ctypes.byref(a), ctypes.byref(b))
        return a.value, b.value

    n_free = property(lambda self: self._stats()[0])
    n_held = property(lambda self: self._stats()[1])

    def alloc(self, count: int = 1) -> List[int]:
        out = (ctypes.c_int * max(count, 1))()
        _b.check(_b.lib().illm_pool_alloc(self._ptr, count, out))
        return list(out[:count])

    def free(self, items) -> None:
        items = list(items)
        _b.check(_b.lib().illm_pool_release(self._ptr, _b.ints(items), len(items)))

    def is_held(self, i: int) -> bool:
        return bool(_b.lib().illm_pool_is_held(self._ptr, i))

    def check(self) -> None:
        _b.check(_b.lib().illm_pool_check(self._ptr))


class PageLedger:
    def __init__(self, num_pages: int, page_size: int, num_slots: int, window=None):
        out = ctypes.c_void_p()
        _b.check(_b.lib().illm_ledger_create(num_pages, page_size, num_slots, int(window or 0), ctypes.byref(out)))
        self._ptr = out
        self.num_slots = num_slots
        self.pool = IndexPool(num_pages, "page", _ptr=ctypes.c_void_p(_b.lib().illm_ledger_pool(out)), _owner=self)

    def __del__(self):
        if self._ptr and _b._lib is not None:
            _b._lib.illm_ledger_free_handle(self._ptr)

    def pages_needed(self, slot: int, new_len: int) -> int:
        return _b.lib().illm_ledger_pages_needed(self._ptr, slot, new_len)

    def reserve(self, slot: int, new_len: int) -> None:
        _b.check(_b.lib().illm_ledger_reserve(self._ptr, slot, new_len))

    def release_outside_window(self, slot: int, seq_len: int) -> None:
        _b.check(_b.lib().illm_ledger_release_outside_window(self._ptr, slot, seq_len))

    def release_all(self, slot: int) -> None:
        _b.check(_b.lib().illm_ledger_release_all(self._ptr, slot))

    def release_beyond(self, slot: int, seq_len: int) -> None:
        _b.check(_b.lib().illm_ledger_release_beyond(self._ptr, slot, seq_len))

    def row(self, slot: int, width: int, out=None):
        buf = (ctypes.c_int * max(width, 1))()
        _b.check(_b.lib().illm_ledger_row(self._ptr, slot, width, buf))
        if out is not None:
            out[:width] = list(buf[:width])
        return list(buf[:width])

    def check(self) -> None:
        _b.check(_b.lib().illm_ledger_check(self._ptr))

    @property
    def pages(self) -> List[Dict[int, int]]:
        """Per slot: logical page -> physical page."""
        res = []
        for slot in range(self.num_slots):
            lo, ph = (ctypes.c_int * 4096)(), (ctypes.c_int * 4096)()
            n = _b.lib().illm_ledger_pages(self._ptr, slot, lo, ph, 4096)
            res.append({lo[i]: ph[i] for i in range(min(n, 4096))})
        return res


@dataclass
class StepPlan:
    ticket: int
    slots: List[int]
    q_lens: List[int]
    past: List[int]
    tables: List[np.ndarray]       # per paged group: int32 [B, width]


class SequenceCache:
    """`requests`: cache entry number -> PagedKV | FixedState | None.  Made here, the cache is
    host-only (bookkeeping without device storage); `SequenceCache.of_engine` looks into the cache
    that an engine owns."""

    def __init__(self, requests: Dict[int, object], num_slots: int, num_pages: int, page_size: int, max_seq_len: int,
                 _wrap=None, _owner=None):
        self._owner = _owner
        if _wrap is None:
            reqs = {str(k): (None if v is None else v.to_json()) for k, v in requests.items()}
            out = ctypes.c_void_p()
            _b.check(_b.lib().illm_cache_create(json.dumps(reqs).encode(), num_slots, num_pages, page_size, max_seq_len,
                                                ctypes.byref(out)))
            self._ptr = out
        else:
            self._ptr = ctypes.c_void_p(_b.lib().illm_cache_wrap(_wrap))

    @classmethod
    def wrap(cls, sequence_cache_ptr, owner):
        return cls(None, 0, 0, 0, 0, _wrap=sequence_cache_ptr, _owner=owner)

    def __del__(self):
        if self._ptr and _b._lib is not None:
            _b._lib.illm_cache_free_handle(self._ptr)

    def stats(self) -> dict:
        return _b.call_json(_b.lib().illm_cache_stats, self._ptr)

    num_slots = property(lambda self: self.stats()["num_slots"])
    num_pages = property(lambda self: self.stats()["num_pages"])
    page_size = property(lambda self: self.stats()["page_size"])
    width = property(lambda self: self.stats()["width"])
    max_seq_len = property(lambda self: self.stats()["max_seq_len"])
    seq_len = property(lambda self: self.stats()["seq_len"])
    slots_free = property(lambda self: self.stats()["slots_free"])

    def alloc_slot(self) -> int:
        out = ctypes.c_int()
        _b.check(_b.lib().illm_cache_alloc_slot(self._ptr, ctypes.byref(out)))
        return out.value

    def free_slot(self, slot: int) -> None:
        _b.check(_b.lib().illm_cache_free_slot(self._ptr, slot))

    def reset(self) -> None:
        _b.check(_b.lib().illm_cache_reset(self._ptr))

    def check(self) -> None:
        _b.check(_b.lib().illm_cache_check(self._ptr))

    def plan_step(self, slots: Sequence[int], q_lens: Sequence[int]) -> StepPlan:
        st = self.stats()
        n, groups, width = len(slots), len(st["paged"]), st["width"]
        tables = np.empty((max(groups, 1), max(n, 1), width), dtype=np.int32)
        past = (ctypes.c_longlong * max(n, 1))()
        ticket = ctypes.c_int()
        if len(q_lens) != n:
            raise CacheError("a step needs as many lengths as slots, and at least one")
        _b.check(_b.lib().illm_cache_plan_step(self._ptr, _b.ints(slots), _b.ints(q_lens), n,
                                               tables.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), past, ctypes.byref(ticket)))
        return StepPlan(ticket.value, list(slots), list(q_lens), list(past[:n]), [tables[g, :n] for g in range(groups)])

    def commit_step(self, plan: StepPlan) -> None:
        _b.check(_b.lib().illm_cache_commit_step(self._ptr, plan.ticket))

    def abandon_step(self, plan: StepPlan) -> None:
        _b.check(_b.lib().illm_cache_abandon_step(self._ptr, plan.ticket))

    def pages_free(self) -> List[int]:
        return [g["pages_free"] for g in self.stats()["paged"]]

    def pages_of(self, group: int, slot: int) -> Dict[int, int]:
        return {int(k): v for k, v in self.stats()["paged"][group]["pages"][slot].items()}
