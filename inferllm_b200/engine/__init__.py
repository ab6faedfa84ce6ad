"""The engine, the programming entry point and the generation loop as Python sees them: thin faces
over the C++ core (`engine/engine.h`, `engine/model_api.h`, `engine/generate.h`).  Token ids go in as
Python lists; logits come back as float32 torch tensors on the device the engine runs on.  The engine
works on a CUDA stream of its own; every call that exchanges device memory with torch orders that
stream against torch's current stream (the one waits for the other, the host for neither), so the
tensors can be used like the results of any torch operation."""
from __future__ import annotations

import ctypes
import json
from dataclasses import asdict, dataclass, field
from typing import Callable, List, Optional, Sequence

from .. import binding as _b
from ..binding import EngineError, RequestTooLong   # noqa: F401
from ..cache import SequenceCache
from ..config import ArchConfig, config_from_folder


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
    cuda_graphs: bool = True       # replay one-token-per-sequence steps and single prompts from captured CUDA graphs
    gemm: str = "auto"             # bfloat16 products: "auto" | "tc" | "library"
    poison_freed_pages: bool = False    # fill pages that go back to the pool with NaN (a check, not for serving)

    def to_json(self, stream: int) -> str:
        d = asdict(self)
        d["max_tokens"] = self.max_tokens or 0
        d["max_seq_len"] = self.max_seq_len or 0
        d["max_batch"] = self.max_batch or 0
        d["stream"] = stream
        return json.dumps(d)


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


def _need_cuda(device_id: int) -> None:
    import torch
    if not torch.cuda.is_available():
        raise EngineError("inferllm_b200 needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(device_id)


def caller_stream(device_id: Optional[int] = None) -> ctypes.c_void_p:
    """torch's current stream as the library takes a caller's stream: the legacy default stream
    (handle 0) is named by CUDA's cudaStreamLegacy (1), since 0 means "none" there."""
    import torch
    s = int(torch.cuda.current_stream(device_id).cuda_stream)
    return ctypes.c_void_p(s if s else 1)


def _flatten(items):
    slots = [int(it.slot) for it in items]
    n_tok = [len(it.tokens) for it in items]
    toks = [int(t) for it in items for t in it.tokens]
    n_want = [len(it.want) for it in items]
    want = [int(w) for it in items for w in it.want]
    return slots, n_tok, toks, n_want, want


class Engine:
    """A model, its cache and the step function (see `engine/engine.h`)."""

    def __init__(self, config: ArchConfig, options: EngineOptions, _ptr=None, _owner=None):
        self.options = options
        self._owner = _owner
        self._cache = None
        self._children = []       # weak references to samplers made on this engine: they go before it does
        if _ptr is None:
            out = ctypes.c_void_p()
            _need_cuda(options.device_id)
            _b.check(_b.lib().illm_engine_create(config.handle(), options.to_json(0).encode(), ctypes.byref(out)))
            _ptr = out
        self._ptr = _ptr
        self.config = config
        info = self.info()
        self.vocab_size = info["vocab_size"]
        self.device_id = info["device"]

    def _adopt(self, child) -> None:
        import weakref
        self._children.append(weakref.ref(child))

    def _release_children(self) -> None:
        for ref in getattr(self, "_children", []):
            child = ref()
            if child is not None:
                child._free()
        self._children = []

    def __del__(self):
        self._release_children()
        if getattr(self, "_owner", None) is None and getattr(self, "_ptr", None) and _b._lib is not None:
            _b._lib.illm_engine_free(self._ptr)
        self._ptr = None

    # ---- construction

    @classmethod
    def from_folder(cls, folder: str, options: EngineOptions, model_name: Optional[str] = None):
        config = config_from_folder(folder, model_name)
        eng = cls(config, options)
        _b.check(_b.lib().illm_engine_load_folder(eng._ptr, folder.encode()))
        return eng

    @classmethod
    def from_config(cls, config: ArchConfig, options: EngineOptions, seed: int = 0):
        """Random weights made on the device, without a file."""
        eng = cls(config, options)
        _b.check(_b.lib().illm_engine_load_random(eng._ptr, int(seed)))
        return eng

    # ---- sequences

    def new_sequence(self) -> int:
        out = ctypes.c_int()
        _b.check(_b.lib().illm_engine_new_sequence(self._ptr, ctypes.byref(out)))
        return out.value

    def end_sequence(self, slot: int) -> None:
        _b.check(_b.lib().illm_engine_end_sequence(self._ptr, slot))

    def sequence_length(self, slot: int) -> int:
        out = ctypes.c_longlong()
        _b.check(_b.lib().illm_engine_sequence_length(self._ptr, slot, ctypes.byref(out)))
        return out.value

    def limits(self) -> Limits:
        out = (ctypes.c_longlong * 4)()
        _b.check(_b.lib().illm_engine_limits(self._ptr, out))
        return Limits(*[int(v) for v in out])

    # ---- the step

    def step(self, items: Sequence[StepItem], device_ids=None):
        """Run one step; float32 logits [number of wanted places, vocab] on the device, in the order of
        the items and of each item's `want`.  `device_ids` (int32 tensor on the device, one id per
        item) gives the tokens of a one-token-per-sequence step without a round trip through the host."""
        import torch
        slots, n_tok, toks, n_want, want = _flatten(items)
        if device_ids is not None and (device_ids.dtype != torch.int32 or device_ids.numel() != len(items)):
            raise EngineError("device_ids needs one int32 id per item and items of one token each")
        out = torch.empty((len(want), self.vocab_size), dtype=torch.float32, device=f"cuda:{self.device_id}")
        _b.check(_b.lib().illm_engine_step(self._ptr, len(slots), _b.ints(slots), _b.ints(n_tok), _b.ints(toks), _b.ints(n_want),
                                           _b.ints(want), device_ids.data_ptr() if device_ids is not None else None,
                                           out.data_ptr() if len(want) else None, None, caller_stream(self.device_id)))
        return out

    def warm_up(self, prompt_tokens: int = 0, batch_sizes: Sequence[int] = ()) -> None:
        sizes = list(batch_sizes)
        _b.check(_b.lib().illm_engine_warm_up(self._ptr, int(prompt_tokens), _b.ints(sizes), len(sizes)))

    def check_device_errors(self) -> None:
        """Read the kernels' error words (synchronises); EngineError naming what a kernel reported."""
        _b.check(_b.lib().illm_engine_check_device_errors(self._ptr))

    def set_gemm(self, name: str) -> None:
        """Which kernels run the bfloat16 products from now on (captured graphs are dropped)."""
        _b.check(_b.lib().illm_engine_set_gemm(self._ptr, name.encode()))

    # ---- looking inside

    def info(self) -> dict:
        return _b.call_json(_b.lib().illm_engine_info, self._ptr)

    @property
    def cache(self) -> SequenceCache:
        if self._cache is None:
            self._cache = SequenceCache.wrap(_b.lib().illm_engine_cache(self._ptr), self)
        return self._cache

    @property
    def last_upload_bytes(self) -> int:
        return self.info()["last_upload_bytes"]

    def cache_tensors(self, group: int = 0):
        """(k, v) of a paged group as torch tensors [entries, pages, kv heads, page_size, head_dim]
        that view the engine's own storage."""
        import torch
        st = self.cache.stats()
        g = st["paged"][group]
        shape = (len(g["entries"]), st["num_pages"], g["request"]["n_kv_heads"], st["page_size"], g["request"]["head_dim"])
        dtype = torch.float32 if self.info()["dtype"] == "float32" else torch.bfloat16
        return tuple(device_view(g[name], shape, dtype, self.device_id) for name in ("k", "v"))

    def state_tensor(self, group: int = 0):
        import torch
        st = self.cache.stats()
        g = st["states"][group]
        dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}[g["request"]["dtype"]]
        return device_view(g["state"], (len(g["entries"]), st["num_slots"], *g["request"]["shape"]), dtype, self.device_id)

    def order(self, direction: int) -> None:
        """0: the engine's stream waits for what torch's current stream holds now; 1: the other way round."""
        _b.check(_b.lib().illm_engine_order(self._ptr, caller_stream(self.device_id), direction))

    def _copy(self, dst: int, src: int, nbytes: int) -> None:
        """Copy device memory on torch's current stream."""
        dev = ctypes.c_void_p()
        _b.check(_b.lib().illm_test_device(caller_stream(self.device_id), ctypes.byref(dev)))
        _b.check(_b.lib().illm_copy_device(dev, ctypes.c_void_p(dst), ctypes.c_void_p(src), nbytes))


class _Raw:
    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def device_view(ptr: int, shape, dtype, device_id: int = 0):
    """A torch tensor that views device memory of the library (no copy; valid as long as its owner)."""
    import torch
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    if n == 0:
        return torch.empty(shape, dtype=dtype, device=f"cuda:{device_id}")
    return torch.as_tensor(_Raw(int(ptr), nbytes), device=f"cuda:{device_id}").view(dtype).view(*shape)


# ---- generation


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


def plan_batches(prompt_lens: Sequence[int], max_new_tokens: int, limits: Limits) -> List[List[int]]:
    """Cut the requests, in order, into batches that fit the slots and the pages (`engine/generate.h`)."""
    lens = list(prompt_lens)
    return _b.call_json(_b.lib().illm_plan_batches, _b.ints(lens), len(lens), int(max_new_tokens), limits.max_batch,
                        limits.num_pages, limits.page_size, limits.max_seq_len)


class _LoopCallbacks(ctypes.Structure):
    _fields_ = [("user", ctypes.c_void_p)] + [(n, ctypes.c_void_p) for n in (
        "limits", "new_sequence", "end_sequence", "step", "choose", "read_async", "finish_read", "select", "clock", "on_token")]


def generate(backend, prompts: Sequence[Sequence[int]], choose: Callable, max_new_tokens: int, stop_ids: Sequence[int] = (),
             on_token: Optional[Callable] = None, clock: Optional[Callable] = None) -> GenerationResult:
    """The library's generation loop over a backend and a chooser written in Python (stand-ins in
    tests, or an engine driven from Python).  `backend` has `limits()`, `new_sequence()`,
    `end_sequence(slot)`, `step(items, device_ids=None)` and may have `read_tokens_async(toks)` (returns
    a function that gives the list); `choose(logits, requests, steps, histories)` returns one token per
    row (a list, or anything with `tolist()`; indexable by a list of rows if it is no list)."""
    I, LL, P = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
    PI, PLL = ctypes.POINTER(I), ctypes.POINTER(LL)
    objects, reads, error = {}, {}, []

    counter = [0]

    def keep(obj) -> int:
        counter[0] += 1
        h = counter[0]
        objects[h] = obj
        if len(objects) > 64:
            objects.pop(min(objects))
        return h

    def guarded(fn):
        def wrapped(*a):
            try:
                return fn(*a) or 0
            except BaseException as e:     # handed back to the caller when the loop has unwound
                error.append(e)
                return 1
        return wrapped

    def cb_limits(_u, out):
        lim = backend.limits()
        out[0], out[1], out[2], out[3] = lim.max_batch, lim.num_pages, lim.page_size, lim.max_seq_len

    def cb_new(_u, slot):
        slot[0] = backend.new_sequence()

    def cb_end(_u, slot):
        backend.end_sequence(slot)

    def cb_step(_u, n, slots, n_tok, toks, n_want, want, ids, logits):
        items, to, wo = [], 0, 0
        for i in range(n):
            items.append(StepItem(slots[i], [toks[to + j] for j in range(n_tok[i])], [want[wo + j] for j in range(n_want[i])]))
            to += n_tok[i]
            wo += n_want[i]
        out = backend.step(items) if ids < 0 else backend.step(items, device_ids=objects[ids])
        logits[0] = keep(out)

    def cb_choose(_u, logits, n, requests, steps, has_hist, hist_lens, hist, tokens):
        hs = None
        if has_hist:
            hs, off = [], 0
            for i in range(n):
                hs.append([hist[off + j] for j in range(hist_lens[i])])
                off += hist_lens[i]
        tokens[0] = keep(choose(objects[logits], [requests[i] for i in range(n)], [steps[i] for i in range(n)], hs))

    def as_list(t):
        return [int(x) for x in (t.tolist() if hasattr(t, "tolist") else t)]

    def cb_read(_u, tokens, ticket):
        t = objects[tokens]
        f = getattr(backend, "read_tokens_async", None)
        ticket[0] = keep(None)
        reads[ticket[0]] = f(t) if f is not None else (lambda: as_list(t))

    def cb_finish(_u, ticket, out, cap, n):
        vals = as_list(reads.pop(ticket)())
        for i, v in enumerate(vals[:cap]):
            out[i] = v
        n[0] = len(vals)

    def cb_select(_u, tokens, idx, n, out):
        t, rows = objects[tokens], [idx[i] for i in range(n)]
        out[0] = keep([t[i] for i in rows] if isinstance(t, (list, tuple)) else t[rows])

    table = _LoopCallbacks()
    funcs = [
        ctypes.CFUNCTYPE(I, P, PLL)(guarded(cb_limits)), ctypes.CFUNCTYPE(I, P, PI)(guarded(cb_new)),
        ctypes.CFUNCTYPE(I, P, I)(guarded(cb_end)), ctypes.CFUNCTYPE(I, P, I, PI, PI, PI, PI, PI, LL, PLL)(guarded(cb_step)),
        ctypes.CFUNCTYPE(I, P, LL, I, PI, PI, I, PI, PI, PLL)(guarded(cb_choose)), ctypes.CFUNCTYPE(I, P, LL, PI)(guarded(cb_read)),
        ctypes.CFUNCTYPE(I, P, I, PI, I, PI)(guarded(cb_finish)), ctypes.CFUNCTYPE(I, P, LL, PI, I, PLL)(guarded(cb_select)),
        ctypes.CFUNCTYPE(ctypes.c_double, P)(lambda _u: float(clock())) if clock else None,
        ctypes.CFUNCTYPE(None, P, I, I)(lambda _u, r, t: on_token(r, t)) if on_token else None]
    for name, f in zip([n for n, _ in _LoopCallbacks._fields_[1:]], funcs):
        setattr(table, name, ctypes.cast(f, P) if f is not None else None)
    lens = [len(p) for p in prompts]
    flat = [int(t) for p in prompts for t in p]
    stop = [int(s) for s in stop_ids]
    out = ctypes.c_void_p()
    rc = _b.lib().illm_generate_with_callbacks(ctypes.byref(table), len(lens), _b.ints(lens), _b.ints(flat), int(max_new_tokens),
                                               _b.ints(stop), len(stop), ctypes.byref(out))
    if error:
        raise error[0]
    _b.check(rc)
    return GenerationResult(**json.loads(_b.take_string(out)))


# ---- the programming entry point


@dataclass
class ModelConfig:
    """Fields of the reference's ModelConfig (include/model.h:14-23).  `compt_type`: "bfloat16" or
    "float32"; `device_type` must be "gpu"; `nr_thread` and `enable_mmap` are accepted and have no
    effect; `nr_ctx` is the longest sequence; `device_id` the GPU ordinal.  `max_tokens` (not in the
    reference) sizes the cache for batches; default `nr_ctx`."""

    compt_type: str = "bfloat16"
    device_type: str = "gpu"
    nr_thread: int = 1
    nr_ctx: int = 2048
    device_id: int = 0
    enable_mmap: bool = True
    max_tokens: Optional[int] = None
    max_batch: Optional[int] = None
    page_size: int = 64
    cuda_graphs: bool = True
    gemm: str = "auto"
    poison_freed_pages: bool = False


class Model:
    """The entry point in the manner of the reference's `inferllm::Model` (include/model.h:27-59): `load`,
    `init`, `prefill`, `decode`, `decode_iter`, `get_remain_token`, `reset_token`, `decode_summary`,
    plus `generate` for batches of requests.  A face of `illm::Model` (`engine/model_api.h`)."""

    def __init__(self, config: ModelConfig, model_name: Optional[str] = None):
        self.config = config
        d = asdict(config)
        d["max_tokens"] = config.max_tokens or 0
        d["max_batch"] = config.max_batch or 0
        if config.device_type.lower() in ("gpu", "cuda"):
            _need_cuda(config.device_id)
        out = ctypes.c_void_p()
        _b.check(_b.lib().illm_model_create(json.dumps(d).encode(), _b.enc(model_name), ctypes.byref(out)))
        self._ptr = out
        self._engine = None

    def _drop_engine(self) -> None:
        if self._engine is not None:
            self._engine._release_children()
            self._engine._ptr = None
            self._engine = None

    def __del__(self):
        if getattr(self, "_ptr", None) and _b._lib is not None:
            self._drop_engine()
            _b._lib.illm_model_free(self._ptr)
            self._ptr = None

    def load(self, model_path: str) -> None:
        self._drop_engine()
        _b.check(_b.lib().illm_model_load(self._ptr, model_path.encode()))

    def load_random(self, config: ArchConfig, seed: int = 0) -> None:
        self._drop_engine()
        _b.check(_b.lib().illm_model_load_random(self._ptr, config.handle(), int(seed)))

    @property
    def engine(self) -> Engine:
        if self._engine is None:
            out = ctypes.c_void_p()
            _b.check(_b.lib().illm_model_engine(self._ptr, ctypes.byref(out)))
            self._engine = Engine(None, EngineOptions(dtype=self.config.compt_type, device_id=self.config.device_id), _ptr=out,
                                  _owner=self)
        return self._engine

    def _ends(self):
        return _b.call_json(_b.lib().illm_model_end_tokens, self._ptr)

    end_token = property(lambda self: self._ends()["end_token"])
    end_tokens = property(lambda self: self._ends()["end_tokens"])

    def init(self, top_k: int, top_p: float, temp: float, repeat_penalty: float, repeat_last_n: int, seed: int,
             end_token: int) -> None:
        _b.check(_b.lib().illm_model_init(self._ptr, top_k, top_p, temp, repeat_penalty, repeat_last_n, seed, end_token))

    def get_remain_token(self) -> int:
        out = ctypes.c_uint()
        _b.check(_b.lib().illm_model_get_remain_token(self._ptr, ctypes.byref(out)))
        return out.value

    def reset_token(self) -> None:
        _b.check(_b.lib().illm_model_reset_token(self._ptr))

    def prefill(self, prompt: Sequence[int]) -> None:
        p = [int(t) for t in prompt]
        _b.check(_b.lib().illm_model_prefill(self._ptr, _b.ints(p), len(p)))

    def decode(self, user_input: Sequence[int]) -> int:
        p, out = [int(t) for t in user_input], ctypes.c_int()
        _b.check(_b.lib().illm_model_decode(self._ptr, _b.ints(p), len(p), ctypes.byref(out)))
        return out.value

    def decode_iter(self) -> int:
        out = ctypes.c_int()
        _b.check(_b.lib().illm_model_decode_iter(self._ptr, ctypes.byref(out)))
        return out.value

    def decode_summary(self) -> str:
        return _b.call_text(_b.lib().illm_model_decode_summary, self._ptr)

    def warm_up(self, prompt_tokens: int = 0, batch_sizes: Sequence[int] = ()) -> None:
        sizes = list(batch_sizes)
        _b.check(_b.lib().illm_model_warm_up(self._ptr, int(prompt_tokens), _b.ints(sizes), len(sizes)))

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 128, stop_ids: Optional[Sequence[int]] = None,
                 on_token=None) -> GenerationResult:
        """Generate for many requests.  `stop_ids` default to the end token given to `init`; where that
        is one of the configuration's end tokens, to all of them."""
        lens = [len(p) for p in prompts]
        flat = [int(t) for p in prompts for t in p]
        stop = None if stop_ids is None else _b.ints(int(s) for s in stop_ids)
        cb = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_int, ctypes.c_int)(lambda _u, r, t: on_token(r, t)) if on_token else None
        out = ctypes.c_void_p()
        _b.check(_b.lib().illm_model_generate(self._ptr, len(lens), _b.ints(lens), _b.ints(flat), int(max_new_tokens), stop,
                                              0 if stop_ids is None else len(list(stop_ids)),
                                              ctypes.cast(cb, ctypes.c_void_p) if cb else None, None, ctypes.byref(out)))
        return GenerationResult(**json.loads(_b.take_string(out)))
