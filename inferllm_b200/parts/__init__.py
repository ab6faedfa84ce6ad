"""Parts as Python sees them.

Two things live here.  (1) Base classes with which a mixer, a feed-forward or a position encoding
is written in Python and registered under a kind of its own (`register_mixer("my_kind")` and so on):
the library then builds it wherever a ModelSpec names that kind, hands it its tensors and calls it
on the tokens of each step, with torch tensors that view the library's device memory.  (2) A
sandbox in which one part of the library is built, loaded and run without a model (`PartSandbox`),
for tests of single parts.  The parts themselves, their interfaces and registries are the C++
core's (`parts/parts.h`); the C interface for parts in other languages is `binding/foreign.h`.
"""
from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

from .. import binding as _b
from ..cache import FixedState, PagedKV, SequenceCache   # noqa: F401
from ..config import PartSpec

I, LL, P = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
PI, PLL = ctypes.POINTER(I), ctypes.POINTER(LL)


class StepInfo(ctypes.Structure):
    _fields_ = [("T", I), ("B", I), ("K", I), ("max_q", I), ("is_decode", I), ("max_len", LL), ("max_seq_len", LL),
                ("ids", P), ("token_pos", P), ("token_seq", P), ("want_rows", P), ("slots", P), ("seq_lens", P), ("cu_q", P),
                ("q_lens", PI), ("host_slots", PI), ("past", PLL), ("err", P), ("stream", P), ("dtype", I), ("page_size", I)]


class CacheInfo(ctypes.Structure):
    _fields_ = [("kind", I), ("k", P), ("v", P), ("block_table", P), ("width", I), ("num_pages", I), ("page_size", I),
                ("window", I), ("n_kv_heads", I), ("head_dim", I), ("dtype", I), ("writes", I), ("state", P), ("slots", P),
                ("num_slots", I), ("elements", LL), ("state_dtype", I)]


class ForeignPart(ctypes.Structure):
    _fields_ = [("user", P), ("describe", P), ("create", P), ("destroy", P), ("load", P), ("mixer_forward", P),
                ("ffn_forward", P), ("encode_and_store", P)]


@dataclass
class TensorDecl:
    """A tensor that a part needs.  `init`: "matrix" -> N(0, 0.02); "norm" -> 1 + N(0, 0.02); "int" -> an
    integer table (kept int32)."""

    shape: Tuple[int, ...]
    init: str = "matrix"


def _torch_stream(handle):
    """The step's stream as a torch stream (cudaStreamLegacy, 1, is torch's default stream)."""
    import torch
    h = int(handle or 0)
    return torch.cuda.default_stream() if h in (0, 1) else torch.cuda.ExternalStream(h)


def _torch_dtype(code: int):
    import torch
    return {0: torch.float32, 1: torch.bfloat16, 5: torch.int32}[code]


class StepView:
    """What a part written in Python sees of a step: int32 torch tensors on the device (`ids`,
    `token_pos`, `token_seq`, `slots`, `seq_lens`, `cu_q`, `want_rows`, `err`), and on the host the
    lists `q_lens`, `host_slots`, `past`.  A part that reads the host fields must say
    `graph_safe = False`."""

    def __init__(self, info: StepInfo, device_id: int):
        from ..engine import device_view
        import torch
        self.T, self.B, self.K, self.max_q = info.T, info.B, info.K, info.max_q
        self.is_decode, self.max_len, self.max_seq_len = bool(info.is_decode), info.max_len, info.max_seq_len
        self.page_size, self.dtype = info.page_size, _torch_dtype(info.dtype)
        for name, n in (("ids", info.T), ("token_pos", info.T), ("token_seq", info.T), ("want_rows", info.K),
                        ("slots", info.B), ("seq_lens", info.B), ("cu_q", info.B + 1), ("err", 1)):
            setattr(self, name, device_view(getattr(info, name), (n,), torch.int32, device_id))
        self.q_lens = [info.q_lens[i] for i in range(info.B)]
        self.host_slots = [info.host_slots[i] for i in range(info.B)]
        self.past = [info.past[i] for i in range(info.B)]
        self.stream = info.stream


class KVCacheView:
    """A mixer's keys and values for the step: `k`, `v` [pages, kv heads, page_size, head_dim],
    `block_table` int32 [B, width], `page_size`, `window`, `writes`."""

    def __init__(self, c: CacheInfo, B: int, device_id: int):
        from ..engine import device_view
        import torch
        shape = (c.num_pages, c.n_kv_heads, c.page_size, c.head_dim)
        self.k = device_view(c.k, shape, _torch_dtype(c.dtype), device_id)
        self.v = device_view(c.v, shape, _torch_dtype(c.dtype), device_id)
        self.block_table = device_view(c.block_table, (B, c.width), torch.int32, device_id)
        self.page_size, self.window, self.writes = c.page_size, c.window or None, bool(c.writes)


class StateCacheView:
    """A mixer's fixed-size state: `state` [slots, elements] and `slots`, int32 [B] on the device."""

    def __init__(self, c: CacheInfo, B: int, device_id: int):
        from ..engine import device_view
        import torch
        self.state = device_view(c.state, (c.num_slots, c.elements), _torch_dtype(c.state_dtype), device_id)
        self.slots = device_view(c.slots, (B,), torch.int32, device_id)


def _cache_view(c: CacheInfo, B: int, device_id: int):
    if c.kind == 1:
        return KVCacheView(c, B, device_id)
    if c.kind == 2:
        return StateCacheView(c, B, device_id)
    return None


# ---- parts written in Python


@dataclass
class RuntimeInfo:
    """Where a part written in Python runs: the compute dtype (a torch dtype) and the device."""

    dtype: object
    device: object


class Part:
    """Base of parts written in Python.  `spec` is the PartSpec the part is built from; `rt` is None
    when the part is only asked for its tensors (checking a folder, writing a random one)."""

    graph_safe = False       # see Mixer::graph_safe in parts/parts.h
    pad_safe = False
    takes_partials = False

    def __init__(self, spec: PartSpec, runtime: Optional[RuntimeInfo]):
        self.spec = spec
        self.rt = runtime

    def tensors(self) -> Dict[str, TensorDecl]:
        return {}

    def load(self, tensors: Dict[str, object]) -> None:
        """Receive the declared tensors (torch tensors on the device that view memory the library
        holds for this part, in the dtype the storage rule keeps them in)."""


class Mixer(Part):
    def cache_request(self):
        """`PagedKV`, `FixedState` or None."""
        return None

    def forward(self, h, ctx: StepView, cache, writes: bool):
        """h [T, H] in the compute dtype -> [T, H]."""
        raise NotImplementedError


class FeedForward(Part):
    graph_safe = True

    def forward(self, h, ctx: StepView):
        raise NotImplementedError


class PositionEncoding(Part):
    def encode_and_store(self, qkv, geometry, ctx: StepView, kv: KVCacheView):
        """Encode positions into the Q and K heads of `qkv` [T, (heads + 2 kv heads) * head_dim] in place
        and store the new K and V in the cache if `kv.writes`; `geometry` = (heads, kv heads, head_dim)."""
        raise NotImplementedError


_REGISTERED = {}     # (family, kind) -> everything that has to stay alive while the kind is registered


def _register(family: str, kind: str, cls):
    import torch
    from ..engine import device_view
    instances, texts, errors = {}, {}, []

    def guarded(fn):
        def wrapped(*a):
            try:
                return fn(*a) or 0
            except BaseException as e:
                errors.append(e)
                import traceback
                traceback.print_exc()
                return 1
        return wrapped

    def describe(_u, spec_json):
        try:
            part = cls(PartSpec.from_json(json.loads(spec_json.decode())), None)
            req = part.cache_request() if isinstance(part, Mixer) else None
            d = {"tensors": [[n, list(t.shape), t.init] for n, t in part.tensors().items()],
                 "cache": None if req is None else req.to_json(), "graph_safe": bool(part.graph_safe),
                 "pad_safe": bool(part.pad_safe), "takes_partials": bool(part.takes_partials)}
        except Exception as e:
            d = {"error": f"{type(e).__name__}: {e}"}
        texts["last"] = ctypes.create_string_buffer(json.dumps(d).encode())      # stays valid until the next call
        return ctypes.addressof(texts["last"])

    def create(_u, spec_json, dtype, on_device, instance):
        rt = RuntimeInfo(_torch_dtype(dtype), torch.device("cuda", torch.cuda.current_device())) if on_device else None
        part = cls(PartSpec.from_json(json.loads(spec_json.decode())), rt)
        part._loaded = {}
        h = max(instances, default=0) + 1
        instances[h] = part
        instance[0] = h

    def destroy(_u, instance):
        instances.pop(instance, None)

    def load(_u, instance, name, ptr, dtype, shape, ndim):
        part = instances[instance]
        t = device_view(ptr, [shape[i] for i in range(ndim)], _torch_dtype(dtype), torch.cuda.current_device())
        part._loaded[name.decode()] = t
        if set(part._loaded) == set(part.tensors()):
            part.load(dict(part._loaded))

    def device_of(step):
        return torch.cuda.current_device()

    def mixer_forward(_u, instance, step, cache, h, out, T, H, writes):
        part, s = instances[instance], step.contents
        dev = device_of(s)
        with torch.cuda.stream(_torch_stream(s.stream)):
            ctx = StepView(s, dev)
            x = device_view(h, (T, H), ctx.dtype, dev)
            y = part.forward(x, ctx, _cache_view(cache.contents, s.B, dev), bool(writes))
            device_view(out, (T, H), ctx.dtype, dev).copy_(y)

    def ffn_forward(_u, instance, step, h, out, T, H):
        part, s = instances[instance], step.contents
        dev = device_of(s)
        with torch.cuda.stream(_torch_stream(s.stream)):
            ctx = StepView(s, dev)
            y = part.forward(device_view(h, (T, H), ctx.dtype, dev), ctx)
            device_view(out, (T, H), ctx.dtype, dev).copy_(y)

    def encode_and_store(_u, instance, step, cache, qkv, T, width, nh, nkv, d):
        part, s = instances[instance], step.contents
        dev = device_of(s)
        with torch.cuda.stream(_torch_stream(s.stream)):
            ctx = StepView(s, dev)
            x = device_view(qkv, (T, width), ctx.dtype, dev)
            y = part.encode_and_store(x, (nh, nkv, d), ctx, KVCacheView(cache.contents, s.B, dev))
            if y is not None and y.data_ptr() != x.data_ptr():
                x.copy_(y)

    S = ctypes.c_char_p
    PS, PC = ctypes.POINTER(StepInfo), ctypes.POINTER(CacheInfo)
    funcs = {
        "describe": ctypes.CFUNCTYPE(P, P, S)(describe),
        "create": ctypes.CFUNCTYPE(I, P, S, I, I, PLL)(guarded(create)),
        "destroy": ctypes.CFUNCTYPE(None, P, LL)(destroy),
        "load": ctypes.CFUNCTYPE(I, P, LL, S, P, I, PLL, I)(guarded(load)),
        "mixer_forward": ctypes.CFUNCTYPE(I, P, LL, PS, PC, P, P, LL, LL, I)(guarded(mixer_forward)),
        "ffn_forward": ctypes.CFUNCTYPE(I, P, LL, PS, P, P, LL, LL)(guarded(ffn_forward)),
        "encode_and_store": ctypes.CFUNCTYPE(I, P, LL, PS, PC, P, LL, LL, I, I, I)(guarded(encode_and_store)),
    }
    table = ForeignPart()
    for name, f in funcs.items():
        setattr(table, name, ctypes.cast(f, P))
    _b.check(_b.lib().illm_register_foreign_part(family.encode(), kind.encode(), ctypes.byref(table)))
    _REGISTERED[(family, kind)] = (table, funcs, instances, texts, errors)
    return cls


def register_mixer(kind: str):
    return lambda cls: _register("mixer", kind, cls)


def register_feed_forward(kind: str):
    return lambda cls: _register("feed_forward", kind, cls)


def register_position(kind: str):
    return lambda cls: _register("position", kind, cls)


def unregister_part(family: str, kind: str):
    _b.check(_b.lib().illm_unregister_part(family.encode(), kind.encode()))
    _REGISTERED.pop((family, kind), None)


def registered_parts(family: str):
    return _b.call_json(_b.lib().illm_registered_parts, family.encode())


# ---- the sandbox


class _Proxy:
    """A part of the library built in a sandbox."""

    def __init__(self, sandbox, family: str, spec: PartSpec):
        self.sandbox, self.family, self.spec = sandbox, family, spec
        out = ctypes.c_void_p()
        _b.check(_b.lib().illm_sandbox_build(sandbox._ptr, family.encode(), json.dumps(spec.to_json()).encode(), ctypes.byref(out)))
        self._ptr = out
        sandbox._adopt(self)

    def _free(self) -> None:
        if getattr(self, "_ptr", None) and _b._lib is not None and getattr(self.sandbox, "_ptr", None):
            _b._lib.illm_part_free(self._ptr)       # (its tensors live on the sandbox's device)
        self._ptr = None

    def __del__(self):
        self._free()

    def describe(self) -> dict:
        return _b.call_json(_b.lib().illm_part_describe, self._ptr)

    def tensors(self) -> Dict[str, TensorDecl]:
        return {n: TensorDecl(tuple(s), i) for n, s, i in self.describe()["tensors"]}

    def cache_request(self):
        c = self.describe().get("cache")
        if not c:
            return None
        if c["kind"] == "kv":
            return PagedKV(c["n_kv_heads"], c["head_dim"], c["window"])
        return FixedState(tuple(c["shape"]), c["dtype"])

    def load(self, tensors: Dict[str, object]) -> None:
        """`tensors`: name -> torch tensor on the device (float32, bfloat16, float16 or int32)."""
        tensors = {k: v.contiguous() for k, v in tensors.items()}
        desc = {k: {"ptr": v.data_ptr(), "dtype": str(v.dtype).replace("torch.", ""), "shape": list(v.shape)}
                for k, v in tensors.items()}
        _b.check(_b.lib().illm_sandbox_load(self.sandbox._ptr, self._ptr, json.dumps(desc).encode()))

    def forward(self, *args, **kw):
        return getattr(self.sandbox, f"_{self.family}_forward")(self, *args, **kw)


class ResidualStream:
    """The float32 residual stream [T, H] with at most one addition pending (see parts/parts.h): `x`
    is the torch tensor the stream works on, in place."""

    def __init__(self, sandbox, x):
        self.sandbox, self.x, self._deltas = sandbox, x, []
        out = ctypes.c_void_p()
        _b.check(_b.lib().illm_stream_create(sandbox._ptr, x.data_ptr(), x.shape[0], x.shape[1], ctypes.byref(out)))
        self._ptr = out
        sandbox._adopt(self)

    def _free(self) -> None:
        if getattr(self, "_ptr", None) and _b._lib is not None and getattr(self.sandbox, "_ptr", None):
            _b._lib.illm_stream_free(self._ptr)
        self._ptr = None

    def __del__(self):
        self._free()

    def add(self, delta) -> None:
        import torch
        self._deltas.append(delta)       # the stream reads it later
        _b.check(_b.lib().illm_stream_add(self._ptr, delta.data_ptr(), 0 if delta.dtype == torch.float32 else 1))

    def flush(self):
        _b.check(_b.lib().illm_stream_flush(self._ptr))
        return self.x

    @property
    def pending(self):
        return True if _b.lib().illm_stream_has_pending(self._ptr) else None


class PartSandbox:
    """The minimum an engine gives a part under test: a device, a cache for the part's request and step
    contexts made the way the engine makes them."""

    def __init__(self, requests, dtype: str, num_slots=4, num_pages=16, page_size=16, max_seq_len=256):
        import torch
        self.dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
        reqs = {str(k): (None if v is None else v.to_json()) for k, v in requests.items()}
        out = ctypes.c_void_p()
        _b.check(_b.lib().illm_sandbox_create(json.dumps(reqs).encode(), dtype.encode(), num_slots, num_pages, page_size, max_seq_len,
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream or 1), ctypes.byref(out)))
        self._ptr = out
        self.cache = SequenceCache.wrap(_b.lib().illm_sandbox_cache(out), self)
        self._dev = ctypes.c_void_p(_b.lib().illm_sandbox_device(out))
        self.B = 0
        self._children = []      # weak references to parts, streams and blocks: they go before the device does

    def _adopt(self, child) -> None:
        import weakref
        self._children.append(weakref.ref(child))

    def __del__(self):
        for ref in getattr(self, "_children", []):
            child = ref()
            if child is not None:
                child._free()
        if getattr(self, "_ptr", None) and _b._lib is not None:
            self.cache = None
            _b._lib.illm_sandbox_free(self._ptr)
        self._ptr = None

    def build(self, family: str, spec: PartSpec) -> _Proxy:
        return _Proxy(self, family, spec)

    def begin_step(self, slots, q_lens, ids=None, want=()):
        """Plan a step for `slots` bringing `q_lens` tokens and upload its description."""
        want = list(want)
        _b.check(_b.lib().illm_sandbox_begin_step(self._ptr, _b.ints(slots), _b.ints(q_lens), len(list(slots)),
                                                  None if ids is None else _b.ints(ids), _b.ints(want), len(want)))
        self.B = len(list(slots))

    def commit_step(self):
        _b.check(_b.lib().illm_sandbox_commit_step(self._ptr))

    def step_view(self) -> StepView:
        import torch
        info = StepInfo()
        _b.check(_b.lib().illm_sandbox_step_info(self._ptr, ctypes.byref(info)))
        return StepView(info, torch.cuda.current_device())

    def cache_view(self, entry: int, writes: bool = True):
        import torch
        c = CacheInfo()
        _b.check(_b.lib().illm_sandbox_cache_info(self._ptr, entry, 1 if writes else 0, ctypes.byref(c)))
        return _cache_view(c, self.B, torch.cuda.current_device())

    def error_word(self) -> int:
        return int(self.step_view().err.item())

    def _take(self, ptr, rows, cols, dtype):
        import torch
        out = torch.empty((rows, cols), dtype=dtype, device="cuda")
        _b.check(_b.lib().illm_copy_device(self._dev, out.data_ptr(), ptr, out.numel() * out.element_size()))
        return out

    def _mixer_forward(self, part, h, entry=0, writes=True):
        h = h.contiguous()
        out, cols = ctypes.c_void_p(), ctypes.c_longlong()
        _b.check(_b.lib().illm_sandbox_mixer_forward(self._ptr, part._ptr, h.data_ptr(), h.shape[0], h.shape[1], entry,
                                                     1 if writes else 0, ctypes.byref(out), ctypes.byref(cols)))
        return self._take(out, h.shape[0], cols.value, self.dtype)

    def _feed_forward_forward(self, part, h):
        h = h.contiguous()
        out, cols = ctypes.c_void_p(), ctypes.c_longlong()
        _b.check(_b.lib().illm_sandbox_ffn_forward(self._ptr, part._ptr, h.data_ptr(), h.shape[0], h.shape[1], ctypes.byref(out),
                                                   ctypes.byref(cols)))
        return self._take(out, h.shape[0], cols.value, self.dtype)

    def _norm_forward(self, part, stream: ResidualStream, rows=None):
        out = ctypes.c_void_p()
        n = stream.x.shape[0] if rows is None else rows.numel()
        _b.check(_b.lib().illm_sandbox_norm_forward(self._ptr, part._ptr, stream._ptr, None if rows is None else rows.data_ptr(),
                                                    n, ctypes.byref(out)))
        return self._take(out, n, stream.x.shape[1], self.dtype)

    def stream(self, x) -> ResidualStream:
        return ResidualStream(self, x)

    def block(self, kind: str, mixer: _Proxy, ffn: _Proxy, norms: Dict[str, _Proxy]):
        out = ctypes.c_void_p()
        _b.check(_b.lib().illm_sandbox_block(self._ptr, kind.encode(), mixer._ptr, ffn._ptr,
                                             json.dumps({r: n._ptr.value for r, n in norms.items()}).encode(), ctypes.byref(out)))
        return _Block(self, out, (mixer, ffn, norms))


def block_norm_roles(kind: str):
    return tuple(_b.call_json(_b.lib().illm_block_norm_roles, kind.encode()))


class _Block:
    def __init__(self, sandbox, ptr, parts):
        self.sandbox, self._ptr, self._parts = sandbox, ptr, parts
        sandbox._adopt(self)

    def _free(self) -> None:
        if getattr(self, "_ptr", None) and _b._lib is not None and getattr(self.sandbox, "_ptr", None):
            _b._lib.illm_block_free(self._ptr)
        self._ptr = None

    def __del__(self):
        self._free()

    def forward(self, stream: ResidualStream, entry=0, writes=True):
        _b.check(_b.lib().illm_sandbox_block_forward(self.sandbox._ptr, self._ptr, stream._ptr, entry, 1 if writes else 0))
