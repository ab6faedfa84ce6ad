"""Interfaces and registries of the parts that a layer is put together from.

A part is built from a `PartSpec` (its sizes and constants) and a `Runtime` (device and
compute dtype); it never learns which model it is in.  It declares the tensors it needs
under names of its own (`tensors()`), receives them (`load()`), and runs on the tokens of
one step (`forward`).  The kinds are looked up by name in the registries below, so a test
or a user can add a mixer, feed-forward, norm, position encoding or block arrangement
without touching this package:

    @register_mixer("my_mixer")
    class MyMixer(Mixer): ...

The reference has the same seam one level lower: modules take their sizes as constructor
arguments and own their weights by name (`AttentionModule`, `LlamaFFNModule`,
src/core/graph.h:84-123, src/core/graph.cpp:57-79).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

import torch

from ..config.base import ConfigError, PartSpec


@dataclass
class Runtime:
    """Where and in which precision a model runs.  `dtype` is the dtype of activations,
    matrices and cache pages: bfloat16 (serving) or float32 (everything in true 32-bit)."""

    device: torch.device
    dtype: torch.dtype
    page_size: int = 64

    @property
    def is_f32(self) -> bool:
        return self.dtype == torch.float32


@dataclass
class TensorDecl:
    """A tensor that a part needs.  `init`: "matrix" -> N(0, 0.02); "norm" -> 1 + N(0, 0.02);
    "int" -> an integer table (kept int32).  Used by the loader to check shapes and by the
    random-weights writer."""

    shape: Tuple[int, ...]
    init: str = "matrix"


# ---- what a mixer may ask of the cache


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every position (or of the last `window` positions) of a sequence."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedState:
    """State of a fixed size per sequence, zeroed when a slot is handed out."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    """Base of all parts."""

    def __init__(self, spec: PartSpec, runtime: Optional[Runtime]):
        self.spec = spec
        self.rt = runtime

    def tensors(self) -> Dict[str, TensorDecl]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receive the declared tensors (on the device, in their stored dtype or float32 in
        the float32 mode) and bring them into the form the kernels want."""


class Norm(Part):
    def forward(self, stream: "ResidualStream", rows=None) -> torch.Tensor:
        """Fold the stream's pending addition in and return the normed rows in the compute
        dtype; `rows` (int32 tensor) restricts it to those rows."""
        raise NotImplementedError


class PositionEncoding(Part):
    # True: `encode_and_store` also takes the packed projection as unreduced slices of a split
    # matrix product (`kernels.ops.SplitKPartials`) and adds them up itself.  False (default): it
    # always gets a finished tensor.
    takes_partials = False

    def prepare(self) -> None:
        """Build device tables; called once after construction on a device."""

    def rotation_table(self):
        """(cos/sin table float32 [positions, rot_dim/2, 2] or None, rot_dim) if all this encoding
        does is the rotate-half rotation of the first rot_dim channels of every Q and K head by
        angles from that table (rot_dim 0: nothing at all), so that a mixer whose kernel can do that
        itself may skip `encode_and_store`; None (default) for any other encoding."""
        return None

    def encode_and_store(self, qkv, geometry, ctx, kv):
        """Encode positions into the Q and K heads of the packed projection `qkv` and store the
        new K and V in the cache (if `kv.writes`).  Returns the tensor that holds the encoded
        queries in its first heads * head_dim columns: `qkv` itself (encoded in place) or, when
        `qkv` arrived as unreduced slices of a split matrix product, a new tensor."""
        raise NotImplementedError


class Mixer(Part):
    # True promises that a one-token-per-sequence step launches the same kernels with the same
    # arguments whenever the batch size is the same (everything that varies is read from device
    # memory), so the engine may capture it in a CUDA graph.  A mixer that reads host-side
    # fields of the step context (q_lens, past, ...) leaves it False.
    graph_safe = False

    # True when tokens appended behind a sequence's real tokens in a step change nothing that is
    # kept (they may leave keys and values behind the sequence's length in its own pages, which the
    # next tokens overwrite) and nothing the real tokens get back, and when a step of many tokens
    # of one sequence launches the same kernels whenever the token count is the same.  The engine
    # then pads single prompts to whole buckets of tokens and replays them from captured graphs.
    pad_safe = False

    def cache_request(self):
        """`PagedKV`, `FixedState` or None."""
        return None

    def forward(self, h: torch.Tensor, ctx, cache, writes: bool) -> torch.Tensor:
        """h [T, H] in the compute dtype -> [T, H]; `cache` is the view of this entry's
        storage for the step (a `KVView`, a `StateView` or None)."""
        raise NotImplementedError

    def forward_deferred(self, h, ctx, cache, writes):
        """Like `forward`, but the result may be the unreduced slices of a split matrix product
        (`kernels.ops.SplitKPartials`), for a caller that only adds it to the residual stream
        (`ResidualStream.add` takes both).  By default the same as `forward`."""
        return self.forward(h, ctx, cache, writes)


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError

    def forward_deferred(self, h, ctx):
        """See `Mixer.forward_deferred`."""
        return self.forward(h, ctx)


class Block:
    """An arrangement of norms, a mixer and a feed-forward around the residual stream."""

    def __init__(self, mixer: Mixer, ffn: FeedForward, norms: Dict[str, Norm]):
        self.mixer, self.ffn, self.norms = mixer, ffn, norms

    @staticmethod
    def norm_roles():
        """Names of the norms this arrangement needs (keys of LayerSpec.names)."""
        return ()

    def forward(self, stream: "ResidualStream", ctx, cache, writes: bool) -> None:
        raise NotImplementedError


class ResidualStream:
    """The float32 residual stream [T, H] with at most one addition pending.  A part's output
    is not added at once: the next norm adds it while it reads the row anyway (one kernel for
    add + norm), which is also where the sum is rounded: never, it stays float32."""

    def __init__(self, x: torch.Tensor):
        self.x = x
        self.pending = None     # a tensor [T, H], or kernels.ops.SplitKPartials of that shape

    def add(self, delta) -> None:
        """`delta`: a tensor in the compute dtype, or the unreduced slices of a split matrix
        product; `ops.add_rmsnorm` and `ops.residual_add` take either."""
        if self.pending is not None:
            self.flush()
        self.pending = delta

    def flush(self) -> torch.Tensor:
        if self.pending is not None:
            from ..kernels import ops
            ops.residual_add(self.x, self.pending)
            self.pending = None
        return self.x


# ---- registries

_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}}


def _register(family: str, kind: str):
    def deco(cls):
        _REGISTRIES[family][kind] = cls
        return cls
    return deco


def register_mixer(kind): return _register("mixer", kind)
def register_feed_forward(kind): return _register("feed_forward", kind)
def register_norm(kind): return _register("norm", kind)
def register_position(kind): return _register("position", kind)
def register_block(kind): return _register("block", kind)


def lookup(family: str, kind: str):
    reg = _REGISTRIES[family]
    if kind not in reg:
        raise ConfigError(f"unknown {family} kind '{kind}'; registered: {', '.join(sorted(reg))}")
    return reg[kind]


def build_part(family: str, spec: PartSpec, runtime: Optional[Runtime]):
    return lookup(family, spec.kind)(spec, runtime)
