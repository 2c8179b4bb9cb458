"""What a part is, and the registries parts are chosen from.

A model is put together from parts of seven kinds: ``mixer`` (attention here), ``feed_forward``
(dense or routed experts), ``norm``, ``position`` (position encoding), ``block`` (how a layer
arranges the other four), ``embedding`` (token ids to the residual stream) and ``head`` (the residual
stream to logits).  A part takes every size and constant as a constructor parameter, names
the checkpoint tensors it needs (``tensor_specs``), receives them (``load``) and runs on the tokens
of one step (``forward``).  No part knows which model it is in; an architecture is a function from
its configuration to a ``ModelSpec`` that names parts and parameters layer by layer.

Registering a new part: ``@register("mixer", "my_mixer") class MyMixer(Mixer): ...`` in any module
that is imported before the model is built.  The framework's files do not change.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

KINDS = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")
_REGISTRY: dict[str, dict[str, type]] = {k: {} for k in KINDS}


def register(kind: str, name: str) -> Callable[[type], type]:
    if kind not in _REGISTRY:
        raise KeyError(f"unknown part kind {kind!r}; kinds: {KINDS}")

    def deco(cls: type) -> type:
        _REGISTRY[kind][name] = cls
        return cls

    return deco


def registered(kind: str) -> list[str]:
    return sorted(_REGISTRY[kind])


def make(kind: str, choice) -> Any:
    """Instantiate ``(name, params)`` of the given kind."""
    name, params = choice
    try:
        cls = _REGISTRY[kind][name]
    except KeyError:
        raise KeyError(f"no {kind} part named {name!r}; registered: {registered(kind)}") from None
    return cls(**params)


# ------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor a part needs.

    ``kind``: ``"matrix"`` is held in the model's compute dtype (bfloat16 or float32); ``"f32"`` is
    held in float32 whatever the compute dtype (norm gains, router gate and bias: a tensor stored in
    32-bit stays so); ``"i32"`` integer tables.  ``init`` tells the random-weights mode how to draw
    it: ``"normal"`` N(0, 0.02), ``"gain"`` 1 + U(-0.1, 0.1), ``"bias"`` U(-0.05, 0.05).
    """
    name: str
    shape: tuple[int, ...]
    kind: str = "matrix"
    init: str = "normal"


@dataclass(frozen=True)
class CacheStream:
    """One paged tensor a mixer keeps per token: ``heads`` rows of ``width`` elements in the activation
    dtype.  Softmax attention keeps two (keys and values); a mixer that attends over one latent vector
    keeps one; widths need not be equal."""
    name: str
    heads: int
    width: int


@dataclass(frozen=True)
class Retention:
    """Which cached positions a request's future queries can still read.  The cache manager gives a
    page back as soon as no position of it is needed any more, and never asks again about a page it
    gave back, so what is needed may only shrink as the request grows.  The base keeps everything."""

    def needed_ranges(self, length: int) -> list[tuple[int, int | None]]:
        """Half-open position ranges ``(lo, hi)`` that queries at positions ``>= length`` may read, given
        that ``length`` tokens are cached; ``hi`` None: no upper end.  The last range must be open."""
        return [(0, None)]


@dataclass(frozen=True)
class KeepAll(Retention):
    pass


@dataclass(frozen=True)
class Window(Retention):
    """A query at position p reads the keys ``p - window + 1 .. p`` only."""
    window: int = 1

    def needed_ranges(self, length):
        return [(max(0, length - self.window + 1), None)]


@dataclass(frozen=True)
class CacheSpec:
    """A mixer's need of paged per-token storage: its streams and what is retained.  Layers with equal
    specs form one group of the cache manager: they share pages ids and block tables."""
    streams: tuple[CacheStream, ...]
    retention: Retention = KeepAll()

    @property
    def window(self) -> int | None:
        return getattr(self.retention, "window", None)


def KVCacheSpec(n_kv_heads: int, head_dim: int, window: int | None = None) -> CacheSpec:
    """Keys and values of softmax attention: two streams of ``n_kv_heads`` x ``head_dim``; ``window`` None:
    all keys are kept, W: only the last W positions."""
    return CacheSpec((CacheStream("k", n_kv_heads, head_dim), CacheStream("v", n_kv_heads, head_dim)),
                     KeepAll() if window is None else Window(int(window)))


class LayerCache:
    """What a mixer sees of the cache in one step: its own pages of every stream it declared
    (``streams[name]`` ``[num_pages, heads, page_size, width]``) and its group's block table (int32
    ``[requests in the step, pages per request]``, -1 where a page was given back).  ``write`` False:
    this layer reads a cache another layer wrote.  ``k`` / ``v`` are the streams of those names."""

    def __init__(self, k=None, v=None, page_size: int = 0, block_table=None, write: bool = True, streams=None):
        self.streams = dict(streams) if streams is not None else {"k": k, "v": v}
        self.page_size, self.block_table, self.write = page_size, block_table, write

    @property
    def k(self):
        return self.streams["k"]

    @property
    def v(self):
        return self.streams["v"]


@dataclass
class StepContext:
    """Per-step facts every part may read.  All tensors are on the device; ``T`` tokens in the step.

    The tokens of request row ``r`` are the rows ``req_start[r] .. req_start[r+1]`` of every activation,
    in position order; its per-request state (a mixer's ``state_spec``) is row ``req_slot[r]`` of each
    state tensor.  A part that reads only these device arrays (no ``host``, no ``.item()``) may declare
    itself ``graph_safe``; one part that is not turns captured decode steps off for the whole model.
    ``positions`` carries one coordinate per position axis; the step function feeds every axis the
    token's text position (a caller cannot hand a token several coordinates: image inputs are not built)."""
    n_tokens: int
    positions: torch.Tensor            # int32 [T, axes]   position fed to the position encoding
    tok_pos: torch.Tensor              # int32 [T]         index of the token in its request's cache
    tok_req: torch.Tensor              # int32 [T]         row of the token's request in this step
    req_slot: torch.Tensor             # int32 [R]         state slot of each request of the step
    req_start: torch.Tensor            # int32 [R+1]       first token row of each request
    req_len_after: torch.Tensor        # int32 [R]         tokens cached once the step is done
    status: torch.Tensor               # int32 [4]         device error words
    dtype: torch.dtype                 # activation dtype
    max_new_tokens_per_req: int = 0    # largest portion in the step
    max_len_after: int = 0             # largest req_len_after (host copy, for launch sizing)
    host: dict = field(default_factory=dict)   # host copies of the small arrays, for parts that need them
    # how the step's tokens fall into requests, for mixers that treat single tokens and portions
    # differently: rows of requests that bring exactly one token, and (request row, first token row,
    # tokens) of the others.  None: derived from host["req_start"], or one portion holding everything.
    dec_tok: torch.Tensor | None = None        # int32 [n_dec] token rows (device)
    n_dec: int = 0
    spans: list | None = None
    work: dict = field(default_factory=dict)   # per-step scratch shared by the layers (tile lists and the like)


class Part:
    """Base of every part."""

    # True when ``forward`` reads nothing from the host (no ``ctx.host``, no ``.item()``, no shapes that
    # depend on data): a decode step of such parts can be captured in a CUDA graph and replayed.
    graph_safe = False

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def load(self, fetch: Callable[[str], torch.Tensor]) -> None:
        """Receive the tensors named in ``tensor_specs``: ``fetch(name)`` returns the device tensor in
        the dtype its kind asks for."""

    def children(self) -> list["Part"]:
        return []


class Norm(Part):
    def forward(self, h: torch.Tensor, delta, out, rows=None, store_h=True) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    """Turns positions into what a mixer consumes.  ``rotary_tables`` returns ``(inv_freq float32
    [rd/2], pair_axis int32 [rd/2] or None, rotary_dim, n_axes)`` or None when nothing is rotated."""

    n_axes = 1

    def rotary_tables(self, device):
        return None


class Mixer(Part):
    def cache_spec(self) -> CacheSpec | None:
        """What the mixer keeps per token in pages (streams and retention); None: nothing."""
        return None

    def state_spec(self) -> dict[str, tuple[tuple[int, ...], torch.dtype]]:
        """Per-request state of fixed size: name -> (shape, dtype).  The cache manager keeps one row per
        state slot, zeroed when a request takes the slot."""
        return {}

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache | None,
                state: dict[str, torch.Tensor]) -> torch.Tensor:
        """``x`` [T, hidden] in the activation dtype -> the layer's contribution to the residual stream,
        [T, hidden] or [T, S, hidden] (S partial results the next norm sums in order)."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    """Token ids to the float32 residual stream: ``forward(ids int32 [T], ctx) -> [T, hidden]``."""

    def forward(self, ids: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    """The residual stream to logits: ``forward(h, pending, rows, ctx)`` adds the last layer's pending
    contribution for the wanted token rows ``rows`` (int32) and returns float32 ``[len(rows), vocab]``."""

    def forward(self, h: torch.Tensor, pending, rows: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """Arrangement of norm, mixer and feed-forward in one layer.  ``forward`` takes the residual stream
    ``h`` (float32) and the not-yet-added contribution of the layer before, and returns the new pending
    contribution; every addition to ``h`` happens inside a norm kernel."""

    def forward(self, h, pending, ctx, cache, state):
        raise NotImplementedError
