"""What every part shares: the registries, the runtime it is built in, and buffers.

A part is chosen by the ``kind`` of a :class:`~qwen_triton_b200.config.PartSpec`
and built with that spec's parameters; it never sees the model it is in.

Interfaces (what a new part must offer):

* every part:  ``expected_tensors(params, prefix) -> {name: TensorSpec}`` (classmethod; no device),
  ``__init__(params, prefix, runtime)``, ``load(source)`` with ``source(name) -> CPU tensor``.
* norm:        ``apply(stream, rows=None) -> Tensor``: folds the pending delta into the
  residual stream and returns the normed rows in the activation dtype.  A norm that sets
  ``offers_scaled_rows`` also takes ``lazy=True`` and may then hand on ``ScaledRows`` (the rows times its
  weight, the rows' factor left to the consumer's product) to a consumer that sets ``takes_scaled_rows``.
* position:    ``__init__(params, runtime)``, ``table(max_positions) -> float32 [P, rotary_dim]`` (cos | sin) or ``None``
  for no encoding, and ``key() -> tuple`` that names the table's content (equal keys share one table).  Column i
  and rotary_dim / 2 + i of a row are the cos and sin of the angle of rotation pair i; the pair is elements
  (i, i + rotary_dim / 2) of a head, or (2i, 2i + 1) if the part has ``interleaved = True``.
* mixer:       ``cache_request() -> KVRequest | StateRequest | None`` and
  ``forward(x, ctx, cache) -> GemmOut`` where ``cache`` is the view of the cache entry this call
  uses (``cache.writable`` tells whether it owns it).
* feed-forward: ``forward(x, ctx) -> GemmOut``.
* block:       ``forward(stream, ctx, cache) -> None``: arranges norm, mixer and feed-forward
  around the residual stream; ``cache_requests()`` says what it keeps per sequence: its mixer's
  request, or a list of requests if it has several such parts (``cache`` is then a tuple of views).
* a part whose work in a step is kernel launches only (no host reads, no shapes that depend on data) may set
  ``graph_safe = True``; a block reports it for the parts it runs.  One-token steps are captured in CUDA graphs
  only if the embedding, every block, the final norm and the head say so.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping

import torch

from ..config.spec import PartSpec
from ..ops.kernels import GemmOut, ScaledRows

_REGISTRIES: dict[str, dict[str, type]] = {"norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "block": {},
                                           "embedding": {}, "head": {}}


def _register(family: str, kind: str, cls: type | None = None):
    def put(c: type) -> type:
        existing = _REGISTRIES[family].get(kind)
        if existing is not None and existing is not c:
            raise ValueError(f"{family} kind {kind!r} is already registered")
        _REGISTRIES[family][kind] = c
        return c

    return put if cls is None else put(cls)


def register_norm(kind: str, cls: type | None = None): return _register("norm", kind, cls)
def register_position(kind: str, cls: type | None = None): return _register("position", kind, cls)
def register_mixer(kind: str, cls: type | None = None): return _register("mixer", kind, cls)
def register_feed_forward(kind: str, cls: type | None = None): return _register("feed_forward", kind, cls)
def register_block(kind: str, cls: type | None = None): return _register("block", kind, cls)
def register_embedding(kind: str, cls: type | None = None): return _register("embedding", kind, cls)
def register_head(kind: str, cls: type | None = None): return _register("head", kind, cls)


def part_class(family: str, spec: PartSpec) -> type:
    try:
        return _REGISTRIES[family][spec.kind]
    except KeyError:
        raise KeyError(f"no {family} of kind {spec.kind!r}; registered: {sorted(_REGISTRIES[family])}") from None


# ----------------------------------------------------------------------------- what a mixer keeps per sequence
@dataclass(frozen=True)
class KVRequest:
    """Keys and values per token: all of them (``window`` None) or the last ``window``."""

    kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateRequest:
    """A fixed-size block per sequence, zeroed when the sequence starts."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ----------------------------------------------------------------------------- buffers
class Workspace:
    """Named device buffers shared by all layers; sized once, before the first step.

    Parts ``declare`` what they need when they are built; ``allocate`` makes one buffer per name
    (the largest request wins); ``view`` hands out the leading elements in the wanted shape.
    No step allocates device memory afterwards.
    """

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self._need: dict[str, tuple[int, torch.dtype]] = {}
        self._buffers: dict[str, torch.Tensor] = {}
        self._views: dict[tuple, torch.Tensor] = {}

    def declare(self, name: str, numel: int, dtype: torch.dtype) -> None:
        old = self._need.get(name)
        if old is not None and old[1] != dtype:
            raise ValueError(f"workspace buffer {name!r} requested as {old[1]} and {dtype}")
        self._need[name] = (max(int(numel), old[0] if old else 0), dtype)

    def allocate(self) -> None:
        for name, (numel, dtype) in self._need.items():
            current = self._buffers.get(name)
            if current is None or current.numel() < numel:
                self._buffers[name] = torch.empty(max(numel, 1), dtype=dtype, device=self.device)
        self._views.clear()

    def view(self, name: str, *shape: int) -> torch.Tensor:
        """The leading elements of a buffer in ``shape``.  Views are kept by (name, shape): a step asks for the same
        few dozen again and again, and making one costs two tensor operations on the host."""
        key = (name, shape)
        found = self._views.get(key)
        if found is not None:
            return found
        if len(self._views) >= 4096:
            self._views.clear()
        found = self._views[key] = self._make_view(name, shape)
        return found

    def _make_view(self, name: str, shape: tuple[int, ...]) -> torch.Tensor:
        count = 1
        for dim in shape:
            count *= dim
        buffer = self._buffers[name]
        if count > buffer.numel():
            raise ValueError(f"workspace buffer {name!r} holds {buffer.numel()} elements, {count} wanted")
        return buffer[:count].view(*shape)

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


@dataclass
class Runtime:
    """Where and how parts are built: device, activation dtype, token limit per step, buffers."""

    device: torch.device
    dtype: torch.dtype                      # activations, matrices and caches: bfloat16 or float32
    max_step_tokens: int
    max_positions: int
    workspace: Workspace
    page_tokens: int = 64
    options: dict[str, Any] = field(default_factory=dict)
    sm_count: int = 0                       # streaming multiprocessors of the device (0: ask it)

    def __post_init__(self) -> None:
        if self.sm_count <= 0:
            from ..ops import kernels
            self.sm_count = kernels.sm_count(self.device)


class DeferredProduct:
    """A product x W^T that has not been launched yet.  Whoever takes it launches it together with what it does
    next (a norm adds it to the stream and prepares itself in the product's epilogue); whoever only wants its
    value calls ``run()``."""

    def __init__(self, linear, x) -> None:
        self.linear, self.x = linear, x

    def run(self) -> GemmOut:
        return self.linear(self.x)

    def value(self) -> torch.Tensor:
        """The finished matrix in float (for tests and host-side use)."""
        return self.run().value()


class ResidualStream:
    """The float residual stream [T, H] with at most one pending addition.

    A part's output is not added at once: it is kept as ``pending`` and folded in by the next norm
    kernel, which reads the stream anyway.  The addition may also be a product that is still to be
    launched (``DeferredProduct``): ``take_deferred`` hands it to a norm that fuses with it, reading
    ``pending`` launches it and gives its result.
    """

    def __init__(self, residual: torch.Tensor) -> None:
        self.residual = residual
        self._pending: GemmOut | DeferredProduct | None = None

    @property
    def pending(self) -> GemmOut | None:
        if isinstance(self._pending, DeferredProduct):
            self._pending = self._pending.run()
        return self._pending

    @pending.setter
    def pending(self, value: GemmOut | None) -> None:
        self._pending = value

    def add(self, delta: "GemmOut | DeferredProduct") -> None:
        if self._pending is not None:
            raise RuntimeError("the residual stream already has a pending addition; apply a norm first")
        self._pending = delta

    def take_deferred(self) -> DeferredProduct | None:
        """The pending addition if it is a product not launched yet (it is then no longer pending), else None."""
        if isinstance(self._pending, DeferredProduct):
            deferred, self._pending = self._pending, None
            return deferred
        return None


TensorSource = Callable[[str], torch.Tensor]


def to_device(tensor: torch.Tensor, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    return tensor.to(device=device, dtype=dtype).contiguous()


def params_of(spec: PartSpec) -> Mapping[str, Any]:
    return spec.params
