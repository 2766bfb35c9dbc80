"""Architecture-neutral description of a causal language model.

An architecture's typed configuration (for example ``Qwen3Config``) turns
itself into a :class:`ModelSpec`.  Everything below the configuration layer
(parts, cache, engine, weight loader) reads only the spec, so no part knows
which model it is in.

The spec is plain data:

* one :class:`LayerSpec` per set of layer weights, naming the block
  arrangement, the mixer, the feed-forward and the norm by registry kind with
  their sizes and constants as parameters;
* ``schedule``: the order in which layers run.  It is a list of
  :class:`LayerCall`, so a layer may be named twice, and a call may read the
  cache that an earlier call wrote instead of owning one.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Sequence


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by registry ``kind`` with its sizes and constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """Weights and parts of one layer.

    ``prefix`` is the tensor-name prefix of the layer in the checkpoint
    (``model.layers.3``).  ``block`` names the arrangement of the parts
    (``pre_norm``); the arrangement's parameters give the sub-prefixes under
    which each part finds its tensors.  ``extra`` holds, by a name the block
    arrangement knows, the parts a layer has beyond one mixer, one
    feed-forward and one kind of norm: ``pre_norm`` reads ``mixer_norm`` and
    ``feed_forward_norm`` from it (another norm kind in one of the two places);
    an arrangement with a second mixer beside the first finds it there.
    """

    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    norm: PartSpec
    extra: Mapping[str, PartSpec] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``layer``      index into ``ModelSpec.layers`` (whose weights run);
    ``cache_of``   ``None``: this call owns a cache entry of its own (if its
                   mixer asks for one).  An integer ``j``: this call reads the
                   cache entry that schedule position ``j`` (earlier) owns and
                   writes nothing.
    """

    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: PartSpec
    layers: Sequence[LayerSpec]
    schedule: Sequence[LayerCall]
    final_norm: PartSpec
    head: PartSpec
    max_positions: int
    eos_token_ids: tuple[int, ...] = ()

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0:
            raise ValueError("vocab_size and hidden_size must be positive")
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        for pos, call in enumerate(self.schedule):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"schedule[{pos}] names layer {call.layer}, but there are {len(self.layers)} layers")
            if call.cache_of is not None:
                if not 0 <= call.cache_of < pos:
                    raise ValueError(f"schedule[{pos}] reads the cache of position {call.cache_of}, which does not run earlier")
                if self.schedule[call.cache_of].cache_of is not None:
                    raise ValueError(f"schedule[{pos}] reads the cache of position {call.cache_of}, which owns none")
