"""Arrangements of norm, mixer and feed-forward around the residual stream.

``pre_norm``: h += mixer(norm(h)); h += feed_forward(norm(h)) (qwen_triton/models/core.py:126-152).
Each addition is left pending on the stream and folded in by the next norm kernel.
"""
from __future__ import annotations

from ..config.spec import LayerSpec
from ..weights.tensors import TensorSpec
from .base import ResidualStream, Runtime, part_class, register_block


@register_block("pre_norm")
class PreNormBlock:
    def __init__(self, layer: LayerSpec, runtime: Runtime) -> None:
        names = self._names(layer)
        norms = self._norm_specs(layer)
        self.mixer_norm = part_class("norm", norms[0])(norms[0].params, names["mixer_norm"], runtime)
        self.feed_forward_norm = part_class("norm", norms[1])(norms[1].params, names["feed_forward_norm"], runtime)
        self.mixer = part_class("mixer", layer.mixer)(layer.mixer.params, names["mixer"], runtime)
        self.feed_forward = part_class("feed_forward", layer.feed_forward)(layer.feed_forward.params,
                                                                           names["feed_forward"], runtime)

    @staticmethod
    def _names(layer: LayerSpec) -> dict[str, str]:
        p = layer.block.params
        return {key: f"{layer.prefix}.{p.get(key, key)}" for key in ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm")}

    @staticmethod
    def _norm_specs(layer: LayerSpec):
        """The norm in front of the mixer and the one in front of the feed-forward: ``layer.norm`` for both unless
        ``layer.extra`` names another kind for one of them."""
        return layer.extra.get("mixer_norm", layer.norm), layer.extra.get("feed_forward_norm", layer.norm)

    @classmethod
    def expected_tensors(cls, layer: LayerSpec) -> dict[str, TensorSpec]:
        names = cls._names(layer)
        out: dict[str, TensorSpec] = {}
        norms = cls._norm_specs(layer)
        out.update(part_class("norm", norms[0]).expected_tensors(norms[0].params, names["mixer_norm"]))
        out.update(part_class("norm", norms[1]).expected_tensors(norms[1].params, names["feed_forward_norm"]))
        out.update(part_class("mixer", layer.mixer).expected_tensors(layer.mixer.params, names["mixer"]))
        out.update(part_class("feed_forward", layer.feed_forward).expected_tensors(layer.feed_forward.params,
                                                                                   names["feed_forward"]))
        return out

    def cache_requests(self):
        """What this block keeps per sequence: its mixer's request.  (A block with several such parts returns a
        list, and its ``forward`` then gets a tuple of cache views in the same order.)"""
        return self.mixer.cache_request()

    def parts(self) -> tuple:
        """The parts this block runs in a step."""
        return (self.mixer_norm, self.feed_forward_norm, self.mixer, self.feed_forward)

    @property
    def graph_safe(self) -> bool:
        """True if a one-token step through this block only launches kernels (every part says so of itself)."""
        return all(getattr(part, "graph_safe", False) for part in self.parts())

    def load(self, source) -> None:
        for part in self.parts():
            part.load(source)

    @staticmethod
    def _normed(norm, stream: ResidualStream, consumer):
        """The consumer's input: ``ScaledRows`` where the norm offers them and the consumer takes them."""
        if getattr(norm, "offers_scaled_rows", False) and getattr(consumer, "takes_scaled_rows", False):
            return norm.apply(stream, lazy=True)
        return norm.apply(stream)

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        x = self._normed(self.mixer_norm, stream, self.mixer)
        stream.add(self.mixer.forward(x, ctx, cache))
        x = self._normed(self.feed_forward_norm, stream, self.feed_forward)
        stream.add(self.feed_forward.forward(x, ctx))
