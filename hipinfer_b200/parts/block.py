"""Arrangements of a layer's parts. "pre_norm": x += mixer(norm(x)); x += feed_forward(norm(x)),
the order of the reference's attn_rows and mlp_rows (src/api.cu:1673, 1712).

A block kind declares its slots (`SLOTS`: slot name -> registry role) and builds the parts the
`LayerSpec` gives under those names; a layer that gives other names, or lacks one, is refused
with a message. Every block has an attribute `mixer`: the part whose `cache_need()` and
`state_need()` the cache manager serves."""
from __future__ import annotations

from ..kernels import ops
from .registry import Part, build_part, register_part


def build_slots(block: Part, layer, slots, ctx, prefix) -> list:
    """Builds the parts of `layer` (a LayerSpec) for the slots {name: role} of a block kind, sets each as the
    attribute of its slot name on `block`, and returns them in the slots' order."""
    extra = sorted(set(layer.parts) - set(slots))
    if extra:
        raise ValueError(f"layer {layer.prefix!r}: block {layer.block!r} has no part {extra}; its parts are {sorted(slots)}")
    built = []
    for name, role in slots.items():
        part = build_part(role, layer.part(name), ctx, prefix)
        setattr(block, name, part)
        built.append(part)
    return built


class PreNormBlock(Part):
    """params: layer (the LayerSpec)."""

    SLOTS = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.parts = build_slots(self, params["layer"], self.SLOTS, ctx, prefix)

    def param_specs(self):
        return [s for p in self.parts for s in p.param_specs()]

    def load(self, tensors):
        for p in self.parts:
            p.load(tensors)

    def weight_bytes(self):
        return sum(p.weight_bytes() for p in self.parts)

    takes_pending = True

    @staticmethod
    def _normed(norm, x, pending, consumer):
        if pending is None:
            # a few rows: a consumer that says so gets the norm unevaluated and folds it into its first product
            if getattr(consumer, "takes_lazy_norm", False) and hasattr(norm, "lazy"):
                lazy = norm.lazy(x)
                if lazy is not None:
                    return lazy
            return norm.forward(x)
        if norm.takes_pending:
            return norm.forward(x, pending=pending)
        pending.finish()
        return norm.forward(x)

    def forward(self, x, batch, cache, state, pending=None):
        """pending: a sum the layer before has yet to add into x. Returns what this layer leaves
        to be added (None when x is complete)."""
        left = self.mixer.forward(self._normed(self.mixer_norm, x, pending, self.mixer), x, batch, cache, state)
        pending = left if isinstance(left, ops.Pending) else None
        left = self.feed_forward.forward(self._normed(self.feed_forward_norm, x, pending, self.feed_forward), x, batch)
        return left if isinstance(left, ops.Pending) else None


register_part("block", "pre_norm", PreNormBlock)
