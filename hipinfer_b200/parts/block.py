"""Arrangements of a layer's parts. "pre_norm": x += mixer(norm(x)); x += feed_forward(norm(x)),
the order of the reference's attn_rows and mlp_rows (src/api.cu:1673, 1712).

A block kind declares its slots (`SLOTS`: slot name -> registry role) and builds the parts the
`LayerSpec` gives under those names; a layer that gives other names, or lacks one, is refused
with a message. Every block has an attribute `mixer`: the part whose `cache_need()` and
`state_need()` the cache manager serves."""
from __future__ import annotations

from ..kernels import ops
from . import planes
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
    takes_next_norm = True      # forward() accepts next_norm=: the norm that reads x after this layer (the next layer's first)

    @staticmethod
    def _normed(norm, x, pending, consumer, feed=None):
        if pending is None:
            # a few rows: a consumer that says so gets the norm unevaluated and folds it into its first product
            if getattr(consumer, "takes_lazy_norm", False) and hasattr(norm, "lazy"):
                lazy = norm.lazy(x, feed) if feed is not None else norm.lazy(x)
                if lazy is not None:
                    return lazy
            return norm.forward(x)
        if norm.takes_pending:
            return norm.forward(x, pending=pending)
        pending.finish()
        return norm.forward(x)

    @staticmethod
    def _feed_of(norm, producer, rows):
        """Buffers for `norm` that `producer` (the part whose last product writes the norm's input) may fill, or None."""
        if norm is None or not getattr(producer, "takes_norm_feed", False) or not hasattr(norm, "feed"):
            return None
        return norm.feed(rows)

    def forward(self, x, batch, cache, state, pending=None, next_norm=None):
        """pending: what the layer before left: a sum it has yet to add into x (kernels.ops.Pending), or the first
        norm of this layer prepared by its last product (kernels.fast.NormFeed). Returns what this layer leaves in
        the same way (None when x is complete and nothing is prepared)."""
        if planes.dumping(batch):
            return self._forward_dumped(x, batch, cache, state, pending)
        feed_in = None
        if pending is not None and not isinstance(pending, ops.Pending):
            feed_in, pending = pending, None
        rows = x.shape[0]
        xn = self._normed(self.mixer_norm, x, pending, self.mixer, feed_in)
        feed = self._feed_of(self.feed_forward_norm, self.mixer, rows)
        left = (self.mixer.forward(xn, x, batch, cache, state, norm_feed=feed) if feed is not None
                else self.mixer.forward(xn, x, batch, cache, state))
        pending = left if isinstance(left, ops.Pending) else None
        xn = self._normed(self.feed_forward_norm, x, pending, self.feed_forward, feed)
        feed = self._feed_of(next_norm, self.feed_forward, rows)
        left = (self.feed_forward.forward(xn, x, batch, norm_feed=feed) if feed is not None
                else self.feed_forward.forward(xn, x, batch))
        if isinstance(left, ops.Pending):
            return left
        return feed if feed is not None and feed.filled else None

    def _forward_dumped(self, x, batch, cache, state, pending):
        """The same layer with every sum finished and every norm evaluated where a plane is recorded (parts/planes.py)."""
        if isinstance(pending, ops.Pending):
            pending.finish()
        xn = self.mixer_norm.forward(x)
        planes.record(batch, "mixer_norm", xn)
        left = self.mixer.forward(xn, x, batch, cache, state)
        if isinstance(left, ops.Pending):
            left.finish()
        planes.record(batch, "after_mixer", x)
        xn = self.feed_forward_norm.forward(x)
        planes.record(batch, "feed_forward_norm", xn)
        left = self.feed_forward.forward(xn, x, batch)
        if isinstance(left, ops.Pending):
            left.finish()
        planes.record(batch, "after_feed_forward", x)
        return None


register_part("block", "pre_norm", PreNormBlock)
