"""Arrangements of a layer's parts. "pre_norm": x += mixer(norm(x)); x += feed_forward(norm(x)),
the order of the reference's attn_rows and mlp_rows (src/api.cu:1673, 1712)."""
from __future__ import annotations

from ..kernels import ops
from .registry import Part, build_part, register_part


class PreNormBlock(Part):
    """params: layer (the LayerSpec)."""

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        ls = params["layer"]
        self.mixer_norm = build_part("norm", ls.mixer_norm, ctx, prefix)
        self.mixer = build_part("mixer", ls.mixer, ctx, prefix)
        self.feed_forward_norm = build_part("norm", ls.feed_forward_norm, ctx, prefix)
        self.feed_forward = build_part("feed_forward", ls.feed_forward, ctx, prefix)
        self.parts = [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def param_specs(self):
        return [s for p in self.parts for s in p.param_specs()]

    def load(self, tensors):
        for p in self.parts:
            p.load(tensors)

    def weight_bytes(self):
        return sum(p.weight_bytes() for p in self.parts)

    takes_pending = True

    @staticmethod
    def _normed(norm, x, pending):
        if pending is None:
            return norm.forward(x)
        if norm.takes_pending:
            return norm.forward(x, pending=pending)
        pending.finish()
        return norm.forward(x)

    def forward(self, x, batch, cache, state, pending=None):
        """pending: a sum the layer before has yet to add into x. Returns what this layer leaves
        to be added (None when x is complete)."""
        left = self.mixer.forward(self._normed(self.mixer_norm, x, pending), x, batch, cache, state)
        pending = left if isinstance(left, ops.Pending) else None
        left = self.feed_forward.forward(self._normed(self.feed_forward_norm, x, pending), x, batch)
        return left if isinstance(left, ops.Pending) else None


register_part("block", "pre_norm", PreNormBlock)
