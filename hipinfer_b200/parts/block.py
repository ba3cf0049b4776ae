"""Arrangements of a layer's parts. "pre_norm": x += mixer(norm(x)); x += feed_forward(norm(x)),
the order of the reference's attn_rows and mlp_rows (src/api.cu:1673, 1712)."""
from __future__ import annotations

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

    def forward(self, x, batch, cache, state):
        # a part may take the norm itself (forward_prenorm) to fuse it into its first kernel;
        # a part without that method gets the normalised rows
        if hasattr(self.mixer, "forward_prenorm"):
            self.mixer.forward_prenorm(self.mixer_norm, x, batch, cache, state)
        else:
            self.mixer.forward(self.mixer_norm.forward(x), x, batch, cache, state)
        if hasattr(self.feed_forward, "forward_prenorm"):
            self.feed_forward.forward_prenorm(self.feed_forward_norm, x, batch)
        else:
            self.feed_forward.forward(self.feed_forward_norm.forward(x), x, batch)


register_part("block", "pre_norm", PreNormBlock)
