"""RMSNorm: y = w * (x / sqrt(mean(x^2) + eps)), plain weight (not 1 + w), computed in
32-bit from the 32-bit residual stream and rounded once (src/kernels.cuh:108-125 rounds x*r
to fp16 before the product with w, to match a half-precision framework)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import ParamSpec
from .registry import Part, register_part, to_compute


class RMSNorm(Part):
    """params: name (tensor name relative to the prefix), size, eps."""

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.size, self.eps = int(params["size"]), float(params["eps"])
        self.name = prefix + params["name"]
        self.weight = None

    def param_specs(self):
        return [ParamSpec(self.name, (self.size,), init="ones")]

    def load(self, tensors):
        self.weight = to_compute(tensors[self.name], self.ctx)

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    takes_pending = True

    def lazy(self, x, feed=None):
        """The norm of x left to its consumer (kernels.ops.LazyNorm) where a consumer could fold it into its product, else
        None. feed: what `feed()` gave and the product that wrote x has filled; the consumer then needs no prologue."""
        if self.weight is None or not ops.lazy_norm_applies(x, self.weight, self.ctx.dtype):
            return None
        ok = feed is not None and feed.filled and feed.weight is self.weight
        return ops.LazyNorm(x, self.weight, self.eps, self.ctx.dtype, feed if ok else None)

    def feed(self, rows):
        """Buffers that the product which writes this norm's input rows may fill on its way (x times this norm's weight in
        bf16, and the pieces of the rows' sums of squares), for steps of a few rows; else None. See kernels.fast.NormFeed."""
        if self.weight is None or self.ctx.dtype != torch.bfloat16:
            return None
        return ops.make_norm_feed(self.weight, self.eps, rows)

    def forward(self, x, rows=None, out=None, pending=None):
        """pending: a sum that has yet to be added into x (it is added before the norm)."""
        M = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = torch.empty(M, self.size, dtype=self.ctx.dtype, device=x.device)
        return ops.rmsnorm(x, self.weight, self.eps, out, rows, pending)


register_part("norm", "rmsnorm", RMSNorm)
