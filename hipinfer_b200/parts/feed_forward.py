"""The dense feed-forward: SwiGLU. act = silu(xn Wg^T) * (xn Wu^T), silu(g) = g / (1 + e^-g)
(src/kernels.cuh:100-105), out = act Wd^T added into the residual stream
(src/api.cu:1708-1718). Gate and up are one matrix with rows interleaved in groups of 16
(16 gate rows, 16 up rows, ...), so that a tile of the product holds matching pairs and the
activation can be applied in the product's epilogue; the reference stores its weights the
same way for the same reason (scripts/export.py:97-101). The loader side of that choice is
here: `load` interleaves, nothing outside this file sees the layout.

params: hidden_size, intermediate_size, and the three tensor names.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import ParamSpec
from . import planes
from .registry import Part, register_part, to_compute

GROUP = 16


class SwiGLU(Part):
    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        if self.inter % GROUP:
            raise ValueError(f"SwiGLU: intermediate_size {self.inter} must be a multiple of {GROUP} "
                             f"(gate and up rows are interleaved in groups of {GROUP})")
        self.names = {k: prefix + params.get(k + "_name", f"mlp.{k}_proj.weight") for k in ("gate", "up", "down")}
        self.wgu = self.wdown = None

    def param_specs(self):
        return [ParamSpec(self.names["gate"], (self.inter, self.hidden)),
                ParamSpec(self.names["up"], (self.inter, self.hidden)),
                ParamSpec(self.names["down"], (self.hidden, self.inter))]

    def load(self, tensors):
        g, u = to_compute(tensors[self.names["gate"]], self.ctx), to_compute(tensors[self.names["up"]], self.ctx)
        dt = g.dtype if g.dtype == u.dtype else torch.float32
        I, H = self.inter, self.hidden
        gu = torch.stack([g.to(dt).reshape(I // GROUP, GROUP, H), u.to(dt).reshape(I // GROUP, GROUP, H)], 1)
        self.wgu = ops.Weight(gu.reshape(2 * I, H).contiguous())
        self.wdown = ops.Weight(to_compute(tensors[self.names["down"]], self.ctx))

    def weight_bytes(self):
        return self.wgu.nbytes + self.wdown.nbytes

    takes_lazy_norm = True
    takes_norm_feed = True     # forward() accepts norm_feed=: buffers of the norm that reads x next (see parts/block.py)

    def forward(self, xn, x, batch, norm_feed=None):
        act = torch.empty(xn.shape[0], self.inter, dtype=self.ctx.dtype, device=xn.device)
        if isinstance(xn, ops.LazyNorm):     # a few rows: the norm in the gate/up product's prologue
            if not ops.norm_linear_swiglu(xn, self.wgu, act, GROUP):
                ops.linear_swiglu(xn.materialize(), self.wgu, act, GROUP)
        else:
            ops.linear_swiglu(xn, self.wgu, act, GROUP)
        planes.record(batch, "activation", act)
        if ops.linear_add_rows(act, self.wdown, x, norm_feed):            # a few rows: added in the product's epilogue
            return None
        return ops.linear_deferred(act, self.wdown, x, accumulate=True)   # the next norm may add it


register_part("feed_forward", "swiglu", SwiGLU)
