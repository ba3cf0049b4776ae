"""The attention mixer: grouped-query causal attention over the paged cache.

In the reference's order (src/api.cu:1668-1691): one fused projection whose rows are
[q (Hq D); k (Hkv D); v (Hkv D)] (scripts/export.py:278), the position encoding on q and k and
the cache write, attention with scale 1/sqrt(D) (src/api.cu:600) where query head h reads kv
head h // G (src/kernels.cuh:1347) and key kp is visible to a query at qp iff kp <= qp
(1416-1418), then the output projection added into the residual stream (epilogue 1,
src/kernels.cuh:881-889). The projection's result stays in 32-bit until after the rotation, so
q and k are rounded once. `window` > 0 hides keys at or before qp - window (the reference only
guards against models that need it, src/api.cu:1296-1300); such a mixer's cache need is of
kind "window", so its pages can be given back as the window passes them.

Every size is a parameter: n_heads, n_kv_heads, head_dim, hidden_size, window, scale, the
position encoding's PartSpec, and the four tensor names.
"""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..weights import ParamSpec
from . import planes
from .registry import CacheNeed, Mixer, build_part, register_part, to_compute


class AttentionMixer(Mixer):
    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        p = params
        self.hidden = int(p["hidden_size"])
        self.n_heads, self.n_kv_heads, self.head_dim = int(p["n_heads"]), int(p["n_kv_heads"]), int(p["head_dim"])
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"attention: {self.n_heads} heads are not a multiple of {self.n_kv_heads} kv heads")
        self.window = int(p.get("window") or 0)
        self.scale = float(p.get("scale") or 1.0 / math.sqrt(self.head_dim))
        self.names = {k: prefix + p.get(k + "_name", f"self_attn.{k}_proj.weight") for k in ("q", "k", "v", "o")}
        self.position = build_part("position", p["position"], ctx, prefix)
        self.wqkv = self.wo = None

    def param_specs(self):
        Hq, Hkv, D, H = self.n_heads, self.n_kv_heads, self.head_dim, self.hidden
        return [ParamSpec(self.names["q"], (Hq * D, H)), ParamSpec(self.names["k"], (Hkv * D, H)),
                ParamSpec(self.names["v"], (Hkv * D, H)), ParamSpec(self.names["o"], (H, Hq * D))]

    def load(self, tensors):
        q, k, v = (to_compute(tensors[self.names[n]], self.ctx) for n in "qkv")
        dt = q.dtype if q.dtype == k.dtype == v.dtype else torch.float32
        self.wqkv = ops.Weight(torch.cat([q.to(dt), k.to(dt), v.to(dt)], 0).contiguous())
        self.wo = ops.Weight(to_compute(tensors[self.names["o"]], self.ctx))

    def weight_bytes(self):
        return self.wqkv.nbytes + self.wo.nbytes

    def cache_need(self):
        return CacheNeed("window" if self.window else "full", self.n_kv_heads, self.head_dim, self.window)

    takes_lazy_norm = True
    takes_norm_feed = True     # forward() accepts norm_feed=: buffers of the norm that reads x next (see parts/block.py)

    def forward(self, xn, x, batch, cache, state, norm_feed=None):
        T = xn.shape[0]
        Hq, Hkv, D = self.n_heads, self.n_kv_heads, self.head_dim
        q = torch.empty(T, Hq * D, dtype=self.ctx.dtype, device=xn.device)
        slot_map = batch.slot_maps[cache.group] if cache.write else None
        if isinstance(xn, ops.LazyNorm):     # a few rows: norm, projection, rotation and cache write as one kernel
            folded = getattr(self.position, "norm_project_rotate_and_store", None)
            if folded is not None and folded(xn, self.wqkv, batch.positions, slot_map, q, cache.k, cache.v, Hq, Hkv):
                return self._attend_and_project(q, x, batch, cache, norm_feed)
            xn = xn.materialize()
        fused = getattr(self.position, "project_rotate_and_store", None)    # many rows: the rotation in the product's epilogue
        if fused is not None and fused(xn, self.wqkv, batch.positions, slot_map, q, cache.k, cache.v, Hq, Hkv):
            return self._attend_and_project(q, x, batch, cache, norm_feed)
        qkv = torch.empty(T, (Hq + 2 * Hkv) * D, dtype=torch.float32, device=xn.device)
        pending = ops.linear_deferred(xn, self.wqkv, qkv)      # a few rows: the rotation adds the product's slices
        if pending is not None and not self.position.takes_pending:
            pending.finish()
            pending = None
        if pending is None:
            self.position.rotate_and_store(qkv, batch.positions, slot_map, q, cache.k, cache.v, Hq, Hkv)
        else:
            self.position.rotate_and_store(qkv, batch.positions, slot_map, q, cache.k, cache.v, Hq, Hkv, pending=pending)
        return self._attend_and_project(q, x, batch, cache, norm_feed)

    def _attend_and_project(self, q, x, batch, cache, norm_feed=None):
        T = q.shape[0]
        Hq, Hkv, D = self.n_heads, self.n_kv_heads, self.head_dim
        att = torch.empty(T, Hq * D, dtype=self.ctx.dtype, device=q.device)
        ops.attention(q, cache.k, cache.v, batch, cache.group, att, Hq, Hkv, D, self.ctx.page_size, self.window,
                      self.scale)
        planes.record(batch, "q", q)
        planes.record(batch, "attention", att)
        if ops.linear_add_rows(att, self.wo, x, norm_feed):            # a few rows: added in the product's epilogue
            return None
        return ops.linear_deferred(att, self.wo, x, accumulate=True)   # the next norm may add it


register_part("mixer", "attention", AttentionMixer)
