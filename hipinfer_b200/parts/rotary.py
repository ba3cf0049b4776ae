"""Rotary position encoding as a part: `(head_dim, rotary_dim, theta, scaling)` in, a table of
(cos, sin) per position out, and the operation that rotates q and k and stores k, v in their
pages (the reference's rope_cache_kernel, src/kernels.cuh:1126-1151, does the same on a
contiguous cache).

inv_freq[i] = theta^(-2i/rotary_dim) (scripts/export.py:109-111). Scaling "llama3" rescales
each frequency by its wavelength: kept below original_max/high_freq_factor, divided by
`factor` above original_max/low_freq_factor, interpolated between; the reference copies these
values from another framework's module (scripts/export.py:104-108), here they are computed.
The angle float32(p) * inv_freq is a 32-bit product and cos/sin are evaluated in double on
the device (src/api.cu:1430-1441); the table holds positions [0, ctx.max_model_len).

Pairing is half-split: dimension d pairs with d + rotary_dim/2 (src/kernels.cuh:127-136);
dimensions beyond rotary_dim pass through. A position encoding of kind "none" is rotary_dim 0.
"""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from .registry import Part, register_part


def rope_inv_freq(rotary_dim: int, theta: float, scaling=None) -> torch.Tensor:
    """float32 [rotary_dim / 2], computed in float64 on the host."""
    i = torch.arange(0, rotary_dim, 2, dtype=torch.float64)
    inv = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -i / rotary_dim)
    if scaling is not None:
        kind = scaling.get("rope_type")
        if kind != "llama3":
            raise ValueError(f"rotary scaling of type {kind!r} is not implemented (implemented: 'llama3')")
        factor, low, high = float(scaling["factor"]), float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        orig = float(scaling["original_max_position_embeddings"])
        wavelen = 2.0 * math.pi / inv
        smooth = (orig / wavelen - low) / (high - low)
        blended = (1.0 - smooth) * inv / factor + smooth * inv
        inv = torch.where(wavelen < orig / high, inv, torch.where(wavelen > orig / low, inv / factor, blended))
    return inv.to(torch.float32)


class RotaryEmbedding(Part):
    """params: head_dim, rotary_dim (default head_dim), theta, scaling (None or a dict with
    rope_type "llama3", factor, low_freq_factor, high_freq_factor,
    original_max_position_embeddings), pairing ("half", the only one implemented)."""

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not (0 <= self.rotary_dim <= self.head_dim):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        if params.get("pairing", "half") != "half":
            raise ValueError(f"rotary pairing {params['pairing']!r} is not implemented (implemented: 'half')")
        self.inv_freq = rope_inv_freq(self.rotary_dim, params["theta"], params.get("scaling")) if self.rotary_dim else None
        self.table = None
        if not ctx.is_meta:
            if self.rotary_dim:
                self.table = ops.rope_table(self.inv_freq.to(ctx.device), ctx.max_model_len)
            else:
                self.table = torch.zeros(ctx.max_model_len, 0, 2, dtype=torch.float32, device=ctx.device)

    takes_pending = True

    def rotate_and_store(self, qkv, positions, slot_map, q_out, k_cache, v_cache, n_heads, n_kv_heads, pending=None):
        """q of qkv rotated into q_out; k rotated and v raw into the pages at slot_map (None: no write).
        pending: qkv has yet to be summed from its product's slices (kernels.ops.Pending)."""
        return ops.rope_kv_write(qkv, positions, slot_map, self.table, q_out, k_cache, v_cache, n_heads, n_kv_heads,
                                 self.head_dim, self.rotary_dim, self.ctx.page_size, pending)


    def project_rotate_and_store(self, xn, weight, positions, slot_map, q_out, k_cache, v_cache, n_heads, n_kv_heads) -> bool:
        """rotate_and_store of xn @ weight.T as one kernel (the rotation in the product's epilogue)
        where one exists for these sizes; False: nothing was done. A position part need not have this method."""
        if not self.rotary_dim:
            return False
        return ops.linear_rope_kv_write(xn, weight, positions, slot_map, self.table, q_out, k_cache, v_cache, n_heads,
                                        n_kv_heads, self.head_dim, self.rotary_dim, self.ctx.page_size)


    def norm_project_rotate_and_store(self, lazy_norm, weight, positions, slot_map, q_out, k_cache, v_cache, n_heads,
                                      n_kv_heads) -> bool:
        """rotate_and_store of RMSNorm(x) @ weight.T for a few rows as one kernel (the norm in the product's prologue,
        the rotation in its epilogue); `lazy_norm` is a kernels.ops.LazyNorm. False: nothing was done. Optional, like
        project_rotate_and_store."""
        if not self.rotary_dim:
            return False
        return ops.norm_linear_rope_kv_write(lazy_norm, weight, positions, slot_map, self.table, q_out, k_cache, v_cache,
                                             n_heads, n_kv_heads, self.head_dim, self.rotary_dim, self.ctx.page_size)


register_part("position", "rope", RotaryEmbedding)
