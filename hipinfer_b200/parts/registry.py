"""Registries of part kinds, and the interfaces the parts implement.

A part is built from `(params, ctx, prefix)`: `params` is its PartSpec's dictionary, `ctx` the
`BuildContext` (compute element type, device, page size, longest sequence), `prefix` the
tensor-name prefix of its layer. No part knows which model it is in.

Interfaces (duck-typed; the base classes below give the defaults):

  every part      param_specs() -> [ParamSpec]; load(tensors: {name: tensor}); weight_bytes()
  norm            forward(x_f32 [T, H], rows=None) -> normalised rows in ctx.act_dtype
  position        the object a mixer of kind "attention" asks for; see parts/rotary.py
  mixer           cache_need() -> CacheNeed | None; state_need() -> {name: (shape, dtype)};
                  forward(xn, x, batch, cache, state): ADDS its output into the float32
                  residual stream x [T, H]; `cache` is its LayerCache (or None), `state` the
                  {name: tensor [slots, *shape]} it declared (index with batch.req_state_slot)
  feed_forward    forward(xn, x, batch): adds its output into x
  block           forward(x, batch, cache, state): one layer in its arrangement
  embedding       forward(tokens int32 [T]) -> x float32 [T, H]
  head            forward(xn [W, H]) -> logits float32 [W, V]
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch


@dataclass(frozen=True)
class BuildContext:
    dtype: torch.dtype            # compute element type of activations and the cache
    device: Any
    page_size: int = 16
    max_model_len: int = 2048

    @staticmethod
    def meta() -> "BuildContext":
        return BuildContext(torch.float32, "meta")

    @property
    def is_meta(self) -> bool:
        return str(self.device) == "meta"


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps per token in the paged cache. `kind` names the retention rule ("full": everything;
    "window": the last `window` tokens; or one added with cache.register_retention, which reads `extra`).
    By default the layer gets keys "k" and values "v" of kv_heads x head_dim; `planes` ((name, heads, width), ...)
    asks for other tensors instead (a latent, keys and values of different widths). Layers whose needs are equal
    share a group: one page pool and one block table per request."""

    kind: str
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    planes: Tuple[Tuple[str, int, int], ...] = ()
    extra: Tuple[Tuple[str, object], ...] = ()

    def key(self) -> tuple:
        return (self.kind, self.window, self.kv_heads, self.head_dim, self.planes, self.extra)


class Part:
    # A mixer's or feed-forward's forward() adds its result into the residual rows x it is given.
    # It may instead return a kernels.ops.Pending: a sum not yet added into x, which the next
    # reader of x adds on its way. A norm (or block) whose forward() has a `pending` argument
    # sets takes_pending; for any other part the sum is finished before the part runs.
    takes_pending = False

    def __init__(self, params: Dict[str, Any], ctx: BuildContext, prefix: str = ""):
        self.params, self.ctx, self.prefix = params, ctx, prefix

    def param_specs(self):
        return []

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass

    def weight_bytes(self) -> int:
        return 0


class Mixer(Part):
    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        return {}


_REGISTRIES: Dict[str, Dict[str, Callable]] = {k: {} for k in
                                               ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")}


def register_part(role: str, kind: str, cls: Callable) -> None:
    """Register class `cls` as part kind `kind` for `role` (one of the registry names)."""
    if role not in _REGISTRIES:
        raise KeyError(f"unknown part role {role!r}; roles: {sorted(_REGISTRIES)}")
    _REGISTRIES[role][kind] = cls


def build_part(role: str, spec, ctx: BuildContext, prefix: str = ""):
    reg = _REGISTRIES[role]
    if spec.kind not in reg:
        raise KeyError(f"no {role} of kind {spec.kind!r} is registered; registered: {sorted(reg)}")
    return reg[spec.kind](spec.params, ctx, prefix)


def registered_parts(role: str) -> List[str]:
    return sorted(_REGISTRIES[role])


def to_compute(t: torch.Tensor, ctx: BuildContext) -> torch.Tensor:
    """A stored weight as the compute path wants it: float32 for the 32-bit path; as stored
    (bfloat16 stays bfloat16, a tensor stored in 32-bit stays so) for the bfloat16 path."""
    if ctx.dtype == torch.float32 and t.dtype != torch.float32:
        return t.to(torch.float32)
    return t.contiguous()
