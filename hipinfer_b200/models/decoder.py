"""A decoder assembled from a `ModelSpec`: embedding, the layers in the order the spec lists,
final norm, head. It knows parts only through the interfaces of `hipinfer_b200/parts/registry.py`.

It also derives, from the spec alone, what the cache manager has to provide: which steps keep
a cache, how those fall into groups of equal need, and which per-request state each step's
mixer declared.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..cache import CacheGroupSpec
from ..kernels import ops
from ..parts import planes
from ..parts.registry import BuildContext, build_part
from ..parts.spec import ModelSpec, PartSpec


@dataclass(frozen=True)
class StepCachePlan:
    group: int   # cache group of the step's mixer
    slot: int    # which of the group's layer caches
    write: bool  # False: the step reads the cache another step writes


class DecoderModel:
    def __init__(self, spec: ModelSpec, ctx: BuildContext):
        spec.validate()
        self.spec, self.ctx = spec, ctx
        self.embedding = build_part("embedding", spec.embedding, ctx)
        self.layers = [build_part("block", PartSpec(ls.block, {"layer": ls}), ctx, ls.prefix) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, ctx)
        self.head = build_part("head", spec.head, ctx)
        self._plan_cache()

    # ---------------------------------------------------------------- what the cache must provide
    def _plan_cache(self):
        keys: List[tuple] = []
        counts: List[int] = []
        self.cache_plan: List[Optional[StepCachePlan]] = []
        self.state_specs: Dict[Tuple[int, str], Tuple[Tuple[int, ...], torch.dtype]] = {}
        for i, st in enumerate(self.spec.order):
            mixer = self.layers[st.layer].mixer
            need = mixer.cache_need()
            for name, (shape, dtype) in mixer.state_need().items():
                self.state_specs[(i, name)] = (tuple(shape), dtype)
            if need is None:
                if st.reads_cache_of is not None:
                    raise ValueError(f"order[{i}] reads a cache but its mixer keeps none")
                self.cache_plan.append(None)
                continue
            key = need.key()
            if st.reads_cache_of is not None:
                src = self.cache_plan[st.reads_cache_of]
                src_need = self.layers[self.spec.order[st.reads_cache_of].layer].mixer.cache_need()
                if src is None or src_need.key() != key:
                    raise ValueError(f"order[{i}] reads the cache of step {st.reads_cache_of}, whose mixer keeps a "
                                     f"different kind of cache")
                self.cache_plan.append(StepCachePlan(src.group, src.slot, False))
                continue
            if key not in keys:
                keys.append(key)
                counts.append(0)
            g = keys.index(key)
            self.cache_plan.append(StepCachePlan(g, counts[g], True))
            counts[g] += 1
        self.cache_groups = [CacheGroupSpec(f"{k[0]}{k[1] or ''}-h{k[2]}-d{k[3]}" + "".join(f"-{p[0]}" for p in k[4]),
                                            k[0], n, k[2], k[3], k[1], k[4], k[5]) for k, n in zip(keys, counts)]

    # ---------------------------------------------------------------- weights
    def param_specs(self):
        seen, out = set(), []
        for part in [self.embedding] + self.layers + [self.final_norm, self.head]:
            for s in part.param_specs():
                if s.name not in seen:
                    seen.add(s.name)
                    out.append(s)
        return out

    def load(self, tensors) -> None:
        for part in [self.embedding] + self.layers + [self.final_norm, self.head]:
            part.load(tensors)

    def step_weight_bytes(self) -> int:
        """Bytes of weights one decode step reads: every layer as often as the order runs it,
        the final norm and the head matrix once; the embedding table only through the head
        when tied (the reference counts the same, src/api.cu:1522-1537)."""
        return (sum(self.layers[st.layer].weight_bytes() for st in self.spec.order)
                + self.final_norm.weight_bytes() + self.head.weight_bytes())

    # ---------------------------------------------------------------- forward
    def forward(self, batch, storage) -> torch.Tensor:
        """Run the batch's tokens from the cache; logits float32 [len(batch.want_rows), vocab]."""
        x = self.embedding.forward(batch.tokens)
        planes.record(batch, "embedding", x)
        # what a layer leaves for the next reader of x: a sum not yet added (kernels.ops.Pending: the next norm adds
        # it), or that next norm already prepared by the layer's last product (kernels.fast.NormFeed); else None
        carry = None
        order = self.spec.order
        for i, st in enumerate(order):
            layer = self.layers[st.layer]
            cache, state = storage.layer_cache(self.cache_plan[i]), storage.layer_state(i)
            if carry is not None and not layer.takes_pending:
                if isinstance(carry, ops.Pending):
                    carry.finish()
                carry = None
            kw = {}
            if carry is not None:
                kw["pending"] = carry
            if getattr(layer, "takes_next_norm", False) and i + 1 < len(order):
                kw["next_norm"] = getattr(self.layers[order[i + 1].layer], "mixer_norm", None)
            batch.dump_step = i
            left = layer.forward(x, batch, cache, state, **kw)
            carry = left if left is not None and not isinstance(left, torch.Tensor) else None
            if planes.dumping(batch):          # a dumped step leaves nothing pending: x is whole where a plane is taken
                if isinstance(carry, ops.Pending):
                    carry.finish()
                carry = None
                if (i, "after_feed_forward") not in batch.dump:
                    planes.record(batch, "after_feed_forward", x)
        pending = carry if isinstance(carry, ops.Pending) else None
        if batch.n_want == 0:
            if pending is not None:
                pending.finish()
            return torch.empty(0, self.spec.vocab_size, dtype=torch.float32, device=x.device)
        if pending is not None and not self.final_norm.takes_pending:
            pending.finish()
            pending = None
        if pending is not None:
            return self.head.forward(self.final_norm.forward(x, rows=batch.want_rows, pending=pending))
        return self.head.forward(self.final_norm.forward(x, rows=batch.want_rows))
