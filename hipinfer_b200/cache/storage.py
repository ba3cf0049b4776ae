"""Device memory behind the cache manager's page ids and state slots.

Per cache group and plane (keys, values, or what else the group's mixers keep per token) one
tensor [layer cache, page, head, page_size, width] in the compute element type: a (page, head)
pair is one contiguous run of page_size * width elements, which is what the attention kernels
stream. Per declared state one tensor [state slot, *shape]. The pools start zeroed: a kernel
that loads a whole page and masks the tail must never meet a NaN pattern there.

The reference allocates `[layer][slot][kv head][max_seq][head_dim]` once (src/api.cu:1409-1411).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .manager import CacheGroupSpec


@dataclass
class LayerCache:
    planes: Dict[str, torch.Tensor]      # plane name -> [page, head, page_size, width]
    group: int
    write: bool

    @property
    def k(self) -> torch.Tensor:
        return self.planes["k"]

    @property
    def v(self) -> torch.Tensor:
        return self.planes["v"]


class CacheStorage:
    def __init__(self, groups: Sequence[CacheGroupSpec], num_pages: Sequence[int], page_size: int, dtype, device,
                 state_specs: Dict[Tuple[int, str], Tuple[Tuple[int, ...], torch.dtype]], num_state_slots: int):
        self.groups, self.page_size, self.dtype = list(groups), page_size, dtype
        self.kv = [{name: torch.zeros(g.n_layers, n, heads, page_size, width, dtype=dtype, device=device)
                    for name, heads, width in g.planes} for g, n in zip(self.groups, num_pages)]
        self.state: Dict[Tuple[int, str], torch.Tensor] = {
            key: torch.zeros((num_state_slots,) + tuple(shape), dtype=dt, device=device)
            for key, (shape, dt) in state_specs.items()}
        self._layer_caches: Dict[Tuple[int, int, bool], LayerCache] = {}
        self._by_step: Dict[int, Dict[str, torch.Tensor]] = {}
        for (step, name), t in self.state.items():
            self._by_step.setdefault(step, {})[name] = t

    def layer_cache(self, plan) -> Optional[LayerCache]:
        if plan is None:
            return None
        key = (plan.group, plan.slot, plan.write)
        if key not in self._layer_caches:
            self._layer_caches[key] = LayerCache({name: t[plan.slot] for name, t in self.kv[plan.group].items()},
                                                 plan.group, plan.write)
        return self._layer_caches[key]

    def layer_state(self, step: int) -> Dict[str, torch.Tensor]:
        return self._by_step.get(step, {})

    def zero_state_slot(self, slot: int) -> None:
        """A request admitted to `slot` starts from zero state."""
        for t in self.state.values():
            t[slot].zero_()

    def bytes_per_token(self) -> int:
        return sum(g.elements_per_token() for g in self.groups) * torch.empty((), dtype=self.dtype).element_size()

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for g in self.kv for t in g.values()) + \
            sum(t.numel() * t.element_size() for t in self.state.values())
