"""Device memory behind the cache manager's page ids and state slots.

Per cache group one tensor [layer cache, K/V, page, kv head, page_size, head_dim] in the
compute element type: a (page, kv head) pair is one contiguous run of page_size * head_dim
elements, which is what the attention kernels stream. Per declared state one tensor
[state slot, *shape]. The pools start zeroed: a kernel that loads a whole page and masks the
tail must never meet a NaN pattern there.

The reference allocates `[layer][slot][kv head][max_seq][head_dim]` once (src/api.cu:1409-1411).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .manager import CacheGroupSpec


@dataclass
class LayerCache:
    k: torch.Tensor      # [page, kv head, page_size, head_dim]
    v: torch.Tensor
    group: int
    write: bool


class CacheStorage:
    def __init__(self, groups: Sequence[CacheGroupSpec], num_pages: Sequence[int], page_size: int, dtype, device,
                 state_specs: Dict[Tuple[int, str], Tuple[Tuple[int, ...], torch.dtype]], num_state_slots: int):
        self.groups, self.page_size, self.dtype = list(groups), page_size, dtype
        self.kv = [torch.zeros(g.n_layers, 2, n, g.kv_heads, page_size, g.head_dim, dtype=dtype, device=device)
                   for g, n in zip(self.groups, num_pages)]
        self.state: Dict[Tuple[int, str], torch.Tensor] = {
            key: torch.zeros((num_state_slots,) + tuple(shape), dtype=dt, device=device)
            for key, (shape, dt) in state_specs.items()}
        self._by_step: Dict[int, Dict[str, torch.Tensor]] = {}
        for (step, name), t in self.state.items():
            self._by_step.setdefault(step, {})[name] = t

    def layer_cache(self, plan) -> Optional[LayerCache]:
        if plan is None:
            return None
        t = self.kv[plan.group][plan.slot]
        return LayerCache(t[0], t[1], plan.group, plan.write)

    def layer_state(self, step: int) -> Dict[str, torch.Tensor]:
        return self._by_step.get(step, {})

    def zero_state_slot(self, slot: int) -> None:
        """A request admitted to `slot` starts from zero state."""
        for t in self.state.values():
            t[slot].zero_()

    def bytes_per_token(self) -> int:
        return sum(g.elements_per_token() for g in self.groups) * torch.empty((), dtype=self.dtype).element_size()

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv) + \
            sum(t.numel() * t.element_size() for t in self.state.values())
