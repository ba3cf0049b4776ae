"""Sampling: greedy (the reference's only mode, "Generation is greedy only for now",
README.md:94; argmax_kernel src/kernels.cuh:1925-1931: lowest index on ties, NaN above all,
all -inf gives 0) and temperature sampling, which the reference lacks.

A temperature draw is the arg max of logits / temperature + Gumbel noise, computed on the
device in one pass over the 32-bit logits. The noise of vocabulary entry i is a counter-based
hash of (seed of the request, position of the token being drawn, i): the draw does not depend
on what else is in the batch, on how the prompt was cut, or on a generator's history.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from ..kernels import ops


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0          # 0: greedy
    seed: int = 0
    max_new_tokens: int = 16
    stop_token_ids: Tuple[int, ...] = ()   # generation ends after one of these is produced
    ignore_eos: bool = True           # the reference generates exactly n_new tokens (scripts/hipinfer.py:476-481)

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")


class Sampler:
    def __init__(self, device):
        self.device = device

    def sample_device(self, logits: torch.Tensor, params: Sequence[SamplingParams], positions: Sequence[int]
                      ) -> torch.Tensor:
        """One token per row of float32 logits [R, V], left on the device (int32 [R]);
        positions[r] is the position the new token will take."""
        R = logits.shape[0]
        if all(p.temperature == 0 for p in params):
            return ops.sample(logits, None, None, None)
        host = torch.empty(3, R, dtype=torch.int32, pin_memory=True)
        host[0] = torch.tensor([p.temperature for p in params], dtype=torch.float32).view(torch.int32)
        host[1] = torch.tensor([p.seed & 0x7FFFFFFF for p in params], dtype=torch.int32)
        host[2] = torch.tensor(list(positions), dtype=torch.int32)
        dev = host.to(self.device, non_blocking=True)
        return ops.sample(logits, dev[0].view(torch.float32), dev[1], dev[2])

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], positions: Sequence[int]) -> List[int]:
        """The same, brought to the host (this waits for the device)."""
        if logits.shape[0] == 0:
            return []
        toks = self.sample_device(logits, params, positions).cpu().tolist()
        ops.check_device_status()          # the copy has waited for the step: a kernel that gave up shows here
        return toks
