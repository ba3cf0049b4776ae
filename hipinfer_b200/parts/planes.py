"""Named planes of a step, for finding the first (layer, sub-step) at which an engine and a reference part ways.

    planes = {}
    logits = runner.step(entries, dump=planes)      # the step runs eagerly, with every sum finished where it is recorded
    planes[(3, "after_mixer")]                       # float32 copy [rows, hidden] of the residual stream after step 3's mixer

Keys are (index into the model's run order, name); the names, in the order they are written within a layer:
"mixer_norm" (the rows the mixer reads), "q" (attention: queries after the position encoding), "attention" (its
output before the output projection), "after_mixer" (residual stream), "feed_forward_norm", "activation" (SwiGLU:
silu(gate) * up), "after_feed_forward" (residual stream). Before the layers: (-1, "embedding"). The reference has the
same aid for its own graph: hi_prefill_debug dumps every layer's intermediates (src/api.cu:1614-1664, 1868-1879),
scripts/layer_diff.py names the planes and reports the first that differs.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

PLANES = ("mixer_norm", "q", "attention", "after_mixer", "feed_forward_norm", "activation", "after_feed_forward")


def record(batch, name: str, tensor: torch.Tensor) -> None:
    """Called by parts: keeps a float32 copy of `tensor` under (batch.dump_step, name) when the step is being dumped."""
    if batch is not None and getattr(batch, "dump", None) is not None:
        batch.dump[(batch.dump_step, name)] = tensor.detach().float().clone()


def dumping(batch) -> bool:
    return batch is not None and getattr(batch, "dump", None) is not None


def first_difference(got: Dict[Tuple[int, str], torch.Tensor], want: Dict[Tuple[int, str], torch.Tensor],
                     tolerance: float) -> Optional[Tuple[Tuple[int, str], float]]:
    """The first plane (in run order, then in the order of PLANES) present in both whose largest |difference| exceeds
    `tolerance` times the largest |value| of the wanted plane, with that relative difference; None when all agree."""
    rank = {n: i for i, n in enumerate(("embedding",) + PLANES)}
    for key in sorted((k for k in got if k in want), key=lambda k: (k[0], rank.get(k[1], len(rank)))):
        g, w = got[key].float().cpu(), want[key].float().cpu()
        if g.shape != w.shape:
            return key, float("inf")
        scale = float(w.abs().max()) or 1.0
        rel = float((g - w).abs().max()) / scale
        if not (rel <= tolerance):
            return key, rel
    return None
