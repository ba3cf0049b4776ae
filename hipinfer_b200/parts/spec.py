"""The description of a model as data: which parts make up each layer, with which constants,
and in which order the layers run. An architecture is a function from its configuration to a
`ModelSpec`; the engine builds the parts from the registries in `hipinfer_b200/parts/registry.py`
and knows nothing else about the architecture.

- A `PartSpec` names a registered kind and carries every size and constant the part needs.
- A `LayerSpec` names the arrangement of a block (for instance "pre_norm") and gives the block's
  parts as a mapping from slot name to `PartSpec`. Which slots there are is the block kind's
  business ("pre_norm": mixer_norm, mixer, feed_forward_norm, feed_forward; a block with norms
  after its mixer and feed-forward as well, or one norm shared by both, is another block kind
  with other slots and needs no change here). Chosen layer by layer: layers of one model may differ.
- `order` is the list of steps in which layers run. A step may name a layer that an earlier
  step named (its weights are used again, with a cache of its own), or say that its mixer
  reads the cache of an earlier step instead of keeping one.

The reference has one hard-wired graph (src/api.cu:1728-1765, 1891-1952).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    prefix: str                       # tensor-name prefix of the layer, e.g. "model.layers.3."
    block: str                        # arrangement kind
    parts: Mapping[str, PartSpec]     # slot name -> part; the block kind says which slots it has

    def part(self, slot: str) -> PartSpec:
        try:
            return self.parts[slot]
        except KeyError:
            raise KeyError(f"layer {self.prefix!r}: block {self.block!r} asks for a part {slot!r}; the layer gives "
                           f"{sorted(self.parts)}") from None


@dataclass(frozen=True)
class RunStep:
    layer: int
    reads_cache_of: Optional[int] = None  # index into `order` of the earlier step whose cache is read


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    order: Tuple[RunStep, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        if not self.order:
            raise ValueError("ModelSpec.order is empty")
        for i, st in enumerate(self.order):
            if not (0 <= st.layer < len(self.layers)):
                raise ValueError(f"order[{i}] names layer {st.layer}; there are {len(self.layers)} layers")
            if st.reads_cache_of is not None:
                j = st.reads_cache_of
                if not (0 <= j < i):
                    raise ValueError(f"order[{i}] reads the cache of step {j}, which is not an earlier step")
                if self.order[j].reads_cache_of is not None:
                    raise ValueError(f"order[{i}] reads the cache of step {j}, which keeps none of its own")


def spec_param_specs(spec: ModelSpec):
    """Every tensor the model of `spec` needs (built on the 'meta' context: no device memory)."""
    from .registry import BuildContext
    from ..models.decoder import DecoderModel

    return DecoderModel(spec, BuildContext.meta()).param_specs()
