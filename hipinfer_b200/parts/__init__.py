from .registry import (BuildContext, CacheNeed, Mixer, Part, build_part, register_part, registered_parts, to_compute)
from .spec import LayerSpec, ModelSpec, PartSpec, RunStep, spec_param_specs
from . import attention, block, embedding, feed_forward, norm, rotary  # noqa: F401  (register the kinds)

__all__ = ["BuildContext", "CacheNeed", "Mixer", "Part", "build_part", "register_part", "registered_parts",
           "to_compute", "LayerSpec", "ModelSpec", "PartSpec", "RunStep", "spec_param_specs"]
