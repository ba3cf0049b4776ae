from .decoder import DecoderModel, StepCachePlan
from . import llama  # noqa: F401  (registers LlamaForCausalLM)
from .llama import llama_spec

__all__ = ["DecoderModel", "StepCachePlan", "llama_spec"]
