from .batch import StepBatch, StepEntry, build_step_batch
from .runner import ModelRunner, StepError

__all__ = ["StepBatch", "StepEntry", "build_step_batch", "ModelRunner", "StepError"]
