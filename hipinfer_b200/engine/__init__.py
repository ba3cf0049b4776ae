from .batch import StepBatch, StepEntry, build_step_batch
from .runner import ModelRunner, StepError
from .scheduler import AdmissionError, Request, Scheduled, Scheduler

__all__ = ["StepBatch", "StepEntry", "build_step_batch", "ModelRunner", "StepError", "AdmissionError", "Request",
           "Scheduled", "Scheduler"]
