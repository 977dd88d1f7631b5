from .batch import KVGroupStep, StepContext, StepEntry, build_step
from .model import DecoderModel, Run, declared_tensors
from .runner import ModelRunner, StepError
from .scheduler import Request, Scheduled, Scheduler, StepPlan

__all__ = ["DecoderModel", "KVGroupStep", "ModelRunner", "Request", "Run", "Scheduled", "Scheduler", "StepContext",
           "StepEntry", "StepError", "StepPlan", "build_step", "declared_tensors"]
