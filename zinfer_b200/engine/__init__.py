from .batch import KVGroupStep, StepContext, StepEntry, build_step
from .model import DecoderModel, Run, declared_tensors
from .runner import ModelRunner, StepError

__all__ = ["DecoderModel", "KVGroupStep", "ModelRunner", "Run", "StepContext", "StepEntry", "StepError",
           "build_step", "declared_tensors"]
