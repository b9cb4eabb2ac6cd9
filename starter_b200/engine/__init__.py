from .batch import StepContext, StepEntry, plan_step
from .model import DecoderModel, expected_tensors
from .runner import ModelRunner, load_model, random_model, resolve_dtype

__all__ = ["DecoderModel", "ModelRunner", "StepContext", "StepEntry", "expected_tensors",
           "load_model", "plan_step", "random_model", "resolve_dtype"]
