from .batch import BatchError, StepContext, StepEntry
from .runner import ModelRunner

__all__ = ["ModelRunner", "StepEntry", "StepContext", "BatchError"]
