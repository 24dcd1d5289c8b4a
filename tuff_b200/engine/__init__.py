from .batch import BatchError, StepContext, StepEntry
from .runner import ModelRunner
from .scheduler import Request, RequestStatus, Scheduler, SchedulerError, StepPlan

__all__ = ["ModelRunner", "StepEntry", "StepContext", "BatchError", "Scheduler", "Request", "RequestStatus",
           "SchedulerError", "StepPlan", "Engine"]


def __getattr__(name):
    if name == "Engine":
        from .engine import Engine
        return Engine
    raise AttributeError(name)
