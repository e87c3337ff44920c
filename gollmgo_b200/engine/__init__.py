from .batch import BatchBuilder, StepBatch, StepEntry
from .scheduler import QueueFull, RequestTooLong, Scheduled, Scheduler, SchedulerOutput
from .sequence import InvalidTransition, SeqState, Sequence

__all__ = ["BatchBuilder", "StepBatch", "StepEntry", "QueueFull", "RequestTooLong", "Scheduled",
           "Scheduler", "SchedulerOutput", "InvalidTransition", "SeqState", "Sequence",
           "Engine", "ModelRunner", "RequestOutput", "TokenResult"]


def __getattr__(name):
    if name in ("Engine", "RequestOutput", "TokenResult"):
        from . import llm_engine
        return getattr(llm_engine, name)
    if name == "ModelRunner":
        from .runner import ModelRunner
        return ModelRunner
    raise AttributeError(name)
