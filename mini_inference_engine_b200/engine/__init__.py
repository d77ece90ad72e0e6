from .batch import BatchBuilder, BatchRow
from .scheduler import Scheduler
from .sequence import Sequence, Status

__all__ = ["BatchBuilder", "BatchRow", "Scheduler", "Sequence", "Status", "LLMEngine", "RequestOutput", "ModelRunner"]


def __getattr__(name):
    if name in ("LLMEngine", "RequestOutput"):
        from . import engine
        return getattr(engine, name)
    if name == "ModelRunner":
        from .runner import ModelRunner
        return ModelRunner
    raise AttributeError(name)
