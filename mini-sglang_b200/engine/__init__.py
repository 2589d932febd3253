from .args import EngineArgs, ServerArgs
from .step import ModelRunner, StepEntry


def __getattr__(name):
    if name == "Engine":
        from .engine import Engine
        return Engine
    if name in ("Scheduler", "Req"):
        from . import scheduler
        return getattr(scheduler, name)
    raise AttributeError(name)
