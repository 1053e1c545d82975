from .step import KVView, ModelRunner, OutOfPages, StateView, StepBatch, StepContext, StepEntry
from .workspace import Workspace
from .loading import load_model, make_runner, parse_dtype
from .scheduler import Request, RequestRefused, Scheduled, Scheduler
from .pipeline import Pipeline

__all__ = ["KVView", "ModelRunner", "OutOfPages", "StateView", "StepBatch", "StepContext", "StepEntry", "Workspace", "load_model", "make_runner", "parse_dtype", "Request", "RequestRefused", "Scheduled", "Scheduler", "Pipeline"]
