from .step import KVView, ModelRunner, OutOfPages, StateView, StepBatch, StepContext, StepEntry
from .workspace import Workspace
from .loading import load_model, make_runner, parse_dtype

__all__ = ["KVView", "ModelRunner", "OutOfPages", "StateView", "StepBatch", "StepContext", "StepEntry", "Workspace", "load_model", "make_runner", "parse_dtype"]
