from .api import Engine
from .batch import StepContext, make_context, pack_step
from .model import Model, expected_tensors

__all__ = ["Engine", "StepContext", "make_context", "pack_step", "Model", "expected_tensors"]
