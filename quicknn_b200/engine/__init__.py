"""Model, step function, generation loop and the Python entry point."""
from .batch import StepBatch
from .engine import Engine, StepError
from .model import Model, as_dtype

__all__ = ["StepBatch", "Engine", "StepError", "Model", "as_dtype"]
