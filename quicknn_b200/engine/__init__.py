"""Model, step function, generation loop and the Python entry point."""
from .batch import StepBatch
from .engine import Engine, StepError
from .generate import GenerationBackend, GenerationResult, PromptError, generate, plan_batches
from .llm import LLM, Conversation
from .model import Model, as_dtype
from ..kernels.lib import KernelError, NonFiniteLogits
from .profile import StepProfiler

__all__ = ["StepBatch", "Engine", "StepError", "GenerationBackend", "GenerationResult", "PromptError",
           "generate", "plan_batches", "LLM", "Conversation", "Model", "as_dtype", "KernelError", "NonFiniteLogits", "StepProfiler"]
