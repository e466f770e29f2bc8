from .model import DecoderModel, expected_tensors
from .step import Engine, MemoryBudgetError, StepContext, StepEntry, StepError

__all__ = ["DecoderModel", "Engine", "MemoryBudgetError", "StepContext", "StepEntry", "StepError",
           "expected_tensors"]
