from .batch import StepContext, StepEntry
from .executor import Executor, StepError
from .model import Model

__all__ = ["StepContext", "StepEntry", "Executor", "StepError", "Model"]
