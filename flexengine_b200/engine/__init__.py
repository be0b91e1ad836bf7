from .step import ModelRunner, StepContext, StepEntry

__all__ = ["ModelRunner", "StepContext", "StepEntry"]
