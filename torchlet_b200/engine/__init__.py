from .runner import ModelRunner, OutOfPages, StepContext, StepEntry

__all__ = ["ModelRunner", "OutOfPages", "StepContext", "StepEntry"]
