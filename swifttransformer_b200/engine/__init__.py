from .step import ModelRunner, OutOfPages, StepContext, StepEntry, StepError

__all__ = ["ModelRunner", "OutOfPages", "StepContext", "StepEntry", "StepError"]
