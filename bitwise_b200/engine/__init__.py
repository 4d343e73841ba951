from .step import OutOfPages, StepEntry, StepError, Stepper

__all__ = ["OutOfPages", "StepEntry", "StepError", "Stepper"]
