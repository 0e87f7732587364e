from .step import Engine, StepEntry, StepError, OutOfPages
