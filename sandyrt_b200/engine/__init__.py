from .step import Engine, StepEntry, StepError  # noqa: F401
