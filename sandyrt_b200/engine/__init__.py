from .step import Engine, SampleRow, StepEntry, StepError  # noqa: F401
