from .runner import ModelRunner, StepEntry, StepError
