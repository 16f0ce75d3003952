from .runner import ModelRunner, StepContext, StepEntry, StepError
