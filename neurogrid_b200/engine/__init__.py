from .runner import ModelRunner, StepEntry, StepError
from .scheduler import Request, Scheduler, StepPlan
