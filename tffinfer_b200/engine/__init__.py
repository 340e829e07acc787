from .batch import StepEntry, StepBatch
from .runner import ModelRunner, OutOfPages, RequestError
from .scheduler import Scheduler, Request, StepPlan, PlanEntry, StepOutput
from .engine import Engine, InferRuntime
