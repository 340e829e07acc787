from .batch import StepEntry, StepBatch, build_step_batch
from .runner import ModelRunner, OutOfPages, RequestError
