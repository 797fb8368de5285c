from .batch import BatchBuilder, StepBatch, StepEntry
from .model import CausalLM
from .scheduler import Request, Scheduler

__all__ = ["BatchBuilder", "StepBatch", "StepEntry", "CausalLM", "Request", "Scheduler"]
