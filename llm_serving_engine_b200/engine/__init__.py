from .scheduler import GenerationRequest, Scheduler
from .step import StepContext, StepEntry, StepRunner

__all__ = ["GenerationRequest", "Scheduler", "StepContext", "StepEntry", "StepRunner"]
