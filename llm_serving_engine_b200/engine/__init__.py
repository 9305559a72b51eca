from .scheduler import IterationScheduler, RequestState, plan_iteration, resolve_page_pressure
from .step import StepContext, StepEntry, StepRunner

__all__ = ["IterationScheduler", "RequestState", "StepContext", "StepEntry", "StepRunner",
           "plan_iteration", "resolve_page_pressure"]
