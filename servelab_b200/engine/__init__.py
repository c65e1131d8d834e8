"""Engine: request state, scheduler, batch descriptor, step function, entry point."""

from .outputs import CompletionOutput, RequestOutput
from .scheduler import ScheduledPortion, Scheduler, SchedulerOutput
from .sequence import RequestMetrics, Sequence, SequenceStatus

__all__ = ["CompletionOutput", "RequestMetrics", "RequestOutput", "ScheduledPortion",
           "Scheduler", "SchedulerOutput", "Sequence", "SequenceStatus"]
