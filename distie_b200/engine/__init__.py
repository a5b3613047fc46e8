"""Step function, scheduler and the Python entry point."""

from .batch import BatchEntry, lay_out
from .scheduler import Emission, ScheduledSeq, Scheduler, SeqState, Sequence, StepPlan

__all__ = [
    "BatchEntry",
    "Emission",
    "ScheduledSeq",
    "Scheduler",
    "SeqState",
    "Sequence",
    "StepPlan",
    "lay_out",
]
