"""The engine: step function, scheduler, trace replay, and the Python entry point."""

from .scheduler import FinishReason, Phase, Scheduler, SchedulerConfig, Sequence, StepPlan
