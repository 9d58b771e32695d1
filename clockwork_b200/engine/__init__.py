from .llm_engine import LLMEngine
from .loading import load_model, random_model
from .scheduler import ScheduledPortion, Scheduler, SchedulerOutput, SchedulerStats
from .sequence import RequestOutput, Sequence, SequenceStatus
from .step import ModelRunner, StepEntry

__all__ = [
    "LLMEngine", "load_model", "random_model", "ScheduledPortion", "Scheduler", "SchedulerOutput",
    "SchedulerStats", "RequestOutput", "Sequence", "SequenceStatus", "ModelRunner", "StepEntry",
]
