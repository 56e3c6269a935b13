from .build import LoadedModel, load_model, make_runner
from .llm_engine import LLMEngine
from .request import Request, RequestOutput, ScheduledChunk, SequenceState, SequenceStatus
from .runner import ModelRunner, StepEntry, StepError
from .scheduler import Scheduler

__all__ = [n for n in dir() if not n.startswith("_")]
