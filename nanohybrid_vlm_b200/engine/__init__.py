from .batch import BatchBuilder, StepBatch, StepItem
from .llm_engine import LLM, LLMEngine, RequestMetrics, StepStats
from .model import CausalLM
from .runner import ModelRunner
from .scheduler import SchedulePlan, Scheduler
from .sequence import Sequence, SequenceStatus

__all__ = ["BatchBuilder", "StepBatch", "StepItem", "LLM", "LLMEngine", "RequestMetrics", "StepStats", "CausalLM",
           "ModelRunner", "SchedulePlan", "Scheduler", "Sequence", "SequenceStatus"]
