from .batch import DeviceStep, HostStep, StepEntry
from .llm_engine import LLM, EngineConfig, LLMEngine, StepStats
from .runner import ModelRunner, build_model, load_model
from .scheduler import Scheduler, SchedulerConfig, SchedulerOutput
from .sequence import CompletionOutput, Request, RequestOutput, Sequence, SeqStatus

__all__ = [
    "DeviceStep", "HostStep", "StepEntry", "LLM", "EngineConfig", "LLMEngine", "StepStats",
    "ModelRunner", "build_model", "load_model", "Scheduler", "SchedulerConfig", "SchedulerOutput",
    "CompletionOutput", "Request", "RequestOutput", "Sequence", "SeqStatus",
]
