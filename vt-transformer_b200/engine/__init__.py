from .batch import StepContext, StepEntry
from .llm import LLM
from .runner import DeviceStatusError, ModelRunner
from .scheduler import ReqResult, Request, Scheduler, SchedulerConfig, StepResult
