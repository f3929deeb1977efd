from .llm import LLMEngine
from .loading import load_model
from .metrics import RequestRecord, percentile, summarise
from .scheduler import Request, RequestRefused, Scheduler, SeqState, SequenceState
from .step import FROM_DEVICE, Runner, StepEntry, StepError, StepResult

__all__ = ["LLMEngine", "Request", "RequestRecord", "RequestRefused", "Runner", "Scheduler",
           "FROM_DEVICE", "SeqState", "SequenceState", "StepEntry", "StepError", "StepResult", "load_model",
           "percentile", "summarise"]
