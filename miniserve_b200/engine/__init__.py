from .engine import Engine
from .llm import LLM
from .loader import load_model, random_model
from .request import Request, RequestState, SamplingParams
from .scheduler import Plan, PlanRow, Scheduler
from .step import StepError, StepFunction, StepRow

__all__ = ["Engine", "LLM", "Plan", "PlanRow", "Request", "RequestState", "SamplingParams", "Scheduler",
           "StepError", "StepFunction", "StepRow", "load_model", "random_model"]
