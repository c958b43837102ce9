from .batch import BatchBuilder, StepEntry
from .engine import (Driver, add_request, generate, has_work, make_driver, prewarm, start, step, stop, stream)
from .llm import LLM
from .loading import load_from_path, random_model
from .request import EngineStats, Request, SamplingParams, StepEvent
from .runner import Runner, build_runner
from .scheduler import Scheduled, Scheduler

__all__ = ["BatchBuilder", "StepEntry", "Driver", "add_request", "generate", "has_work", "make_driver", "prewarm",
           "start", "step", "stop", "stream", "LLM", "load_from_path", "random_model", "EngineStats", "Request",
           "SamplingParams", "StepEvent", "Runner", "build_runner", "Scheduled", "Scheduler"]
