"""A single-GPU inference engine for NVIDIA B200 (sm_100a) in the shape of
alec-tschantz/jax-vllm: model folder in, generated tokens out, for Qwen3 dense.

    from jax_vllm_b200 import load_from_path, make_driver, add_request, step, has_work
"""

from . import registry
from .config import EngineConfig
from .engine import (LLM, SamplingParams, StepEvent, add_request, generate, has_work, load_from_path, make_driver,
                     prewarm, random_model, start, step, stop, stream)
from .weights import WeightError, write_model_folder

__all__ = ["registry", "EngineConfig", "LLM", "SamplingParams", "StepEvent", "add_request", "generate", "has_work",
           "load_from_path", "make_driver", "prewarm", "random_model", "start", "step", "stop", "stream",
           "WeightError", "write_model_folder"]
