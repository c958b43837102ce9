"""Request records, after the reference's (jllm/engine/request.py:5-41), with sampling
temperature and seed added."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class SamplingParams:
    max_new_tokens: int = 64
    eos_id: Optional[int] = None      # generation stops after this token (which is emitted)
    temperature: float = 0.0          # 0: greedy; > 0: a draw from softmax(logits / temperature)
    seed: Optional[int] = None        # None: the request id
    stop_token_ids: tuple = ()        # more tokens that end the generation (emitted, like eos_id)
    ignore_eos: bool = False          # run to max_new_tokens whatever is sampled (for measurements)

    def __post_init__(self):
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
        self.stop_token_ids = tuple(int(t) for t in self.stop_token_ids)

    def stops_at(self, token: int) -> bool:
        if self.ignore_eos:
            return False
        return (self.eos_id is not None and token == self.eos_id) or token in self.stop_token_ids


@dataclass
class Request:
    request_id: int
    prompt_ids: list
    sampling: SamplingParams
    output_ids: list = field(default_factory=list)
    finished: bool = False
    slot: Optional[int] = None
    preemptions: int = 0
    arrival: float = 0.0
    first_token_time: Optional[float] = None

    @property
    def tokens(self) -> list:
        """Everything known of the sequence: the prompt and what was generated so far."""
        return self.prompt_ids + self.output_ids


@dataclass
class StepEvent:
    request_id: int
    token: int
    finished: bool


@dataclass
class EngineStats:
    admissions: int = 0
    scheduler_loops: int = 0
    steps: int = 0                    # batches run on the device
    prefill_tokens: int = 0           # tokens run that were not single decoded tokens
    decode_tokens: int = 0
    emitted_tokens: int = 0
    cache_hit_blocks: int = 0
    cache_hit_tokens: int = 0
    preemptions: int = 0
    finished: int = 0
    # per step (the reference has no counterpart: its pool is always the worst case and its steps are padded)
    last_step_tokens: int = 0         # tokens that the last step ran
    max_step_tokens: int = 0
    pages_in_use: int = 0             # after the last step, in the fullest pool
    max_pages_in_use: int = 0
    pages_total: int = 0
