"""A small convenience class over the functional entry point: load, generate."""

from __future__ import annotations

from . import engine as eng
from .loading import load_from_path
from .request import SamplingParams


class LLM:
    def __init__(self, model_path=None, *, model=None, dtype="bf16", device="cuda:0", max_num_seqs=4,
                 max_model_len=2048, max_prefill_len=None, block_size=16, num_blocks=None, **more):
        if (model is None) == (model_path is None):
            raise ValueError("give either model_path or model")
        self.model = model if model is not None else load_from_path(model_path, dtype=dtype, device=device)
        self.driver = eng.make_driver(self.model, max_num_seqs=max_num_seqs, max_model_len=max_model_len,
                                      max_prefill_len=max_prefill_len, block_size=block_size, num_blocks=num_blocks,
                                      **more)

    def generate(self, prompts, sampling: SamplingParams | list | None = None) -> list:
        return eng.generate(self.driver, prompts, sampling)

    def add_request(self, prompt_ids, sampling=None) -> int:
        return eng.add_request(self.driver, prompt_ids, sampling)

    def step(self):
        return eng.step(self.driver)

    def has_work(self) -> bool:
        return eng.has_work(self.driver)

    @property
    def stats(self):
        return self.driver.stats
