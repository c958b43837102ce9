"""Settings of the engine that are not the model's: cache, batching, precision."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

DTYPES = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp32": torch.float32, "float32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {name}")
        return name
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {name!r}") from None


@dataclass(frozen=True)
class EngineConfig:
    """Names follow the reference's `make_driver` (jllm/engine/engine.py:63-71) where it has
    them: max_num_seqs, max_model_len, max_prefill_len, block_size, num_blocks, dtype."""

    dtype: torch.dtype = torch.bfloat16
    max_num_seqs: int = 4                 # requests live at a time
    max_model_len: int = 2048             # prompt + generated tokens of one request
    max_prefill_len: Optional[int] = None  # longest prompt accepted (None: max_model_len)
    block_size: int = 16                  # tokens in a page of the cache
    num_blocks: Optional[int] = None      # pages in each pool (None: by memory_fraction, else the worst case:
                                          # max_num_seqs * pages of max_model_len)
    memory_fraction: Optional[float] = None   # with num_blocks None: the pool takes this share of the device memory
                                          # that is free when the driver is made (never more than the worst case)
    max_tokens_per_step: int = 2048       # token budget of one step (decoded tokens + prompt portions)
    prefix_cache: bool = True
    decode_split_size: int = 256          # key positions per split of a decoded token's attention
    cuda_graphs: bool = True              # replay decode-only steps from captured graphs
    device: str = "cuda:0"

    def __post_init__(self):
        if self.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("dtype must be torch.bfloat16 or torch.float32")
        for k in ("max_num_seqs", "max_model_len", "block_size", "max_tokens_per_step", "decode_split_size"):
            if getattr(self, k) < 1:
                raise ValueError(f"{k} must be positive")
        if self.max_prefill_len is not None and self.max_prefill_len > self.max_model_len:
            raise ValueError("max_prefill_len must be <= max_model_len")
        if self.num_blocks is not None and self.num_blocks < 1:
            raise ValueError("num_blocks must be positive")
        if self.memory_fraction is not None and not 0.0 < self.memory_fraction <= 1.0:
            raise ValueError("memory_fraction must lie in (0, 1]")

    @property
    def prompt_limit(self) -> int:
        return self.max_prefill_len if self.max_prefill_len is not None else self.max_model_len

    @property
    def pages_per_request(self) -> int:
        return -(-self.max_model_len // self.block_size)

    @property
    def pool_pages(self) -> int:
        return self.num_blocks if self.num_blocks is not None else self.max_num_seqs * self.pages_per_request

    def pages_for_memory(self, bytes_per_page: int, free_bytes: int) -> int:
        """Pages of the pool when it is sized by `memory_fraction`: what fits into that share of `free_bytes`, at
        most the worst case, at least the pages of one request of max_model_len (fewer could never finish one)."""
        worst = self.max_num_seqs * self.pages_per_request
        if self.memory_fraction is None or bytes_per_page <= 0:
            return worst
        fit = int(self.memory_fraction * free_bytes) // bytes_per_page
        if fit < self.pages_per_request:
            raise MemoryError(f"{self.memory_fraction:.2f} of the free device memory ({free_bytes >> 20} MiB) holds {fit} "
                              f"pages of {bytes_per_page} bytes; one request of max_model_len needs {self.pages_per_request}")
        return min(worst, fit)
