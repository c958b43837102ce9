"""Greedy and temperature sampling on the device (csrc/sampling.cu).

The reference samples greedily only (argmax, jllm/engine/generate.py:142 and
jllm/engine/state.py:66).  Temperature sampling here is a draw from
softmax(logits / temperature) whose random numbers are keyed by (seed of the request,
index of the output token, vocabulary index), so a request's tokens do not depend on the
batch it is sampled in.
"""

from __future__ import annotations

import torch

from .. import ops

_MASK64 = (1 << 64) - 1


def mix64(z: int) -> int:
    z &= _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    return z ^ (z >> 31)


def uniform(seed: int, counter: int, v: int) -> float:
    """The uniform number in (0, 1) that the kernel uses for vocabulary index v (a host
    restatement, for tests and for reasoning about reproducibility)."""
    h = mix64((seed + 0x9E3779B97F4A7C15 * (counter + 1)) & _MASK64)
    h = mix64(h ^ ((v * 0xD1342543DE82EF95 + 0x2545F4914F6CDD1D) & _MASK64))
    return ((h >> 40) + 0.5) / 16777216.0


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        self._zeros: dict = {}            # rows -> (temperatures, seeds and counters) of greedy sampling, made once

    def sample(self, logits: torch.Tensor, temperatures, seeds, counters) -> torch.Tensor:
        """One token (int32, on the device) per row of float32 logits."""
        rows = logits.shape[0]
        if not (len(temperatures) == len(seeds) == len(counters) == rows):
            raise ValueError("one temperature, seed and counter per row of logits")
        t = torch.tensor(list(temperatures), dtype=torch.float32).to(self.device, non_blocking=True)
        sc = torch.tensor([[s & ((1 << 63) - 1) for s in seeds], list(counters)], dtype=torch.int64)
        sc = sc.to(self.device, non_blocking=True)
        return ops.sample(logits, t, sc[0].contiguous(), sc[1].contiguous())

    def greedy(self, logits: torch.Tensor) -> torch.Tensor:
        rows = logits.shape[0]
        zeros = self._zeros.get(rows)
        if zeros is None:
            zeros = self._zeros[rows] = (torch.zeros(rows, dtype=torch.float32, device=self.device),
                                         torch.zeros(rows, dtype=torch.int64, device=self.device))
        return ops.sample(logits, zeros[0], zeros[1], zeros[1])
