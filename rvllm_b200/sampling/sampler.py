"""Sampling a batch of logits rows on the device.

Every row is sampled by the kernels (`argmax`, `sample`); only token ids come back to
the host.  (The reference takes the argmax on the device when every request of the
batch is greedy and otherwise copies all logits to the host, src/cuda/engine.rs:98-153.)
A request's k-th draw depends on (seed, k) only.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from .params import SamplingParams


class BatchSampler:
    def __init__(self, ops, device):
        self.ops = ops
        self.device = device

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               counters: Sequence[int]) -> List[int]:
        """One token id per row of `logits`; `counters[i]` is how many tokens row i's
        request has drawn before."""
        if logits.shape[0] == 0:
            return []
        return self.sample_device(logits, params, counters).tolist()

    def sample_device(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                      counters: Sequence[int]) -> torch.Tensor:
        """The same, leaving the ids on the device (int32 [rows]); nothing waits for the GPU."""
        if all(p.is_greedy for p in params):
            return self.ops.argmax(logits)
        dev = logits.device
        temperature = torch.tensor([p.temperature for p in params], dtype=torch.float32, device=dev)
        top_p = torch.tensor([p.top_p for p in params], dtype=torch.float32, device=dev)
        seed = torch.tensor([p.seed & 0x7FFFFFFFFFFFFFFF for p in params], dtype=torch.int64,
                            device=dev)
        counter = torch.tensor(list(counters), dtype=torch.int64, device=dev)
        return self.ops.sample(logits, temperature, top_p, seed, counter)
