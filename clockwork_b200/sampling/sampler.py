"""Turns logits rows into tokens: greedy (first maximal index) or temperature / top-k / top-p
sampling, on the GPU.

Reference: ``clockwork/engine/model_runner.py:134-164``.  The reference draws with
``torch.multinomial`` from a per-request CPU generator seeded once and kept across steps and
preemptions (``:139-145``).  Here each draw uses a uniform number that is a pure function of
(the request's seed, how many tokens the request has generated so far), so a request's draws
do not depend on batching, on preemption, or on what else runs; the token is the first index
whose cumulative probability exceeds that number.
"""

from __future__ import annotations

import torch

from .. import ops
from .params import SamplingParams

_MASK = (1 << 64) - 1


def uniform_for(seed: int, draw_index: int) -> float:
    """A number in [0, 1) with 24 random bits (exact in float32), from a splitmix64 mix."""
    z = (seed * 0x9E3779B97F4A7C15 + (draw_index + 1) * 0xD1B54A32D192ED03) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, device, default_seed: int = 0) -> None:
        self.device = torch.device(device)
        self.default_seed = default_seed

    def sample(self, logits: torch.Tensor, params: list[SamplingParams], draw_indices: list[int]) -> list[int]:
        """One token per row of ``logits`` (float32 [R, vocab], on the device)."""
        return self.sample_device(logits, params, draw_indices).tolist()

    def state_rows(self, params: list[SamplingParams], draw_indices: list[int]) -> list[tuple] | None:
        """Per request (temperature, top_k, top_p, seed, draws): what a request's column of the device
        state table holds about sampling (the kernels derive the draw's uniform number from seed and
        draws exactly as ``uniform_for`` does).  None when every request is greedy."""
        if all(p.greedy for p in params):
            return None
        return [(p.temperature, p.top_k if p.top_k and p.top_k > 0 else 0, p.top_p,
                 p.seed if p.seed is not None else self.default_seed, k) for p, k in zip(params, draw_indices)]

    def sample_device(self, logits: torch.Tensor, params: list[SamplingParams], draw_indices: list[int]) -> torch.Tensor:
        if logits.shape[0] != len(params):
            raise ValueError("one SamplingParams per logits row is needed")
        if all(p.greedy for p in params):
            return ops.argmax(logits)
        host = torch.empty((4, len(params)), dtype=torch.float32)
        for i, (p, k) in enumerate(zip(params, draw_indices)):
            seed = p.seed if p.seed is not None else self.default_seed
            host[0, i] = p.temperature
            host[1, i] = float(p.top_k if p.top_k and p.top_k > 0 else 0)
            host[2, i] = p.top_p
            host[3, i] = uniform_for(seed, k)
        dev = host.to(self.device)
        return ops.sample(logits, dev[0].contiguous(), dev[1].to(torch.int32), dev[2].contiguous(), dev[3].contiguous())
