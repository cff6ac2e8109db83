"""Token sampling (reference: src/compute/sampler.py:6-119).

Greedy rows take the argmax; other rows apply temperature, top-k, top-p and min-p and draw
one token. On the GPU this is one kernel family over the logits with a counter-based
random stream keyed by (seed, step, row), so every tensor-parallel rank draws the same
token without communicating and nothing synchronises with the host.
"""

from __future__ import annotations

import torch

from ..ops import dispatch as ops

__all__ = ["Sampler"]


class Sampler:
    def __init__(self, seed: int = 0) -> None:
        self.seed = seed
        self.step = 0
        self._gen: torch.Generator | None = None

    def to(self, device=None):
        return self

    def forward(self, logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
                top_p: torch.Tensor, min_p: torch.Tensor, *, all_greedy: bool = False,
                rng: torch.Tensor | None = None) -> torch.Tensor:
        """``rng`` is the device-resident ``[seed, step]`` pair staged with the batch; kernels read
        it from memory so a captured graph draws fresh numbers on every replay."""
        self.step += 1
        if all_greedy:
            return ops.argmax(logits)
        if not logits.is_cuda and self._gen is None:
            self._gen = torch.Generator().manual_seed(self.seed)
        return ops.sample(logits, temperature, top_k, top_p, min_p, rng=rng, generator=self._gen)

    __call__ = forward
