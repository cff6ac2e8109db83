"""CUDA-graph capture and replay of the decode forward (reference: src/compute/cuda_graph.py:11-52).

One graph per (batch-size bucket, variant), captured largest first into a shared memory
pool; a step with ``bs`` sequences replays the smallest bucket >= bs with inert padding
rows. Kernels in a graph read all per-step metadata from fixed device buffers, so replay
needs one H2D copy and one launch.
"""

from __future__ import annotations

import torch

from ..parallel.groups import graph_capture

__all__ = ["CUDAGraphRunner", "make_bs_list"]


def _launches() -> int:
    from ..ops import cuda

    return cuda.launch_count


def make_bs_list(max_bs: int) -> list[int]:
    """1, 2, 4, 8, then multiples of 16 up to 128, multiples of 32 beyond."""
    out = [b for b in (1, 2, 4, 8) if b <= max_bs]
    b = 16
    while b <= max_bs:
        out.append(b)
        b += 16 if b < 128 else 32
    if not out or out[-1] != max_bs:
        out.append(max_bs)
    return sorted(set(out))


class CUDAGraphRunner:
    def __init__(self, bs_list: list[int]) -> None:
        self.bs_list = sorted(bs_list)
        self.graphs: dict[tuple, torch.cuda.CUDAGraph] = {}
        self.outputs: dict[tuple, object] = {}
        self.kernels: dict[tuple, int] = {}      # kernel launches recorded in each graph
        self.replayed_kernels = 0                # kernels executed through replays so far
        self.pool = None

    @property
    def max_bs(self) -> int:
        return self.bs_list[-1]

    def pad_bs(self, bs: int) -> int:
        for b in self.bs_list:
            if b >= bs:
                return b
        raise ValueError(f"batch {bs} exceeds the largest captured bucket {self.max_bs}")

    def capture(self, variants, make_inputs, body, warmup: int = 2) -> None:
        """For every bucket (largest first) and every variant: ``make_inputs(bs, variant)`` stages
        an inert batch, ``body(batch)`` launches the forward and returns its output tensor, which
        stays alive as the graph's static output."""
        with graph_capture():
            for bs in reversed(self.bs_list):
                for variant in variants:
                    batch = make_inputs(bs, variant)
                    for _ in range(warmup):
                        body(batch)
                    torch.cuda.synchronize()
                    g = torch.cuda.CUDAGraph()
                    n0 = _launches()
                    with torch.cuda.graph(g, pool=self.pool):
                        out = body(batch)
                    self.kernels[(bs, variant)] = _launches() - n0
                    if self.pool is None:
                        self.pool = g.pool()
                    self.graphs[(bs, variant)] = g
                    self.outputs[(bs, variant)] = out
        torch.cuda.synchronize()

    def replay(self, bs: int, variant):
        key = (bs, variant)
        self.graphs[key].replay()
        self.replayed_kernels += self.kernels[key]
        return self.outputs[key]

    def destroy(self) -> None:
        self.graphs.clear()
        self.outputs.clear()
        self.pool = None
