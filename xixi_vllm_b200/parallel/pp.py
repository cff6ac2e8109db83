"""Pipeline-stage bookkeeping (reference: src/distributed/utils.py:12-66)."""

from __future__ import annotations

__all__ = ["divide", "get_pp_indices", "set_pp_layer_ranges", "IntermediateTensors", "PPMissingLayer"]

_LAYER_COUNTS: list[int] | None = None


def divide(numerator: int, denominator: int) -> int:
    if denominator <= 0 or numerator % denominator:
        raise ValueError(f"{numerator} is not divisible by {denominator}")
    return numerator // denominator


def set_pp_layer_ranges(counts: list[int] | None) -> None:
    """Override the even split with explicit per-stage layer counts (None restores it)."""
    global _LAYER_COUNTS
    _LAYER_COUNTS = list(counts) if counts is not None else None


def get_pp_indices(num_layers: int, pp_rank: int, pp_size: int) -> tuple[int, int]:
    """Half-open layer range of a stage: even split, remainder on the last stage."""
    if _LAYER_COUNTS is not None:
        if len(_LAYER_COUNTS) != pp_size or sum(_LAYER_COUNTS) != num_layers:
            raise ValueError("pp layer counts do not match pp_size / num_layers")
        start = sum(_LAYER_COUNTS[:pp_rank])
        return start, start + _LAYER_COUNTS[pp_rank]
    per = num_layers // pp_size
    start = pp_rank * per
    end = num_layers if pp_rank == pp_size - 1 else start + per
    return start, end


class IntermediateTensors(dict):
    """Named tensors handed from one stage to the next (``hidden_states`` and ``residual``)."""


class PPMissingLayer:
    """Stand-in for a layer another stage owns: passes its first argument through."""

    def __call__(self, x=None, *args, **kwargs):
        return x

    forward = __call__
