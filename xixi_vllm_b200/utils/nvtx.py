"""NVTX ranges around engine phases, enabled with ``XV_NVTX=1`` (off by default: zero cost).

The reference has no tracing hooks; these ranges make step phases (stage, forward, sample,
readback) visible in Nsight Systems timelines.
"""

from __future__ import annotations

import os
from contextlib import contextmanager

_ENABLED = os.environ.get("XV_NVTX", "0") == "1"

__all__ = ["nvtx_range", "enabled"]


def enabled() -> bool:
    return _ENABLED


@contextmanager
def _noop(_name: str):
    yield


@contextmanager
def _range(name: str):
    import torch

    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


nvtx_range = _range if _ENABLED else _noop
