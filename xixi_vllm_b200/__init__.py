"""B200-native Qwen3 inference engine.

Public surface: ``from xixi_vllm_b200 import Engine, EngineConfig, SamplingParams``.
Attributes resolve lazily so importing the package does not pull in torch, the
tokenizer stack or the CUDA extension (reference: src/__init__.py:8-28).
"""

from __future__ import annotations

import importlib
from typing import TYPE_CHECKING, Any

__version__ = "0.1.0"
__all__ = ["Engine", "EngineConfig", "SamplingParams"]

if TYPE_CHECKING:  # pragma: no cover
    from .config import EngineConfig
    from .control.engine import Engine
    from .sampling_params import SamplingParams

_EXPORTS = {
    "Engine": "xixi_vllm_b200.control.engine",
    "EngineConfig": "xixi_vllm_b200.config",
    "SamplingParams": "xixi_vllm_b200.sampling_params",
}


def __getattr__(name: str) -> Any:
    target = _EXPORTS.get(name)
    if target is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    value = getattr(importlib.import_module(target), name)
    globals()[name] = value
    return value
