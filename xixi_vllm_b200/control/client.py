"""Indirection between the facade and the engine core; the only place data parallelism
forks (reference: src/control/client.py:23-98)."""

from __future__ import annotations

from abc import ABC, abstractmethod

from ..config import EngineConfig
from ..data import EngineCoreOutput, Sequence
from .core import EngineCore

__all__ = ["EngineCoreClient", "InprocClient", "make_client"]


class EngineCoreClient(ABC):
    @abstractmethod
    def add_request(self, seq: Sequence) -> None: ...

    @abstractmethod
    def step(self) -> tuple[list[EngineCoreOutput], int]: ...

    @abstractmethod
    def has_unfinished(self) -> bool: ...

    @abstractmethod
    def destroy(self) -> None: ...


class InprocClient(EngineCoreClient):
    """dp=1: the core lives in this process and shares ``Sequence`` objects with the facade."""

    def __init__(self, engine_core: EngineCore) -> None:
        self.engine_core = engine_core

    def add_request(self, seq: Sequence) -> None:
        self.engine_core.add_request(seq)

    def step(self):
        return self.engine_core.step()

    def has_unfinished(self) -> bool:
        return self.engine_core.has_unfinished()

    def destroy(self) -> None:
        self.engine_core.destroy()


def make_client(config: EngineConfig, *, eos_token_id: int, device=None, dtype=None,
                executor=None) -> EngineCoreClient:
    if config.dp_size > 1:
        if executor is not None:
            raise ValueError("dp_size>1 uses replica processes; cannot inject a shared executor")
        from .mp_client import MPClient

        return MPClient(config, eos_token_id=eos_token_id, device=device, dtype=dtype)
    return InprocClient(EngineCore(config, eos_token_id=eos_token_id, device=device, dtype=dtype,
                                   executor=executor))
