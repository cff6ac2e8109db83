"""Prefix-cache indexes selected by ``EngineConfig.prefix_backend``."""

from __future__ import annotations

from typing import Literal

from .hash_index import HashPrefixIndex
from .noop import NoopPrefixIndex
from .radix_index import RadixPrefixIndex

PrefixBackend = Literal["none", "hash", "radix"]

__all__ = ["PrefixBackend", "make_prefix_index", "HashPrefixIndex", "NoopPrefixIndex", "RadixPrefixIndex"]


def make_prefix_index(backend: str):
    if backend == "hash":
        return HashPrefixIndex()
    if backend == "radix":
        return RadixPrefixIndex()
    if backend == "none":
        return NoopPrefixIndex()
    raise ValueError(f"unknown prefix backend {backend!r}")
