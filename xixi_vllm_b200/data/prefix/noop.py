"""``prefix_backend="none"``: never matches, never records (reference: src/data/prefix/noop.py)."""

from __future__ import annotations


class NoopPrefixIndex:
    def match(self, seq, pool) -> list[int]:
        return []

    def publish(self, seq, num_full_blocks: int, pool, *, start: int = 0) -> None:
        return None

    def invalidate(self, block_id: int, pool) -> None:
        return None

    def release_seq(self, seq_id: int) -> None:
        return None
