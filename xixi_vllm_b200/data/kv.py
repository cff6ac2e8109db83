"""Driver-side KV ledger the scheduler talks to (reference: src/data/kv.py:15-119).

Hands out page ids, finds reusable prefixes, publishes full pages after every step so a
prefix is shareable while its owner still runs, and recycles pages when sequences end.
"""

from __future__ import annotations

from .block_manager import BlockManager
from .prefix import RadixPrefixIndex, make_prefix_index
from .sequence import Sequence

__all__ = ["KVManager"]


class KVManager:
    def __init__(self, *, num_blocks: int, block_size: int, prefix_backend: str = "hash") -> None:
        if num_blocks <= 0:
            raise ValueError(f"num_blocks must be > 0, got {num_blocks}")
        self.block_size = block_size
        self.prefix_backend = prefix_backend
        self.num_blocks_total = num_blocks
        self.num_blocks_schedulable = num_blocks
        self.blocks = BlockManager(num_blocks, block_size)
        self.index = make_prefix_index(prefix_backend)
        self.blocks.on_evict = lambda bid: self.index.invalidate(bid, self.blocks)
        if isinstance(self.index, RadixPrefixIndex):
            self.blocks.reclaim_fn = lambda n: self.index.reclaim_pages(n, self.blocks)
        self.last_num_cached_tokens = 0
        # counters for observability
        self.num_prefix_queries = 0
        self.num_prefix_hit_tokens = 0
        self.num_prefix_query_tokens = 0

    @property
    def num_free(self) -> int:
        return self.blocks.num_free

    def usage(self) -> float:
        return self.blocks.num_used / self.num_blocks_total

    def _plan(self, seq: Sequence) -> tuple[int, list[int]]:
        """How many leading pages can be reused, or -1 if the request does not fit right now."""
        need = seq.num_blocks
        if need == 0:
            return 0, []
        hits = self.index.match(seq, self.blocks)[:need]
        # a fully cached prompt still has to compute its last token to get logits
        if hits and len(hits) * self.block_size >= seq.num_tokens:
            hits = hits[:-1]
        cached = self.blocks.cached_ids
        evictable = len(cached) - sum(1 for b in hits if b in cached)
        if self.blocks.num_free + evictable >= need - len(hits):
            return len(hits), hits
        return -1, hits

    def can_allocate(self, seq: Sequence) -> bool:
        return self._plan(seq)[0] >= 0

    def allocate(self, seq: Sequence) -> None:
        seq.bt_clear()
        seq.num_cached_tokens = 0
        need = seq.num_blocks
        if need == 0:
            self.last_num_cached_tokens = 0
            return
        n_hit, hits = self._plan(seq)
        if n_hit < 0:
            raise RuntimeError("not enough KV blocks for sequence")
        for bid in hits:
            self.blocks.acquire_hit(bid)
            seq.bt_append(bid)
        for _ in range(need - n_hit):
            seq.bt_append(self.blocks.allocate_fresh())
        seq.num_cached_tokens = n_hit * self.block_size
        self.last_num_cached_tokens = seq.num_cached_tokens
        self.num_prefix_queries += 1
        self.num_prefix_hit_tokens += seq.num_cached_tokens
        self.num_prefix_query_tokens += seq.num_tokens
        if n_hit > 0 and isinstance(self.index, RadixPrefixIndex):
            self.index.pin_match(seq, n_hit)

    def can_append(self, seq: Sequence) -> bool:
        return self.blocks.can_append(seq)

    def may_append(self, seq: Sequence) -> None:
        self.blocks.may_append(seq)

    def sync_prefix(self, seq: Sequence) -> None:
        """Publish pages that became full in the step that just ran."""
        if self.prefix_backend == "none" or seq.num_scheduled_tokens <= 0:
            return
        before = seq.num_cached_tokens - seq.num_scheduled_tokens
        first = before // self.block_size
        last = min(seq.num_full_blocks(), seq.num_cached_tokens // self.block_size)
        if first < last:
            self.index.publish(seq, last, self.blocks, start=first)

    def publish_range(self, seq: Sequence, before: int, after: int) -> None:
        """Publish the pages that a step filled which took the sequence's KV length from ``before`` to
        ``after`` (one-step-late scheduling: ``num_cached_tokens`` may already count the next step). A
        sequence that lost its pages since (preempted) publishes nothing."""
        if self.prefix_backend == "none" or after <= before or not seq.block_table:
            return
        first = before // self.block_size
        last = min(after // self.block_size, len(seq.block_table))
        if first < last:
            self.index.publish(seq, last, self.blocks, start=first)

    def deallocate(self, seq: Sequence, *, publish: bool = True) -> None:
        # Only pages whose KV was really written may be published: a preempted or
        # just-finished sequence has its newest token's KV still missing.
        n_keep = 0
        if publish and self.prefix_backend != "none":
            n_keep = min(seq.num_full_blocks(), seq.num_cached_tokens // self.block_size,
                         len(seq.block_table))
            if n_keep > 0:
                self.index.publish(seq, n_keep, self.blocks)
        self.index.release_seq(seq.seq_id)
        keep = set(seq.block_table[:n_keep])
        for bid in list(seq.block_table):
            kept = bid in keep
            if not kept and self.prefix_backend == "hash":
                self.index.invalidate(bid, self.blocks)
            self.blocks.release_to_cached_or_free(bid, keep_cached=kept)
            if not kept and self.prefix_backend == "radix" and bid not in self.blocks.used_ids:
                self.index.invalidate(bid, self.blocks)
        seq.bt_clear()
        seq.num_cached_tokens = 0
