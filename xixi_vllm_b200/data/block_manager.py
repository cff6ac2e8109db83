"""Ledger of KV page ids: free, used (ref-counted) and cached-for-prefix-reuse
(reference: src/data/block_manager.py:15-151).

Page ids index the GPU pool tensor one to one. State is kept in flat per-page arrays
rather than per-page objects; the cached set is an insertion-ordered dict used as an LRU
(oldest first).
"""

from __future__ import annotations

from collections import OrderedDict, deque
from typing import Callable

__all__ = ["BlockManager", "NO_HASH"]

NO_HASH = -1


class _BlockView:
    """Read/write view of one page's metadata (``pool.blocks[i].hash`` style access)."""

    __slots__ = ("_p", "_i")

    def __init__(self, pool: "BlockManager", i: int) -> None:
        self._p, self._i = pool, i

    @property
    def ref_count(self) -> int:
        return self._p._ref[self._i]

    @ref_count.setter
    def ref_count(self, v: int) -> None:
        self._p._ref[self._i] = v

    @property
    def hash(self) -> int:
        return self._p._hash[self._i]

    @property
    def token_ids(self) -> list[int]:
        return self._p._tokens[self._i]

    def update(self, h: int, token_ids) -> None:
        self._p._hash[self._i] = h
        self._p._tokens[self._i] = list(token_ids)


class _Blocks:
    def __init__(self, pool: "BlockManager") -> None:
        self._p = pool

    def __getitem__(self, i: int) -> _BlockView:
        return _BlockView(self._p, i)

    def __len__(self) -> int:
        return self._p.num_blocks


class BlockManager:
    def __init__(self, num_blocks: int, block_size: int) -> None:
        if num_blocks <= 0:
            raise ValueError(f"num_blocks must be positive, got {num_blocks}")
        if block_size <= 0:
            raise ValueError(f"block_size must be positive, got {block_size}")
        self.num_blocks = num_blocks
        self.block_size = block_size
        self._ref = [0] * num_blocks
        self._hash = [NO_HASH] * num_blocks
        self._tokens: list[list[int]] = [[] for _ in range(num_blocks)]
        self.blocks = _Blocks(self)
        self.free_ids: deque[int] = deque(range(num_blocks))
        self.used_ids: set[int] = set()
        self.cached_ids: "OrderedDict[int, None]" = OrderedDict()
        # called with a page id just before a cached page is recycled
        self.on_evict: Callable[[int], None] | None = None
        # radix backend: asks the tree for cold leaves; returned pages are already unindexed
        self.reclaim_fn: Callable[[int], list[int]] | None = None
        self.num_evictions = 0

    # --- counts -----------------------------------------------------------------
    @property
    def num_free(self) -> int:
        return len(self.free_ids)

    @property
    def num_cached(self) -> int:
        return len(self.cached_ids)

    @property
    def num_used(self) -> int:
        return len(self.used_ids)

    @property
    def available_slots(self) -> int:
        return len(self.free_ids) + len(self.cached_ids)

    def check_invariants(self) -> None:
        """Every page is in exactly one of free / used / cached; used pages have refs."""
        free, cached = set(self.free_ids), set(self.cached_ids)
        assert len(free) == len(self.free_ids), "duplicate id in free list"
        assert not (free & self.used_ids) and not (free & cached) and not (cached & self.used_ids)
        assert len(free) + len(self.used_ids) + len(cached) == self.num_blocks
        for b in self.used_ids:
            assert self._ref[b] >= 1, f"used page {b} has ref {self._ref[b]}"
        for b in free | cached:
            assert self._ref[b] == 0, f"idle page {b} has ref {self._ref[b]}"

    # --- allocation ---------------------------------------------------------------
    def _clear_meta(self, bid: int) -> None:
        self._hash[bid] = NO_HASH
        self._tokens[bid] = []

    def _recycle_cached(self, bid: int, *, notify: bool) -> None:
        if bid not in self.cached_ids:
            return
        if notify and self.on_evict is not None:
            self.on_evict(bid)
        del self.cached_ids[bid]
        self._ref[bid] = 0
        self._clear_meta(bid)
        self.free_ids.append(bid)
        self.num_evictions += 1

    def _make_room(self) -> None:
        if self.free_ids:
            return
        if self.reclaim_fn is not None and self.cached_ids:
            for bid in self.reclaim_fn(1):
                self._recycle_cached(bid, notify=False)
            if self.free_ids:
                return
        if not self.cached_ids:
            raise RuntimeError("KV block pool exhausted")
        self._recycle_cached(next(iter(self.cached_ids)), notify=True)

    def allocate_fresh(self) -> int:
        self._make_room()
        bid = self.free_ids.popleft()
        self._ref[bid] = 1
        self._clear_meta(bid)
        self.used_ids.add(bid)
        return bid

    def acquire_hit(self, bid: int) -> None:
        """Take a reference on a page found by the prefix index, whatever set it is in."""
        if bid in self.used_ids:
            self._ref[bid] += 1
            return
        if bid in self.cached_ids:
            del self.cached_ids[bid]
        else:
            self.free_ids.remove(bid)
        self._ref[bid] = 1
        self.used_ids.add(bid)

    def release_hit(self, bid: int) -> None:
        """Drop a reference; at zero the page goes straight back to the free list."""
        self._ref[bid] -= 1
        if self._ref[bid] == 0:
            self.used_ids.discard(bid)
            self.cached_ids.pop(bid, None)
            self._clear_meta(bid)
            self.free_ids.append(bid)

    def touch_cached(self, bid: int) -> None:
        if bid in self.cached_ids:
            self.cached_ids.move_to_end(bid)

    def release_to_cached_or_free(self, bid: int, *, keep_cached: bool) -> None:
        """Drop a reference; at zero keep hashed pages in the LRU when asked, else free them."""
        self._ref[bid] -= 1
        if self._ref[bid] > 0:
            return
        self.used_ids.discard(bid)
        if keep_cached and self._hash[bid] != NO_HASH:
            self.cached_ids[bid] = None
            self.cached_ids.move_to_end(bid)
        else:
            self.cached_ids.pop(bid, None)
            self._clear_meta(bid)
            self.free_ids.append(bid)

    # --- decode growth --------------------------------------------------------------
    def _needs_new_page(self, seq) -> bool:
        # The token about to be written is the last of ``seq``; it opens a page when the
        # length is one past a page boundary.
        return len(seq) % self.block_size == 1 or (self.block_size == 1)

    def can_append(self, seq) -> bool:
        return (not self._needs_new_page(seq)) or self.available_slots >= 1

    def may_append(self, seq) -> None:
        if self._needs_new_page(seq) and len(seq.block_table) < seq.num_blocks:
            seq.bt_append(self.allocate_fresh())
