"""Prefix index backed by a radix tree of page-hash chains (reference:
src/data/prefix/radix_index.py:20-129).

Compared with the flat hash map it de-duplicates a sequence's pages onto pages already in
the tree when it publishes, pins the deepest node a live sequence depends on, and frees
whole cold leaves when the pool runs dry.
"""

from __future__ import annotations

from .chain_hash import NO_PARENT, chain_hashes
from .radix_tree import RadixTree


class RadixPrefixIndex:
    def __init__(self) -> None:
        self.tree = RadixTree()
        self._pin: dict[int, object] = {}    # seq_id -> pinned node

    def _repin(self, seq_id: int, node) -> None:
        old = self._pin.pop(seq_id, None)
        if old is not None:
            self.tree.dec_ref(old)
        self.tree.inc_ref(node)
        self._pin[seq_id] = node

    def match(self, seq, pool) -> list[int]:
        n = seq.num_full_blocks()
        if n <= 0:
            return []
        bs = seq.block_size
        key = chain_hashes(seq.token_ids, bs, n)
        ids, _ = self.tree.match_prefix(key)
        hits: list[int] = []
        for i, bid in enumerate(ids[:n]):
            if bid < 0 or pool._hash[bid] != key[i]:
                break
            if pool._tokens[bid] != seq.token_ids[i * bs:(i + 1) * bs]:
                break
            if bid not in pool.used_ids and bid not in pool.cached_ids:
                break
            hits.append(bid)
        return hits

    def publish(self, seq, num_full_blocks: int, pool, *, start: int = 0) -> None:
        if num_full_blocks <= start:
            return
        parent = NO_PARENT
        if start > 0:
            parent = pool._hash[seq.block_table[start - 1]]
            if parent == NO_PARENT:
                start = 0
        bs = seq.block_size
        for i, h in zip(range(start, num_full_blocks),
                        chain_hashes(seq.token_ids, bs, num_full_blocks - start, parent, start)):
            pool.blocks[seq.block_table[i]].update(h, seq.token_ids[i * bs:(i + 1) * bs])

        key = [pool._hash[seq.block_table[i]] for i in range(num_full_blocks)]
        already, leaf = self.tree.insert(key, seq.block_table[:num_full_blocks])
        if already > 0:
            # Pages of the shared prefix exist in the tree under other ids: move this
            # sequence onto them and give its own copies back.
            tree_ids, _ = self.tree.match_prefix(key)
            for i in range(min(already, len(tree_ids), num_full_blocks)):
                mine, theirs = seq.block_table[i], tree_ids[i]
                if mine != theirs:
                    pool.release_hit(mine)
                    pool.acquire_hit(theirs)
                    seq.bt_replace(i, theirs)
        self._repin(seq.seq_id, leaf)

    def invalidate(self, block_id: int, pool) -> None:
        self.tree.detach_leaf_for_block(block_id)

    def release_seq(self, seq_id: int) -> None:
        node = self._pin.pop(seq_id, None)
        if node is not None:
            self.tree.dec_ref(node)

    def pin_match(self, seq, num_cached: int) -> None:
        """After a prefix hit, pin the node covering the reused pages so they cannot be evicted."""
        if num_cached <= 0:
            return
        key = chain_hashes(seq.token_ids, seq.block_size, num_cached)
        _, node = self.tree.match_prefix(key)
        self._repin(seq.seq_id, node)

    def reclaim_pages(self, num_pages: int, pool) -> list[int]:
        """Drop cold unpinned leaves; returns the freed pages that sit in the pool's cached set."""
        out: list[int] = []
        for _ in range(64):
            if len(out) >= num_pages:
                break
            freed = self.tree.evict(max(1, num_pages - len(out)))
            if not freed:
                break
            out.extend(b for b in freed if b in pool.cached_ids)
        return out
