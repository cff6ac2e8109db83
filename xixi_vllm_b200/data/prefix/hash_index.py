"""Prefix index as a flat map ``chain hash -> page id`` (reference: src/data/prefix/hash_index.py:19-70).

A hit is accepted only if the page still stores the same token ids (guards against hash
collisions) and is still live (used or cached).
"""

from __future__ import annotations

from .chain_hash import NO_PARENT, chain_hashes


class HashPrefixIndex:
    def __init__(self) -> None:
        self.hash_to_block_id: dict[int, int] = {}

    def match(self, seq, pool) -> list[int]:
        n = seq.num_full_blocks()
        if n == 0 or not self.hash_to_block_id:
            return []
        bs = seq.block_size
        hits: list[int] = []
        for i, h in enumerate(chain_hashes(seq.token_ids, bs, n)):
            bid = self.hash_to_block_id.get(h)
            if bid is None:
                break
            if pool._tokens[bid] != seq.token_ids[i * bs:(i + 1) * bs]:
                break
            if bid not in pool.used_ids and bid not in pool.cached_ids:
                break
            hits.append(bid)
        return hits

    def publish(self, seq, num_full_blocks: int, pool, *, start: int = 0) -> None:
        """Record pages ``start..num_full_blocks-1``; chain from page ``start-1``'s stored hash."""
        if num_full_blocks <= start:
            return
        parent = NO_PARENT
        if start > 0:
            parent = pool._hash[seq.block_table[start - 1]]
            if parent == NO_PARENT:   # predecessor was never hashed: rebuild the chain
                start = 0
        bs = seq.block_size
        hashes = chain_hashes(seq.token_ids, bs, num_full_blocks - start, parent, start)
        for i, h in zip(range(start, num_full_blocks), hashes):
            bid = seq.block_table[i]
            toks = seq.token_ids[i * bs:(i + 1) * bs]
            pool.blocks[bid].update(h, toks)
            old = self.hash_to_block_id.get(h)
            if old is None or old == bid or pool._tokens[old] == toks:
                self.hash_to_block_id[h] = bid

    def invalidate(self, block_id: int, pool) -> None:
        h = pool._hash[block_id]
        if h != NO_PARENT and self.hash_to_block_id.get(h) == block_id:
            del self.hash_to_block_id[h]

    def release_seq(self, seq_id: int) -> None:
        return None
