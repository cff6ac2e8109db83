"""Compressed radix tree over chains of page hashes; each edge label element carries one
page id (reference: src/data/prefix/radix_tree.py:23-185).

Nodes are reference counted along the path to the root; only unreferenced leaves can be
evicted, coldest first. Recency is a logical clock (a counter bumped on every touch), so
eviction order is deterministic and testable.
"""

from __future__ import annotations

import heapq
import itertools

__all__ = ["RadixTree", "RadixNode"]


class RadixNode:
    __slots__ = ("children", "parent", "key", "value", "ref_count", "access_time")

    def __init__(self, parent=None, key=(), value=(), ref_count: int = 0, stamp: int = 0) -> None:
        self.children: dict[int, "RadixNode"] = {}
        self.parent = parent
        self.key: tuple[int, ...] = tuple(key)
        self.value: tuple[int, ...] = tuple(value)
        self.ref_count = ref_count
        self.access_time = stamp

    def __lt__(self, other: "RadixNode") -> bool:
        return self.access_time < other.access_time


def _common(a, b) -> int:
    n = min(len(a), len(b))
    i = 0
    while i < n and a[i] == b[i]:
        i += 1
    return i


class RadixTree:
    def __init__(self) -> None:
        self._clock = itertools.count(1)
        self.root = RadixNode(ref_count=1)
        self._owner: dict[int, RadixNode] = {}   # page id -> node holding it

    def contains_block(self, block_id: int) -> bool:
        return block_id in self._owner

    def num_nodes(self) -> int:
        n, stack = 0, [self.root]
        while stack:
            node = stack.pop()
            n += 1
            stack.extend(node.children.values())
        return n - 1

    # --- lookup / insert ------------------------------------------------------------
    def _descend(self, key, *, on_partial_split: bool):
        """Walk as far as ``key`` matches. Returns (values, node, matched_len, rest_key_offset)."""
        node, pos, values = self.root, 0, []
        while pos < len(key):
            child = node.children.get(key[pos])
            if child is None:
                break
            child.access_time = next(self._clock)
            m = _common(child.key, key[pos:])
            if m < len(child.key):
                if on_partial_split:
                    child = self._split(child, m)
                    values.extend(child.value)
                    return values, child, pos + m
                values.extend(child.value[:m])
                return values, node, pos + m
            values.extend(child.value)
            node, pos = child, pos + m
        return values, node, pos

    def match_prefix(self, key) -> tuple[list[int], RadixNode]:
        """Page ids along the longest stored prefix of ``key`` and the node that ends it.

        A match that stops inside an edge splits the edge so the returned node ends exactly
        at the match (callers pin that node).
        """
        values, node, _ = self._descend(list(key), on_partial_split=True)
        return values, node

    def insert(self, key, value) -> tuple[int, RadixNode]:
        """Store ``key -> value``. Returns (length already present, node that ends the key)."""
        key, value = list(key), list(value)
        if not key:
            return 0, self.root
        _, node, matched = self._descend(key, on_partial_split=True)
        if matched < len(key):
            node = self._attach(node, key[matched:], value[matched:])
        return matched, node

    # --- pins -------------------------------------------------------------------------
    def inc_ref(self, node: RadixNode) -> None:
        while node is not None and node is not self.root:
            node.ref_count += 1
            node = node.parent

    def dec_ref(self, node: RadixNode) -> None:
        while node is not None and node is not self.root:
            node.ref_count -= 1
            node = node.parent

    # --- eviction -----------------------------------------------------------------------
    def detach_leaf_for_block(self, block_id: int) -> list[int]:
        """The pool recycled ``block_id``: drop its node (and subtree entry) if nobody pins it."""
        node = self._owner.get(block_id)
        if node is None or node is self.root or node.ref_count > 0:
            return []
        freed = list(node.value)
        self._detach(node)
        return freed

    def evict(self, num_slots: int) -> list[int]:
        """Remove unpinned leaves, least recently touched first, until ``num_slots`` pages are freed."""
        heap = [n for n in self._iter_leaves()]
        heapq.heapify(heap)
        freed: list[int] = []
        while heap and len(freed) < num_slots:
            node = heapq.heappop(heap)
            if node is self.root or node.ref_count > 0:
                continue
            parent = node.parent
            freed.extend(node.value)
            self._detach(node)
            if parent is not None and parent is not self.root and not parent.children:
                heapq.heappush(heap, parent)
        return freed

    # --- internals ------------------------------------------------------------------------
    def _iter_leaves(self):
        stack = [self.root]
        while stack:
            node = stack.pop()
            if node.children:
                stack.extend(node.children.values())
            elif node is not self.root:
                yield node

    def _claim(self, node: RadixNode) -> None:
        for bid in node.value:
            self._owner[bid] = node

    def _disown(self, node: RadixNode) -> None:
        for bid in node.value:
            if self._owner.get(bid) is node:
                del self._owner[bid]

    def _attach(self, parent: RadixNode, key, value) -> RadixNode:
        node = RadixNode(parent, key, value, 0, next(self._clock))
        parent.children[node.key[0]] = node
        self._claim(node)
        return node

    def _detach(self, node: RadixNode) -> None:
        if node.parent is None or not node.key:
            return
        stack = [node]
        while stack:   # a pinned-free inner node takes its (necessarily unpinned) subtree along
            n = stack.pop()
            self._disown(n)
            stack.extend(n.children.values())
        node.parent.children.pop(node.key[0], None)

    def _split(self, node: RadixNode, at: int) -> RadixNode:
        """Cut ``node``'s edge after ``at`` elements; returns the new upper node."""
        self._disown(node)
        upper = RadixNode(node.parent, node.key[:at], node.value[:at], node.ref_count, node.access_time)
        node.parent.children[upper.key[0]] = upper
        node.key, node.value, node.parent = node.key[at:], node.value[at:], upper
        upper.children[node.key[0]] = node
        self._claim(upper)
        self._claim(node)
        return upper
