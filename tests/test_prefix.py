"""Chain hashing and the radix tree (CPU only)."""
import struct

import numpy as np
import pytest

from xixi_vllm_b200.data.prefix.chain_hash import _digest_py, chain_hashes, compute_block_hash
from xixi_vllm_b200.data.prefix.radix_tree import RadixTree
from xixi_vllm_b200.ops import hostlib


def test_native_chain_equals_python_chain():
    rng = np.random.default_rng(0)
    toks = rng.integers(0, 151936, size=16 * 20 + 3).tolist()
    got = chain_hashes(toks, 16, 20)
    h, want = -1, []
    for i in range(20):
        h = _digest_py(toks[i * 16:(i + 1) * 16], h)
        want.append(h)
    assert got == want
    assert chain_hashes(toks, 16, 5, parent=want[9], start_block=10) == want[10:15]
    assert compute_block_hash(toks[:16]) == want[0]


def test_native_xxh64_matches_wheel():
    xxhash = pytest.importorskip("xxhash")
    lib = hostlib.get()
    if lib is None:
        pytest.skip("host library not built")
    rng = np.random.default_rng(1)
    for n in (0, 1, 3, 4, 7, 8, 15, 31, 32, 33, 63, 64, 100, 1000):
        d = bytes(rng.integers(0, 256, size=n, dtype=np.uint8))
        assert lib.xv_xxh64(d, n) == xxhash.xxh64_intdigest(d)


def test_chain_is_order_and_parent_sensitive():
    a = chain_hashes(list(range(32)), 16, 2)
    b = chain_hashes(list(range(16, 32)) + list(range(16)), 16, 2)
    assert a[0] != b[0] and a[1] != b[1]
    assert compute_block_hash(list(range(16)), prefix=a[0]) != compute_block_hash(list(range(16)))
    assert struct.pack("<Q", a[0])      # fits in 64 bits


def test_radix_insert_match_split_and_evict():
    t = RadixTree()
    assert t.insert([1, 2, 3, 4], [10, 11, 12, 13])[0] == 0
    matched, leaf2 = t.insert([1, 2, 7, 8], [10, 11, 20, 21])      # shares [1,2], splits the edge
    assert matched == 2
    ids, node = t.match_prefix([1, 2, 3, 4, 5])
    assert ids == [10, 11, 12, 13]
    ids, _ = t.match_prefix([1, 2, 7])
    assert ids == [10, 11, 20]
    assert t.match_prefix([9])[0] == []
    assert t.contains_block(12) and t.contains_block(21)
    t.inc_ref(leaf2)                                               # pin the [1,2,7,8] path
    freed = t.evict(10)
    assert sorted(freed) == [12, 13]                               # only the unpinned leaf goes
    t.dec_ref(leaf2)
    assert sorted(t.evict(10)) == [10, 11, 20, 21]                 # leaf, then its now-childless parent
    assert t.num_nodes() == 0


def test_radix_evicts_coldest_leaf_first():
    t = RadixTree()
    t.insert([1], [1])
    t.insert([2], [2])
    t.insert([3], [3])
    t.match_prefix([1])                 # touch 1: order of coldness is now 2, 3, 1
    assert t.evict(1) == [2]
    assert t.evict(1) == [3]
    assert t.evict(1) == [1]


def test_radix_detach_respects_pins():
    t = RadixTree()
    _, leaf = t.insert([5, 6], [50, 60])
    t.inc_ref(leaf)
    assert t.detach_leaf_for_block(50) == []
    t.dec_ref(leaf)
    assert sorted(t.detach_leaf_for_block(50)) == [50, 60]
    assert not t.contains_block(60)
