"""Sequence, wire messages, block ledger, KV manager (CPU only)."""
import random

import pytest

from xixi_vllm_b200.data import BlockManager, KVManager, ScheduledBatch, Sequence, slots_for_range
from xixi_vllm_b200.sampling_params import SamplingParams


def seq_of(n, bs=16, start=0, **kw):
    return Sequence.from_prompt(list(range(start, start + n)), block_size=bs, sampling=SamplingParams(**kw))


def test_slots_for_range_matches_naive_loop():
    rnd = random.Random(0)
    for bs in (16, 32, 256):
        table = [rnd.randrange(1000) for _ in range(40)]
        for _ in range(50):
            a = rnd.randrange(0, 30 * bs)
            b = a + rnd.randrange(0, 5 * bs)
            want = [table[p // bs] * bs + p % bs for p in range(a, b)]
            assert slots_for_range(table, a, b, bs) == want


def test_sequence_sizes():
    s = seq_of(33)
    assert (s.num_tokens, s.num_blocks, s.num_full_blocks(), s.last_block_num_tokens) == (33, 3, 2, 1)
    assert s.block_token_ids(2) == [32]
    s.append_token(7)
    assert s.last_token == 7 and s.num_completion_tokens == 1
    with pytest.raises(ValueError):
        Sequence.from_prompt([], block_size=16)


def test_sampling_params_validation():
    for bad in (dict(max_tokens=-1), dict(temperature=-0.1), dict(top_p=0.0), dict(top_p=1.5), dict(top_k=0),
                dict(min_p=1.5)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
    SamplingParams(top_p=1.0, top_k=-1, min_p=0.0)


def test_wire_sends_block_table_tail_only():
    s = seq_of(40)
    s.block_table = [5, 6, 7]
    s.num_scheduled_tokens = 40
    w = ScheduledBatch(prefills=[s]).to_wire()
    assert (w.prefills[0].bt_from, w.prefills[0].bt_tail) == (0, [5, 6, 7])
    s.num_cached_tokens = 40
    s.append_token(1)
    d = ScheduledBatch(decodes=[s]).to_wire().decodes          # nothing new: no table traffic at all
    assert (d.seq_ids, d.tokens, d.cached, d.bt_index, d.bt_vals) == ([s.seq_id], [1], [40], [], [])
    s.bt_append(9)
    s.bt_replace(1, 11)           # an edit below the synced mark resends from there
    d = ScheduledBatch(decodes=[s]).to_wire().decodes
    assert (d.bt_index, d.bt_from, d.bt_count, d.bt_vals) == ([0], [1], [3], [11, 7, 9])


def test_block_manager_invariants_random_walk():
    rnd = random.Random(1)
    bm = BlockManager(32, 16)
    held = []
    for _ in range(2000):
        op = rnd.random()
        if op < 0.45 and bm.available_slots:
            held.append(bm.allocate_fresh())
        elif op < 0.6 and held:
            b = rnd.choice(held)
            bm.acquire_hit(b)
            held.append(b)
        elif held:
            b = held.pop(rnd.randrange(len(held)))
            keep = rnd.random() < 0.5
            if keep:
                bm.blocks[b].update(rnd.getrandbits(60), [1])
            bm.release_to_cached_or_free(b, keep_cached=keep)
        bm.check_invariants()
    assert bm.num_free + bm.num_used + bm.num_cached == 32


def test_block_manager_lru_eviction_order_and_exhaustion():
    bm = BlockManager(3, 16)
    evicted = []
    bm.on_evict = evicted.append
    ids = [bm.allocate_fresh() for _ in range(3)]
    for i, b in enumerate(ids):
        bm.blocks[b].update(100 + i, [i])
        bm.release_to_cached_or_free(b, keep_cached=True)
    bm.touch_cached(ids[0])                      # ids[1] is now the coldest
    assert bm.allocate_fresh() == ids[1] and evicted == [ids[1]]
    bm.allocate_fresh(); bm.allocate_fresh()
    with pytest.raises(RuntimeError, match="exhausted"):
        bm.allocate_fresh()


def test_may_append_opens_page_at_boundary():
    kv = KVManager(num_blocks=8, block_size=16, prefix_backend="none")
    s = seq_of(16)
    kv.allocate(s)
    assert len(s.block_table) == 1
    s.append_token(0)                            # 17 tokens: the new token opens page 2
    assert kv.can_append(s)
    kv.may_append(s)
    assert len(s.block_table) == 2
    for _ in range(15):
        s.append_token(0)
        kv.may_append(s)
    assert len(s.block_table) == 2


@pytest.mark.parametrize("backend", ["hash", "radix"])
def test_prefix_reuse_and_last_page_rule(backend):
    kv = KVManager(num_blocks=32, block_size=16, prefix_backend=backend)
    a = seq_of(64)
    kv.allocate(a)
    a.num_scheduled_tokens = 64
    a.num_cached_tokens = 64
    kv.sync_prefix(a)                            # four full pages become shareable while a still runs
    b = Sequence.from_prompt(list(range(48)) + [999] * 10, block_size=16)
    kv.allocate(b)
    assert b.num_cached_tokens == 48 and b.block_table[:3] == a.block_table[:3]
    c = seq_of(64)                               # identical prompt: the last page is recomputed for logits
    kv.allocate(c)
    assert c.num_cached_tokens == 48
    for s in (a, b, c):
        kv.deallocate(s)
    kv.blocks.check_invariants()
    assert kv.blocks.num_used == 0


@pytest.mark.parametrize("backend", ["none", "hash", "radix"])
def test_kv_manager_random_workload_keeps_ledger_consistent(backend):
    rnd = random.Random(2)
    kv = KVManager(num_blocks=48, block_size=16, prefix_backend=backend)
    prefixes = [[rnd.randrange(500) for _ in range(32)] for _ in range(3)]
    live = []
    for _ in range(300):
        if live and (rnd.random() < 0.45 or len(live) > 6):
            s = live.pop(rnd.randrange(len(live)))
            kv.deallocate(s, publish=rnd.random() < 0.8)
        else:
            toks = rnd.choice(prefixes) + [rnd.randrange(500) for _ in range(rnd.randrange(1, 40))]
            s = Sequence.from_prompt(toks, block_size=16)
            if kv.can_allocate(s):
                kv.allocate(s)
                assert len(s.block_table) == s.num_blocks
                s.num_scheduled_tokens = s.num_tokens - s.num_cached_tokens
                s.num_cached_tokens = s.num_tokens
                kv.sync_prefix(s)
                live.append(s)
        kv.blocks.check_invariants()
        refs = {}
        for s in live:
            for b in s.block_table:
                refs[b] = refs.get(b, 0) + 1
        for b, n in refs.items():
            assert kv.blocks.blocks[b].ref_count == n
    if backend != "none":
        assert kv.num_prefix_hit_tokens > 0


def test_hash_and_radix_agree_on_hits():
    rnd = random.Random(3)
    kvs = {b: KVManager(num_blocks=256, block_size=16, prefix_backend=b) for b in ("hash", "radix")}
    base = [rnd.randrange(100) for _ in range(96)]
    for _ in range(40):
        cut = rnd.randrange(0, 96)
        toks = base[:cut] + [rnd.randrange(100, 200) for _ in range(rnd.randrange(1, 50))]
        hits = {}
        for name, kv in kvs.items():
            s = Sequence.from_prompt(toks, block_size=16)
            kv.allocate(s)
            hits[name] = s.num_cached_tokens
            s.num_scheduled_tokens = s.num_tokens - s.num_cached_tokens
            s.num_cached_tokens = s.num_tokens
            kv.sync_prefix(s)
            kv.deallocate(s)
        assert hits["hash"] == hits["radix"]
