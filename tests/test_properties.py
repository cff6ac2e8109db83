"""Property tests (Hypothesis) for the CPU control plane: whatever the scheduler does with a
workload (chunking, mixing, preemption, prefix reuse), every request must end with the tokens a
scheduling-independent "model" assigns to it, budgets must hold at every step and the page ledger must
stay consistent."""
import random

from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from xixi_vllm_b200.control.scheduler import Scheduler
from xixi_vllm_b200.data import KVManager, Sequence
from xixi_vllm_b200.data.sequence import slots_for_range
from xixi_vllm_b200.sampling_params import SamplingParams

EOS = 2
BS = 16


def fake_model(token_ids) -> int:
    """Next token as a pure function of the token history: the same request yields the same text however
    its prompt was chunked, cached, preempted or batched. Emits EOS now and then."""
    h = 0
    for t in token_ids:
        h = (h * 1000003 + t + 1) % 2147483647
    t = h % 37
    return EOS if t == 0 else t + 3


def expected_completion(prompt, max_tokens, ignore_eos):
    toks = list(prompt)
    out = []
    while len(out) < max_tokens:
        t = fake_model(toks)
        toks.append(t)
        out.append(t)
        if t == EOS and not ignore_eos:
            break
    return out


def _check_budgets(batch, max_seqs, budget):
    assert len(batch.prefills) + len(batch.decodes) <= max_seqs
    assert sum(s.num_scheduled_tokens for s in batch.prefills) + len(batch.decodes) <= budget
    assert sum(1 for s in batch.prefills if not s.need_sample) <= 1       # one partial chunk per step
    for s in batch.prefills + batch.decodes:
        assert len(s.block_table) >= -(-(s.num_cached_tokens + s.num_scheduled_tokens) // BS)


request = st.tuples(st.integers(1, 70),          # prompt length
                    st.integers(0, 3),           # which shared prefix (0 = none)
                    st.integers(0, 12),          # max_tokens
                    st.booleans())               # ignore_eos


@settings(max_examples=150, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow])
@given(reqs=st.lists(request, min_size=1, max_size=10),
       num_blocks=st.integers(6, 40), max_seqs=st.integers(1, 6), budget=st.integers(8, 96),
       mix=st.booleans(), backend=st.sampled_from(["none", "hash", "radix"]), seed=st.integers(0, 1000),
       arrivals=st.integers(1, 4))
def test_any_schedule_yields_the_models_tokens(reqs, num_blocks, max_seqs, budget, mix, backend, seed, arrivals):
    rnd = random.Random(seed)
    prefixes = [[], [7] * 32, list(range(100, 148)), [9, 8] * 20]
    kv = KVManager(num_blocks=num_blocks, block_size=BS, prefix_backend=backend)
    sch = Scheduler(kv, max_num_seqs=max_seqs, max_num_batched_tokens=budget, eos_token_id=EOS,
                    mix_prefill_decode=mix)
    pending = []
    for n, which, max_tokens, ignore_eos in reqs:
        prompt = (prefixes[which] + [rnd.randrange(3, 60) for _ in range(n)])
        # a request must fit the pool on its own, or no scheduler could ever run it
        if -(-(len(prompt) + max_tokens) // BS) > num_blocks:
            prompt = prompt[: max(1, num_blocks * BS - max_tokens - 1)]
        seq = Sequence.from_prompt(prompt, block_size=BS,
                                   sampling=SamplingParams(max_tokens=max_tokens, ignore_eos=ignore_eos))
        pending.append((seq, list(prompt), max_tokens, ignore_eos))
    todo = list(pending)
    steps = 0
    while todo or not sch.is_finished():
        for _ in range(arrivals):                  # requests trickle in while others run
            if todo:
                sch.add(todo.pop(0)[0])
        batch = sch.schedule()
        _check_budgets(batch, max_seqs, budget)
        batch.to_wire()
        p_ids = [fake_model(s.token_ids) for s in batch.prefills]
        d_ids = [fake_model(s.token_ids) for s in batch.decodes]
        sch.update(batch, p_ids, d_ids)
        kv.blocks.check_invariants()
        assert sch._holders == sum(1 for w in sch.waiting if w.block_table)
        steps += 1
        assert steps < 5000, "the workload does not terminate"
    for seq, prompt, max_tokens, ignore_eos in pending:
        assert seq.is_finished
        assert seq.token_ids[len(prompt):] == expected_completion(prompt, max_tokens, ignore_eos)
    assert kv.blocks.num_used == 0


@settings(max_examples=150, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow])
@given(reqs=st.lists(request, min_size=1, max_size=10),
       num_blocks=st.integers(6, 40), max_seqs=st.integers(1, 6), budget=st.integers(8, 96),
       mix=st.booleans(), backend=st.sampled_from(["none", "hash", "radix"]), seed=st.integers(0, 1000),
       arrivals=st.integers(1, 4))
def test_one_step_late_schedule_yields_the_models_tokens(reqs, num_blocks, max_seqs, budget, mix, backend, seed,
                                                         arrivals):
    """The same property when step n + 1 is scheduled and launched before step n's tokens are known
    (``advance`` / ``resolve``): the "device" keeps the true history and feeds a row whose input token the host
    does not know yet from the previous step's samples, as the workers do."""
    rnd = random.Random(seed)
    prefixes = [[], [7] * 32, list(range(100, 148)), [9, 8] * 20]
    kv = KVManager(num_blocks=num_blocks, block_size=BS, prefix_backend=backend)
    sch = Scheduler(kv, max_num_seqs=max_seqs, max_num_batched_tokens=budget, eos_token_id=EOS,
                    mix_prefill_decode=mix)
    pending = []
    for n, which, max_tokens, ignore_eos in reqs:
        prompt = (prefixes[which] + [rnd.randrange(3, 60) for _ in range(n)])
        if -(-(len(prompt) + max_tokens) // BS) > num_blocks:
            prompt = prompt[: max(1, num_blocks * BS - max_tokens - 1)]
        seq = Sequence.from_prompt(prompt, block_size=BS,
                                   sampling=SamplingParams(max_tokens=max_tokens, ignore_eos=ignore_eos))
        pending.append((seq, list(prompt), max_tokens, ignore_eos))
    todo = list(pending)
    steps = 0
    inflight = None            # (batch, prefill samples, decode samples) of the launched step
    prev_samples: list[int] = []
    while todo or not sch.is_finished() or inflight is not None:
        for _ in range(arrivals):
            if todo:
                sch.add(todo.pop(0)[0])
        batch = sch.schedule()
        launched = None
        if not batch.is_empty():
            _check_budgets(batch, max_seqs, budget)
            wire = batch.to_wire()
            # the device: resolve references into the previous step's samples, then run the model on the
            # true history (host history up to the pending tokens + the referenced sample)
            d_ids, p_ids, samples = [], [], []
            for s, tok in zip(batch.decodes, wire.decodes.tokens):
                hist = list(s.token_ids)
                if tok < 0:
                    assert s.num_pending == 1 and hist[-1] == -1
                    hist[-1] = prev_samples[-tok - 1]
                else:
                    assert s.num_pending == 0 and hist[-1] == tok
                t = fake_model(hist)
                d_ids.append(t)
                samples.append(t)
            for s in batch.prefills:
                assert s.num_pending == 0 and -1 not in s.token_ids
                t = fake_model(s.token_ids)
                p_ids.append(t)
                if s.need_sample:
                    samples.append(t)
            sch.advance(batch)
            launched = (batch, p_ids, d_ids)
            this_samples = samples
        if inflight is not None:
            sch.resolve(*inflight)
        if launched is not None:
            prev_samples = this_samples
        inflight = launched
        kv.blocks.check_invariants()
        assert sch._holders == sum(1 for w in sch.waiting if w.block_table)
        steps += 1
        assert steps < 5000, "the workload does not terminate"
    for seq, prompt, max_tokens, ignore_eos in pending:
        assert seq.is_finished and seq.num_pending == 0
        assert seq.token_ids[len(prompt):] == expected_completion(prompt, max_tokens, ignore_eos)
    assert kv.blocks.num_used == 0


@settings(max_examples=200, deadline=None, derandomize=True)
@given(table=st.lists(st.integers(0, 500), min_size=1, max_size=12, unique=True),
       start=st.integers(0, 150), count=st.integers(0, 150), bs=st.sampled_from([16, 32, 64]))
def test_slots_for_range_matches_definition(table, start, count, bs):
    end = min(start + count, len(table) * bs)
    start = min(start, end)
    got = [int(x) for x in slots_for_range(table, start, end, bs)]
    assert got == [table[i // bs] * bs + i % bs for i in range(start, end)]


@settings(max_examples=60, deadline=None, derandomize=True)
@given(prompts=st.lists(st.tuples(st.integers(0, 2), st.integers(0, 80), st.integers(1, 40)), min_size=1, max_size=25),
       seed=st.integers(0, 100))
def test_hash_and_radix_backends_report_the_same_hits(prompts, seed):
    """Both prefix indexes implement the same contract (full pages, chained identity): with a pool large
    enough that nothing is evicted they must find exactly the same cached prefix for every request."""
    rnd = random.Random(seed)
    bases = [[rnd.randrange(50) for _ in range(96)] for _ in range(3)]
    kvs = {b: KVManager(num_blocks=4096, block_size=BS, prefix_backend=b) for b in ("hash", "radix")}
    for which, cut, tail in prompts:
        toks = bases[which][:cut] + [rnd.randrange(50, 99) for _ in range(tail)]
        hits = {}
        for name, kv in kvs.items():
            s = Sequence.from_prompt(toks, block_size=BS)
            kv.allocate(s)
            hits[name] = s.num_cached_tokens
            assert s.num_cached_tokens % BS == 0 and s.num_cached_tokens < len(toks)
            s.num_scheduled_tokens = s.num_tokens - s.num_cached_tokens
            s.num_cached_tokens = s.num_tokens
            kv.sync_prefix(s)
            kv.deallocate(s)
            kv.blocks.check_invariants()
        assert hits["hash"] == hits["radix"]


op = st.one_of(
    st.tuples(st.just("insert"), st.lists(st.integers(0, 3), min_size=1, max_size=8)),
    st.tuples(st.just("match"), st.lists(st.integers(0, 3), min_size=0, max_size=9)),
    st.tuples(st.just("evict"), st.integers(1, 6)),
)


@settings(max_examples=300, deadline=None, derandomize=True)
@given(ops=st.lists(op, min_size=1, max_size=40))
def test_radix_tree_behaves_like_a_prefix_dictionary(ops):
    """Model: a dict from every stored key prefix to the value first stored for it. Matching returns the
    values along the longest stored prefix; eviction only ever removes prefixes nothing longer hangs on."""
    from xixi_vllm_b200.data.prefix.radix_tree import RadixTree
    tree, model, fresh = RadixTree(), {}, iter(range(10 ** 6))
    for kind, arg in ops:
        if kind == "insert":
            vals = [next(fresh) for _ in arg]
            known = 0
            while known < len(arg) and tuple(arg[:known + 1]) in model:
                known += 1
            matched, _ = tree.insert(arg, vals)
            assert matched == known
            for i in range(known, len(arg)):
                model[tuple(arg[:i + 1])] = vals[i]
        elif kind == "match":
            want = []
            for i in range(len(arg)):
                if tuple(arg[:i + 1]) not in model:
                    break
                want.append(model[tuple(arg[:i + 1])])
            assert tree.match_prefix(arg)[0] == want
        else:
            freed = set(tree.evict(arg))
            assert len(freed) <= max(arg, 0) + 8            # whole edges go at once, never the whole tree by accident
            gone = [p for p, v in model.items() if v in freed]
            assert len(gone) == len(freed)
            for p in gone:
                del model[p]
            for p in model:                                  # what is left is still closed under taking prefixes
                assert all(p[:i] in model for i in range(1, len(p)))
        for v in model.values():
            assert tree.contains_block(v)
    assert sum(1 for _ in model) == sum(1 for v in set(model.values()))


_isolated: dict = {}


@settings(max_examples=12, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])
@given(lens=st.lists(st.integers(1, 70), min_size=2, max_size=6), shared=st.integers(0, 40),
       blocks=st.integers(8, 24), budget=st.integers(16, 64), max_seqs=st.integers(1, 4),
       backend=st.sampled_from(["none", "hash", "radix"]), new=st.integers(1, 6))
def test_engine_output_of_a_request_does_not_depend_on_its_neighbours(tiny_model_dir, lens, shared, blocks, budget,
                                                                     max_seqs, backend, new):
    """The whole CPU engine (scheduler, page ledger, prefix caches, staging with persistent block-table rows,
    paged oracle attention): under any pool size, token budget and prefix backend, with chunked prefills and
    preemptions, each request generates exactly what it generates when it runs alone in a roomy engine."""
    import torch

    from xixi_vllm_b200 import Engine, EngineConfig, SamplingParams
    g = torch.Generator().manual_seed(shared * 131 + len(lens))
    common = torch.randint(0, 1024, (shared,), generator=g).tolist()
    prompts = [common + torch.randint(0, 1024, (n,), generator=g).tolist() for n in lens]
    need = max(-(-(len(p) + new) // 16) for p in prompts)

    def run(ps, **kw):
        eng = Engine(EngineConfig(model=tiny_model_dir, device="cpu", dtype="float32", context_len=256, **kw))
        try:
            seqs = [eng.add_request(p, SamplingParams(max_tokens=new, ignore_eos=True)) for p in ps]
            while eng.has_unfinished():
                eng.step()
            return [s.token_ids[s.num_prompt_tokens:] for s in seqs]
        finally:
            eng.destroy()

    want = []
    for p in prompts:
        key = (tuple(p), new)
        if key not in _isolated:
            _isolated[key] = run([p], num_kvcache_blocks=64, max_num_seqs=1, max_num_batched_tokens=256,
                                 prefix_backend="none")[0]
        want.append(_isolated[key])
    got = run(prompts, num_kvcache_blocks=max(blocks, need), max_num_seqs=max_seqs, max_num_batched_tokens=budget,
              prefix_backend=backend)
    assert got == want
