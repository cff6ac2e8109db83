"""Scheduler and engine-core semantics with a scripted fake executor (CPU only)."""
import pytest

from xixi_vllm_b200.control.scheduler import Scheduler
from xixi_vllm_b200.data import KVManager, Sequence, SequenceStatus
from xixi_vllm_b200.sampling_params import SamplingParams

EOS = 2


def make(num_blocks=64, max_seqs=4, budget=64, mix=True, backend="none"):
    kv = KVManager(num_blocks=num_blocks, block_size=16, prefix_backend=backend)
    return Scheduler(kv, max_num_seqs=max_seqs, max_num_batched_tokens=budget, eos_token_id=EOS,
                     mix_prefill_decode=mix), kv


def req(n, **kw):
    return Sequence.from_prompt(list(range(10, 10 + n)), block_size=16, sampling=SamplingParams(**kw))


def run_step(sch, token=5):
    b = sch.schedule()
    b.to_wire()
    out = sch.update(b, [token] * len(b.prefills), [token] * len(b.decodes))
    return b, out


def test_prefill_then_decode_and_length_finish():
    sch, kv = make()
    s = req(20, max_tokens=3, ignore_eos=True)
    sch.add(s)
    b, out = run_step(sch)
    assert [x.seq_id for x in b.prefills] == [s.seq_id] and not b.decodes
    assert s.status is SequenceStatus.RUNNING and s.num_completion_tokens == 1
    b, _ = run_step(sch)
    assert [x.seq_id for x in b.decodes] == [s.seq_id]
    _, out = run_step(sch)
    assert s.is_finished and out[-1].is_finished and sch.is_finished()
    kv.blocks.check_invariants()
    assert kv.blocks.num_used == 0


def test_eos_finishes_unless_ignored():
    sch, _ = make()
    a, b = req(5, max_tokens=10), req(5, max_tokens=10, ignore_eos=True)
    sch.add(a); sch.add(b)
    run_step(sch, token=EOS)
    assert a.is_finished and not b.is_finished


def test_max_tokens_zero_finishes_after_prefill():
    sch, _ = make()
    s = req(5, max_tokens=0)
    sch.add(s)
    _, out = run_step(sch)
    assert s.is_finished and out[0].new_token_ids == [] and out[0].is_finished


def test_chunked_prefill_one_partial_chunk_per_step():
    sch, _ = make(budget=32)
    a, b = req(50, max_tokens=2, ignore_eos=True), req(10, max_tokens=2, ignore_eos=True)
    sch.add(a); sch.add(b)
    bt, out = run_step(sch)
    assert [s.num_cached_tokens for s in (a, b)] == [32, 0] and out[0].new_token_ids == []
    assert len(bt.prefills) == 1                      # the partial chunk blocks the queue behind it
    bt, _ = run_step(sch)
    assert a.num_cached_tokens == 50 and a.num_completion_tokens == 1
    assert b.num_cached_tokens == 10 and b.num_completion_tokens == 1   # remaining budget went to b


def test_mixed_mode_decodes_first_then_fills_budget():
    sch, _ = make(budget=40)
    a = req(8, max_tokens=8, ignore_eos=True)
    sch.add(a)
    run_step(sch)
    b = req(100, max_tokens=2, ignore_eos=True)
    sch.add(b)
    bt, _ = run_step(sch)
    assert [s.seq_id for s in bt.decodes] == [a.seq_id]
    assert [s.seq_id for s in bt.prefills] == [b.seq_id] and b.num_cached_tokens == 39


def test_prefill_first_mode_runs_prompts_alone():
    sch, _ = make(mix=False)
    a = req(8, max_tokens=8, ignore_eos=True)
    sch.add(a)
    run_step(sch)
    sch.add(req(8, max_tokens=2, ignore_eos=True))
    bt, _ = run_step(sch)
    assert bt.prefills and not bt.decodes


def test_max_num_seqs_caps_a_step():
    sch, _ = make(max_seqs=2, budget=1000)
    for _ in range(5):
        sch.add(req(4, max_tokens=3, ignore_eos=True))
    bt, _ = run_step(sch)
    assert len(bt.prefills) == 2


def test_preemption_recomputes_and_output_is_complete():
    sch, kv = make(num_blocks=4, max_seqs=4, budget=256)
    a, b = req(16, max_tokens=40, ignore_eos=True), req(16, max_tokens=40, ignore_eos=True)
    sch.add(a); sch.add(b)
    steps = 0
    while not sch.is_finished():
        run_step(sch)
        kv.blocks.check_invariants()
        steps += 1
        assert steps < 500
    assert sch.num_preemptions > 0
    assert a.num_completion_tokens == 40 and b.num_completion_tokens == 40


def _drain(sch, kv, limit=2000):
    steps = 0
    while not sch.is_finished():
        run_step(sch)
        kv.blocks.check_invariants()
        steps += 1
        assert steps < limit, "the scheduler makes no progress"
    return steps


def test_decode_out_of_pages_takes_them_from_a_half_prefilled_prompt():
    """A decoding sequence that needs one more page while a later prompt, cut into chunks, holds the rest of
    the pool: the prompt gives its pages back. (Preempting the decoding sequence instead queued it in front
    of the prompt and restarted it with the pages still missing, forever.)"""
    sch, kv = make(num_blocks=14, max_seqs=2, budget=8)
    a, b = req(105, max_tokens=9, ignore_eos=True), req(97, max_tokens=0)
    sch.add(a)
    run_step(sch)
    sch.add(b)
    _drain(sch, kv)
    assert a.num_completion_tokens == 9 and b.is_finished and kv.blocks.num_used == 0


def test_blocked_prompt_does_not_stop_a_later_prompt_that_already_holds_pages():
    """Queue [page-less prompt that does not fit, half-prefilled prompt holding pages]: the second one must
    still be scheduled, otherwise both wait for each other until the idle guard fires."""
    sch, kv = make(num_blocks=8, max_seqs=4, budget=16)
    big, held = req(100, max_tokens=2, ignore_eos=True), req(60, max_tokens=2, ignore_eos=True)
    sch.add(held)
    run_step(sch)                                   # first 16-token chunk of `held`: it now owns 4 pages
    assert held.block_table and not held.is_finished
    sch.waiting.appendleft(big)                     # a preempted sequence is re-queued at the front like this
    big.status = SequenceStatus.WAITING
    _drain(sch, kv)
    assert big.num_completion_tokens == 2 and held.num_completion_tokens == 2


def test_released_ids_reach_the_wire():
    sch, _ = make()
    s = req(5, max_tokens=1, ignore_eos=True)
    sch.add(s)
    run_step(sch)
    assert s.is_finished
    sch.add(req(5, max_tokens=1))
    b = sch.schedule()
    assert s.seq_id in b.to_wire().released


class FakeExecutor:
    def __init__(self, num_blocks):
        self.num_blocks, self.config = num_blocks, None

    def init_kv(self):
        return KVManager(num_blocks=self.num_blocks, block_size=16, prefix_backend="none")

    def reset_kv(self, prefix_backend=None):
        return self.init_kv()

    def run(self, sched):
        sched.to_wire()
        return len(sched.prefills), len(sched.decodes)

    def read_samples(self, n_p, n_d):
        return [7] * n_p, [7] * n_d

    def destroy(self):
        pass


def _core(tmp_path, num_blocks, **cfg_kw):
    from xixi_vllm_b200.config import EngineConfig
    from xixi_vllm_b200.control.core import EngineCore
    from xixi_vllm_b200.models.synth import make_model_dir
    d = make_model_dir(str(tmp_path / "m"), "tiny", weights=False)
    cfg = EngineConfig(model=d, device="cpu", **cfg_kw)
    return EngineCore(cfg, eos_token_id=EOS, executor=FakeExecutor(num_blocks))


def test_idle_guard_raises_on_kv_exhaustion(tmp_path):
    core = _core(tmp_path, num_blocks=2, max_num_seqs=4, max_num_batched_tokens=256)
    core._MAX_IDLE_STEPS = 5
    core.add_request(req(100, max_tokens=4))          # needs 7 pages, the pool has 2
    with pytest.raises(RuntimeError, match="KV pool exhaustion"):
        for _ in range(10):
            core.step()


def test_core_metrics_count_tokens(tmp_path):
    core = _core(tmp_path, num_blocks=64, max_num_seqs=4, max_num_batched_tokens=256)
    core.add_request(req(20, max_tokens=3, ignore_eos=True))
    total = 0
    while core.has_unfinished():
        total += core.step()[1]
    m = core.metrics.summary()
    assert total == 20 + 2 and m["sampled_tokens"] == 3 and m["requests_finished"] == 1
    assert "xv_steps" in core.metrics.to_prometheus()


def test_one_step_late_core_drains_counts_and_guards(tmp_path):
    """The core in one-step-late mode: outputs arrive one call later, the last launched step is read before
    has_unfinished() turns false or the KV pool is rebuilt, token counts are those of the steps that were read, and
    the idle guard still fires when nothing is in flight and nothing can be scheduled."""
    core = _core(tmp_path, num_blocks=64, max_num_seqs=4, max_num_batched_tokens=256, async_scheduling="on")
    assert core.one_step_late
    core.add_request(req(20, max_tokens=3, ignore_eos=True))
    outs, n = core.step()                       # launches the prefill; nothing to read yet
    assert outs == [] and n == 0 and core.has_unfinished() and core._inflight is not None
    outs, n = core.step()                       # launches decode 1, reads the prefill
    assert n == 20 and [o.new_token_ids for o in outs] == [[7]]
    total, finished = n, 0
    while core.has_unfinished():
        outs, n = core.step()
        total += n
        finished += sum(o.is_finished for o in outs)
    m = core.metrics.summary()
    assert total == 20 + 2 and finished == 1 and m["sampled_tokens"] == 3 and m["requests_finished"] == 1
    assert core._inflight is None
    # reset_kv while a step is in flight: the step is read first
    core.add_request(req(10, max_tokens=5, ignore_eos=True))
    core.step()
    assert core._inflight is not None
    core.reset_kv()
    assert core._inflight is None
    # idle guard
    small = _core(tmp_path / "b", num_blocks=2, max_num_seqs=4, max_num_batched_tokens=256, async_scheduling="on")
    small._MAX_IDLE_STEPS = 5
    small.add_request(req(100, max_tokens=4))
    with pytest.raises(RuntimeError, match="KV pool exhaustion"):
        for _ in range(10):
            small.step()
