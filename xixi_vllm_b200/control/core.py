"""One engine step: schedule, execute, read samples, update (reference: src/control/core.py:25-156).

With ``config.one_step_late`` the order inside ``step()`` becomes: schedule and launch step n + 1, THEN read
step n's samples and apply them, so the host's scheduling, staging, launch, bookkeeping and whatever the
caller does between two ``step()`` calls run while the GPU is busy. ``step()`` then returns the outputs of the
step launched by the previous call."""

from __future__ import annotations

import gc
import time

from ..config import EngineConfig
from ..data import EngineCoreOutput, KVManager, Sequence
from ..utils.metrics import EngineMetrics
from .scheduler import Scheduler

__all__ = ["EngineCore"]


class EngineCore:
    # Consecutive empty schedules tolerated while requests remain; beyond this the KV pool
    # is assumed exhausted and the step raises instead of spinning forever.
    _MAX_IDLE_STEPS = 1024

    def __init__(self, config: EngineConfig, *, eos_token_id: int, device=None, dtype=None,
                 executor=None) -> None:
        self.config = config
        self.eos_token_id = eos_token_id
        if executor is None:
            from .executor import create_executor

            executor = create_executor(config, device, dtype)
        self.executor = executor
        self.metrics = EngineMetrics()
        self._idle_steps = 0
        self.one_step_late = bool(getattr(config, "one_step_late", False))
        self._inflight = None           # (batch, n_prefill, n_decode, prefill tokens, t_schedule, t_launch)
        self._init_kv()

    def _build_scheduler(self) -> Scheduler:
        return Scheduler(
            self.kv,
            max_num_seqs=self.config.max_num_seqs,
            max_num_batched_tokens=self.config.max_num_batched_tokens,
            eos_token_id=self.eos_token_id,
            mix_prefill_decode=self.config.mix_prefill_decode,
        )

    def _init_kv(self) -> None:
        self.kv: KVManager = self.executor.init_kv()
        self.scheduler = self._build_scheduler()
        self.last_num_cached_tokens = 0

    def reset_kv(self, prefix_backend: str | None = None) -> None:
        if self._inflight is not None:          # read the step in flight before its pages go away
            prev, self._inflight = self._inflight, None
            self._read_and_resolve(prev)
        self.kv = self.executor.reset_kv(prefix_backend)
        sampled = self.scheduler.num_sampled
        self.scheduler = self._build_scheduler()
        self.scheduler.num_sampled = sampled
        self.last_num_cached_tokens = 0

    def add_request(self, seq: Sequence) -> None:
        if not seq.t_arrival:
            seq.t_arrival = time.perf_counter()
        self.metrics.requests_added += 1
        self.scheduler.add(seq)

    def has_unfinished(self) -> bool:
        return self._inflight is not None or not self.scheduler.is_finished()

    def step(self) -> tuple[list[EngineCoreOutput], int]:
        """Returns (per-sequence increments, tokens processed this step)."""
        if self.one_step_late:
            return self._step_late()
        t0 = time.perf_counter()
        sched = self.scheduler.schedule()
        if sched.is_empty():
            if sched.released:
                # nothing to run, but workers should still learn about dropped rows
                self.scheduler._released[:0] = sched.released
            if not self.scheduler.is_finished():
                self._idle_steps += 1
                if self._idle_steps >= self._MAX_IDLE_STEPS:
                    raise RuntimeError(
                        "scheduler returned empty for too long while requests remain "
                        f"(idle_steps={self._idle_steps}). Likely KV pool exhaustion "
                        f"(free_blocks={self.kv.num_free})."
                    )
            return [], 0
        self._idle_steps = 0
        t1 = time.perf_counter()
        n_p, n_d = self.executor.run(sched)
        self.last_num_cached_tokens = self.kv.last_num_cached_tokens
        prefill_tokens = sum(s.num_scheduled_tokens for s in sched.prefills)
        metric = prefill_tokens + len(sched.decodes)
        p_ids, d_ids = self.executor.read_samples(n_p, n_d)
        t2 = time.perf_counter()
        outputs = self.scheduler.update(sched, p_ids, d_ids)
        t3 = time.perf_counter()
        by_id = None

        def lookup(seq_id):          # built only when a request finished this step
            nonlocal by_id
            if by_id is None:
                by_id = {s.seq_id: s for s in sched.decodes}
                by_id.update((s.seq_id, s) for s in sched.prefills)
            return by_id.get(seq_id)

        self.metrics.on_step(
            sched, outputs, prefill_tokens, schedule_s=t1 - t0, execute_s=t2 - t1, update_s=t3 - t2,
            kv_usage=self.kv.usage(), preemptions=self.scheduler.num_preemptions, kv=self.kv, now=t3,
            sampled_total=self.scheduler.num_sampled, finished_lookup=lookup,
        )
        return outputs, metric

    def _step_late(self) -> tuple[list[EngineCoreOutput], int]:
        """Launch the next step, then read and apply the one launched by the previous call."""
        t0 = time.perf_counter()
        prev = self._inflight
        sched = self.scheduler.schedule()
        launched = None
        if sched.is_empty():
            if sched.released:
                self.scheduler._released[:0] = sched.released
            if prev is None and not self.scheduler.is_finished():
                self._idle_steps += 1
                if self._idle_steps >= self._MAX_IDLE_STEPS:
                    raise RuntimeError(
                        "scheduler returned empty for too long while requests remain "
                        f"(idle_steps={self._idle_steps}). Likely KV pool exhaustion "
                        f"(free_blocks={self.kv.num_free})."
                    )
        else:
            self._idle_steps = 0
            t1 = time.perf_counter()
            n_p, n_d = self.executor.run(sched)
            self.last_num_cached_tokens = self.kv.last_num_cached_tokens
            prefill_tokens = sum(s.num_scheduled_tokens for s in sched.prefills)
            self.scheduler.advance(sched)
            launched = (sched, n_p, n_d, prefill_tokens, t1 - t0, time.perf_counter())
        self._inflight = launched
        if prev is None:
            return [], 0
        return self._read_and_resolve(prev)

    def _read_and_resolve(self, prev) -> tuple[list[EngineCoreOutput], int]:
        """Reads the samples of a launched step and applies them."""
        p_sched, n_p, n_d, prefill_tokens, schedule_s, t_launch = prev
        p_ids, d_ids = self.executor.read_samples(n_p, n_d)
        t2 = time.perf_counter()
        outputs = self.scheduler.resolve(p_sched, p_ids, d_ids)
        t3 = time.perf_counter()
        by_id = None

        def lookup(seq_id):
            nonlocal by_id
            if by_id is None:
                by_id = {s.seq_id: s for s in p_sched.decodes}
                by_id.update((s.seq_id, s) for s in p_sched.prefills)
            return by_id.get(seq_id)

        self.metrics.on_step(
            p_sched, outputs, prefill_tokens, schedule_s=schedule_s, execute_s=t2 - t_launch, update_s=t3 - t2,
            kv_usage=self.kv.usage(), preemptions=self.scheduler.num_preemptions, kv=self.kv, now=t3,
            sampled_total=self.scheduler.num_sampled, finished_lookup=lookup,
        )
        return outputs, prefill_tokens + len(p_sched.decodes)

    def destroy(self) -> None:
        self.executor.destroy()
        self.kv = None
        self.scheduler = None
        gc.collect()
