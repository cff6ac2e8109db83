"""Continuous-batching scheduler (reference: src/control/scheduler.py:8-218).

Parallelism-agnostic: it owns the waiting/running queues and the KV page budget and emits a
``ScheduledBatch``. Tensor/pipeline fan-out happens in the executor, data-parallel fan-out
in the client.

Policy kept from the reference:
* mixed mode (default): running sequences decode first, then waiting prompts fill what is
  left of the token budget; prefill-first mode runs prompts alone when any can start;
* a prompt that does not fit the remaining budget is chunked, at most one partial chunk
  per step;
* when a decode cannot get a page, sequences are preempted from the tail of ``running``
  and recomputed later;
* a sequence ends on EOS (unless ``ignore_eos``) or at ``max_tokens``; ``max_tokens <= 0``
  ends right after prefill.

One-step-late mode (``advance`` / ``resolve`` instead of ``update``): the engine core launches step n + 1
before it has read step n's samples, so that the host's scheduling, staging and bookkeeping overlap the
GPU's work. ``advance(batch)`` accounts for a launched step at once: KV lengths grow, every sampling row
gets a ``PENDING_TOKEN`` at the end of its ``token_ids`` (and a negative ``last_token`` that names its row
in the step's sample buffer, from which the workers fetch the next input token on the device), sequences
that reach ``max_tokens`` with that token leave ``running``. ``resolve(batch, ...)`` fills the tokens in
when they have been read, publishes the pages the step filled and ends sequences. A sequence that turns
out to have sampled EOS in step n has already been scheduled into step n + 1; that row's sample is
dropped. A preempted sequence with a pending token waits until it is resolved before it is recomputed.
(The reference schedules, runs and updates strictly in turn: src/control/core.py:74-134.)
"""

from __future__ import annotations

from collections import deque

from ..data import EngineCoreOutput, KVManager, ScheduledBatch, Sequence, SequenceStatus
from ..data.sequence import PENDING_TOKEN

__all__ = ["Scheduler"]


class Scheduler:
    def __init__(self, kv: KVManager, *, max_num_seqs: int, max_num_batched_tokens: int,
                 eos_token_id: int, mix_prefill_decode: bool = True) -> None:
        self.kv = kv
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.eos = eos_token_id
        self.mix_prefill_decode = mix_prefill_decode
        self.waiting: deque[Sequence] = deque()
        self.running: deque[Sequence] = deque()
        self._released: list[int] = []   # seq ids whose worker-side rows can be dropped
        self._step = 0
        self.num_preemptions = 0
        self.num_sampled = 0
        self._holders = 0          # waiting sequences that hold pages (prompts in the middle of their chunks)

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def add(self, seq: Sequence) -> None:
        seq.status = SequenceStatus.WAITING
        self.waiting.append(seq)

    # ------------------------------------------------------------------ scheduling
    def schedule(self) -> ScheduledBatch:
        prefills: list[Sequence] = []
        decodes: list[Sequence] = []
        if self.mix_prefill_decode:
            used = self._take_decodes(prefills, decodes, 0)
            if decodes:
                self._take_prefills(prefills, decodes, used, allow_trailing_partial=True)
            else:
                self._prefill_first(prefills, decodes)
        else:
            self._prefill_first(prefills, decodes)
        self._step += 1
        released, self._released = self._released, []
        return ScheduledBatch(prefills=prefills, decodes=decodes, released=released, step_id=self._step)

    def _prefill_first(self, prefills: list[Sequence], decodes: list[Sequence]) -> None:
        self._take_prefills(prefills, decodes, 0, allow_trailing_partial=False)
        if not prefills:
            self._take_decodes(prefills, decodes, 0)

    def _has_room(self, prefills, decodes) -> bool:
        return len(prefills) + len(decodes) < self.max_num_seqs

    def _take_decodes(self, prefills, decodes, used: int) -> int:
        run = self.running
        if not run:
            return used
        n = min(len(run), self.max_num_seqs - len(prefills) - len(decodes), self.max_num_batched_tokens - used)
        if n <= 0:
            return used
        blocks = self.kv.blocks
        if blocks.available_slots >= n:
            # Enough pages even if every sequence opened one: nobody can be preempted, so the
            # queue order is untouched and the per-sequence work is one modulo.
            bs = self.kv.block_size
            it = iter(run)
            for _ in range(n):
                seq = next(it)
                seq.num_scheduled_tokens = 1
                if len(seq.token_ids) % bs == 1 and len(seq.block_table) < seq.num_blocks:
                    seq.block_table.append(blocks.allocate_fresh())
                decodes.append(seq)
            return used + n
        while run and self._has_room(prefills, decodes) and used < self.max_num_batched_tokens:
            seq = run.popleft()
            while not self.kv.can_append(seq) and run:
                self.preempt(run.pop())
            if not self.kv.can_append(seq):
                # Nobody left to preempt among the running sequences: a half-prefilled prompt in the waiting
                # queue may still be sitting on pages. It arrived later than anything that is decoding, so it
                # gives them back and starts over; preempting `seq` instead would put it in front of that
                # prompt, restart it with the pages still missing, and repeat forever.
                self._reset_partial_prefills()
            if not self.kv.can_append(seq):
                self.preempt(seq)
                break
            seq.num_scheduled_tokens = 1
            self.kv.may_append(seq)
            decodes.append(seq)
            used += 1
        if decodes:   # scheduled sequences keep their place at the head of the queue
            run.extendleft(reversed(decodes))
        return used

    def _take_prefills(self, prefills, decodes, used: int, *, allow_trailing_partial: bool) -> int:
        blocked = False
        for seq in list(self.waiting):
            if not self._has_room(prefills, decodes):
                break
            budget = self.max_num_batched_tokens - used
            if budget <= 0:
                break
            if seq.num_pending:
                continue        # preempted with a token still unread: recomputed once the token is known
            if not seq.block_table:
                # First come, first served: once a prompt does not fit, no later prompt may take pages ahead
                # of it. A prompt further back that already holds its pages (it was cut into chunks and a
                # preempted sequence was queued in front of it) must still be allowed to finish, or the two
                # would wait for each other.
                if blocked or not self.kv.can_allocate(seq):
                    blocked = True
                    if self._holders == 0:        # nobody further back holds pages: nothing else can run
                        break
                    continue
                self.kv.allocate(seq)
                self._holders += 1
            need = seq.num_tokens - seq.num_cached_tokens
            if need <= 0:   # nothing to compute (cannot happen with the last-page rule, kept as a guard)
                self._promote(seq)
                continue
            if budget < need and prefills and not allow_trailing_partial:
                break
            chunk = min(need, budget)
            seq.num_scheduled_tokens = chunk
            prefills.append(seq)
            used += chunk
            if chunk == need:
                seq.need_sample = True
                self._promote(seq)
            else:
                seq.need_sample = False
                break   # one partial chunk per step
        return used

    def _reset_partial_prefills(self) -> None:
        """Takes the pages back from waiting sequences that hold some (prompts cut into chunks); they keep
        their place in the queue and recompute from their first token."""
        for w in self.waiting:
            if w.block_table:
                self.kv.deallocate(w, publish=False)
                self._released.append(w.seq_id)
                self.num_preemptions += 1
                self._holders -= 1

    def _promote(self, seq: Sequence) -> None:
        self._holders -= 1
        seq.status = SequenceStatus.RUNNING
        self.waiting.remove(seq)
        self.running.append(seq)

    def preempt(self, seq: Sequence) -> None:
        """Give the sequence's pages back and recompute it later from the front of the queue."""
        if seq.status is SequenceStatus.FINISHED:
            return
        seq.status = SequenceStatus.WAITING
        self.kv.deallocate(seq, publish=False)
        self._released.append(seq.seq_id)
        self.waiting.appendleft(seq)
        self.num_preemptions += 1

    # ------------------------------------------------------------------ post-step
    def update(self, sched: ScheduledBatch, p_ids: list[int], d_ids: list[int]) -> list[EngineCoreOutput]:
        out: list[EngineCoreOutput] = []
        done: set[int] = set()
        if sched.decodes:
            self._apply_decodes(sched.decodes, d_ids, out, done)
        if sched.prefills:
            self._apply(sched.prefills, p_ids, True, out, done)
        if done:
            self.running = deque(s for s in self.running if s.seq_id not in done)
            self._released.extend(done)
        return out

    def _finish(self, seq: Sequence, done: set[int]) -> None:
        seq.status = SequenceStatus.FINISHED
        self.kv.deallocate(seq, publish=True)
        done.add(seq.seq_id)

    def _apply_decodes(self, seqs, token_ids, out, done: set[int]) -> None:
        """``_apply`` for decode rows (one scheduled token, always sampled, ``max_tokens`` >= 2): the loop runs
        once per running sequence per step, so it keeps to the few operations a decode row needs."""
        publish = self.kv.prefix_backend != "none"
        sync = self.kv.sync_prefix
        eos = self.eos
        make = EngineCoreOutput
        emit = out.append
        for seq, tok in zip(seqs, token_ids):
            seq.num_cached_tokens += seq.num_scheduled_tokens
            if publish:
                sync(seq)
            seq.num_scheduled_tokens = 0
            ids = seq.token_ids
            ids.append(tok)
            seq.last_token = tok
            if (tok == eos and not seq.ignore_eos) or len(ids) - seq.num_prompt_tokens >= seq.max_tokens:
                self._finish(seq, done)
                emit(make(seq_id=seq.seq_id, new_token_ids=[tok], is_finished=True))
            else:
                emit(make(seq_id=seq.seq_id, new_token_ids=[tok]))
        self.num_sampled += len(seqs)

    def _apply(self, seqs, token_ids, is_prefill: bool, out, done: set[int]) -> None:
        publish = self.kv.prefix_backend != "none"
        eos = self.eos
        for seq, tok in zip(seqs, token_ids):
            seq.num_cached_tokens += seq.num_scheduled_tokens
            if publish:
                self.kv.sync_prefix(seq)
            seq.num_scheduled_tokens = 0
            if is_prefill and seq.num_cached_tokens < len(seq.token_ids):
                # mid-prompt chunk, or recomputation of a preempted sequence not at its end yet
                out.append(EngineCoreOutput(seq_id=seq.seq_id))
                continue
            if seq.max_tokens <= 0:
                self._finish(seq, done)
                out.append(EngineCoreOutput(seq_id=seq.seq_id, is_finished=True))
                continue
            tok = int(tok)
            seq.token_ids.append(tok)
            seq.last_token = tok
            self.num_sampled += 1
            if (tok == eos and not seq.ignore_eos) or len(seq.token_ids) - seq.num_prompt_tokens >= seq.max_tokens:
                self._finish(seq, done)
                out.append(EngineCoreOutput(seq_id=seq.seq_id, new_token_ids=[tok], is_finished=True))
            else:
                out.append(EngineCoreOutput(seq_id=seq.seq_id, new_token_ids=[tok]))

    # ------------------------------------------------------------------ one-step-late mode
    def advance(self, sched: ScheduledBatch) -> None:
        """Accounts for a step that has been launched but not read (see the module docstring)."""
        leaving = False
        marks_d, marks_p = sched.marks_d, sched.marks_p
        for i, seq in enumerate(sched.decodes):
            before = seq.num_cached_tokens
            after = before + seq.num_scheduled_tokens
            seq.num_cached_tokens = after
            seq.num_scheduled_tokens = 0
            ids = seq.token_ids
            marks_d.append((len(ids), before, after))
            ids.append(PENDING_TOKEN)
            seq.num_pending += 1
            seq.last_token = -(i + 1)
            if len(ids) - seq.num_prompt_tokens >= seq.max_tokens:
                seq.finishing = leaving = True
        k = len(sched.decodes)
        for seq in sched.prefills:
            before = seq.num_cached_tokens
            after = before + seq.num_scheduled_tokens
            seq.num_cached_tokens = after
            seq.num_scheduled_tokens = 0
            ids = seq.token_ids
            if after < len(ids):
                marks_p.append((-1, before, after))      # mid-prompt chunk (or recomputation not at its end yet)
                continue
            if seq.max_tokens <= 0:
                marks_p.append((-2, before, after))      # ends right after its prompt; its sample is not used
                seq.finishing = leaving = True
                k += 1
                continue
            marks_p.append((len(ids), before, after))
            ids.append(PENDING_TOKEN)
            seq.num_pending += 1
            seq.last_token = -(k + 1)
            k += 1
            if len(ids) - seq.num_prompt_tokens >= seq.max_tokens:
                seq.finishing = leaving = True
        if leaving:
            self.running = deque(s for s in self.running if not s.finishing)

    def resolve(self, sched: ScheduledBatch, p_ids: list[int], d_ids: list[int]) -> list[EngineCoreOutput]:
        """Fills in the tokens of a step that ``advance`` accounted for. Returns the per-sequence increments."""
        out: list[EngineCoreOutput] = []
        done: set[int] = set()
        for seq, tok, mark in zip(sched.decodes, d_ids, sched.marks_d):
            self._resolve_one(seq, tok, mark, out, done)
        for seq, tok, mark in zip(sched.prefills, p_ids, sched.marks_p):
            pos, before, after = mark
            if seq.status is SequenceStatus.FINISHED:
                continue
            if pos == -1:
                self.kv.publish_range(seq, before, after)
                out.append(EngineCoreOutput(seq_id=seq.seq_id))
            elif pos == -2:
                self.kv.publish_range(seq, before, after)
                self._finish_late(seq, done)
                out.append(EngineCoreOutput(seq_id=seq.seq_id, is_finished=True))
            else:
                self._resolve_one(seq, tok, mark, out, done)
        if done:
            self.running = deque(s for s in self.running if s.seq_id not in done)
            self._released.extend(done)
        return out

    def _resolve_one(self, seq: Sequence, tok, mark, out, done: set[int]) -> None:
        if seq.status is SequenceStatus.FINISHED:
            return            # it ended at an earlier step whose EOS was read after this row had been launched
        pos, before, after = mark
        self.kv.publish_range(seq, before, after)
        tok = int(tok)
        ids = seq.token_ids
        ids[pos] = tok
        seq.num_pending -= 1
        if seq.num_pending == 0:
            seq.last_token = tok
        self.num_sampled += 1
        hit_eos = tok == self.eos and not seq.ignore_eos
        if hit_eos or (seq.finishing and seq.num_pending == 0):
            if len(ids) > pos + 1:
                # EOS with a later step already accounted for: that step's token will not be used
                del ids[pos + 1:]
                seq.num_pending = 0
                seq.last_token = tok
                seq.num_cached_tokens = min(seq.num_cached_tokens, len(ids))
            self._finish_late(seq, done)
            out.append(EngineCoreOutput(seq_id=seq.seq_id, new_token_ids=[tok], is_finished=True))
        else:
            out.append(EngineCoreOutput(seq_id=seq.seq_id, new_token_ids=[tok]))

    def _finish_late(self, seq: Sequence, done: set[int]) -> None:
        if seq.status is SequenceStatus.WAITING:      # preempted after the step was launched
            self.waiting.remove(seq)
            if seq.block_table:
                self._holders -= 1
        seq.finishing = False
        self._finish(seq, done)

