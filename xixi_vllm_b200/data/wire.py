"""Messages between the driver's scheduler and the workers (reference: src/data/batch.py:21-117).

``ScheduledBatch`` holds live ``Sequence`` objects and never leaves the driver.
``to_wire()`` reduces it to what a forward pass needs. Unlike the reference, a sequence's
block table is sent as a *tail*: only entries the workers have not seen yet
(``bt_from`` = index of the first entry carried). With 16-token pages a 4096-token
context has 256 entries; resending all of them for every sequence on every step would
dominate the control message.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import msgspec

from .sequence import Sequence

__all__ = ["ScheduledBatch", "SeqSchedule", "DecodeBatch", "SchedulerOutput", "EngineCoreOutput"]


class SeqSchedule(msgspec.Struct, array_like=True):
    """Forward-pass input for one sequence.

    ``token_ids`` is ``[last_token]`` for decode and this step's chunk for prefill.
    ``num_cached_tokens`` is the KV length before this step (gives positions and slots).
    ``bt_tail`` are block-table entries ``bt_from, bt_from+1, ...``; earlier entries are
    unchanged since the last message that named this ``seq_id``.
    """

    seq_id: int
    num_cached_tokens: int
    token_ids: list[int]
    bt_from: int = 0
    bt_tail: list[int] = []
    need_sample: bool = False
    temperature: float = 0.0
    top_p: float | None = None
    top_k: int | None = None
    min_p: float | None = None


class DecodeBatch(msgspec.Struct, array_like=True):
    """All decode rows of a step as parallel arrays (one new token per sequence).

    A decode step of 256 sequences is 256 tiny records; building, encoding and decoding them
    as objects costs more host time than the GPU needs for a tensor-parallel step, so they
    travel as flat integer lists. Sampling parameters are not repeated: workers remember them
    from the sequence's prefill message. Block-table growth is sparse (a new page every
    ``block_size`` tokens): ``bt_index[j]`` names the row of this batch whose table gets
    ``bt_count[j]`` entries from ``bt_vals`` starting at table position ``bt_from[j]``.
    """

    seq_ids: list[int] = []
    tokens: list[int] = []
    cached: list[int] = []        # KV length before this step
    bt_index: list[int] = []
    bt_from: list[int] = []
    bt_count: list[int] = []
    bt_vals: list[int] = []

    def __len__(self) -> int:
        return len(self.seq_ids)

    def __bool__(self) -> bool:
        return bool(self.seq_ids)

    @classmethod
    def of(cls, entries) -> "DecodeBatch":
        """From ``(seq_id, token, cached, bt_from, bt_tail)`` tuples (tests, graph capture)."""
        b = cls(seq_ids=[], tokens=[], cached=[], bt_index=[], bt_from=[], bt_count=[], bt_vals=[])
        for i, (sid, tok, cached, start, tail) in enumerate(entries):
            b.seq_ids.append(sid)
            b.tokens.append(tok)
            b.cached.append(cached)
            if tail:
                b.bt_index.append(i)
                b.bt_from.append(start)
                b.bt_count.append(len(tail))
                b.bt_vals.extend(tail)
        return b


class SchedulerOutput(msgspec.Struct, array_like=True):
    prefills: list[SeqSchedule] = []
    decodes: DecodeBatch = msgspec.field(default_factory=DecodeBatch)
    # sequences that finished or were preempted since the previous message: workers
    # drop their cached block-table rows
    released: list[int] = []
    step_id: int = 0


class EngineCoreOutput(msgspec.Struct):
    """Per-sequence increment of one step; empty ``new_token_ids`` means nothing was sampled."""

    seq_id: int
    new_token_ids: list[int] = msgspec.field(default_factory=list)
    is_finished: bool = False


def _entry(s: Sequence, token_ids: list[int], need_sample: bool) -> SeqSchedule:
    start = s.bt_synced
    tail = s.block_table[start:]
    s.bt_synced = len(s.block_table)
    return SeqSchedule(
        seq_id=s.seq_id, num_cached_tokens=s.num_cached_tokens, token_ids=token_ids,
        bt_from=start, bt_tail=tail, need_sample=need_sample,
        temperature=s.temperature, top_p=s.top_p, top_k=s.top_k, min_p=s.min_p,
    )


@dataclass
class ScheduledBatch:
    prefills: list[Sequence] = field(default_factory=list)
    decodes: list[Sequence] = field(default_factory=list)
    released: list[int] = field(default_factory=list)
    step_id: int = 0
    # one-step-late scheduling: per decode / prefill row, (position of its pending token in token_ids or a
    # negative code, KV length before the step, KV length after it), written by Scheduler.advance
    marks_d: list = field(default_factory=list)
    marks_p: list = field(default_factory=list)

    def is_empty(self) -> bool:
        return not self.prefills and not self.decodes

    def to_wire(self) -> SchedulerOutput:
        dec = self.decodes
        d = DecodeBatch(seq_ids=[s.seq_id for s in dec], tokens=[s.last_token for s in dec],
                        cached=[s.num_cached_tokens for s in dec], bt_index=[], bt_from=[], bt_count=[], bt_vals=[])
        for i, s in enumerate(dec):
            n = len(s.block_table)
            if s.bt_synced != n:
                if len(s.token_ids) != s.num_cached_tokens + 1:
                    raise AssertionError(
                        f"decode invariant broken for seq {s.seq_id}: {len(s.token_ids)} tokens, "
                        f"{s.num_cached_tokens} cached")
                d.bt_index.append(i)
                d.bt_from.append(s.bt_synced)
                d.bt_count.append(n - s.bt_synced)
                d.bt_vals.extend(s.block_table[s.bt_synced:])
                s.bt_synced = n
        prefills = []
        for s in self.prefills:
            lo = s.num_cached_tokens
            prefills.append(_entry(s, s.token_ids[lo: lo + s.num_scheduled_tokens], s.need_sample))
        return SchedulerOutput(prefills=prefills, decodes=d, released=list(self.released), step_id=self.step_id)
