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

__all__ = ["ScheduledBatch", "SeqSchedule", "SchedulerOutput", "EngineCoreOutput"]


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


class SchedulerOutput(msgspec.Struct, array_like=True):
    prefills: list[SeqSchedule] = []
    decodes: list[SeqSchedule] = []
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

    def is_empty(self) -> bool:
        return not self.prefills and not self.decodes

    def to_wire(self) -> SchedulerOutput:
        decodes = []
        for s in self.decodes:
            if len(s.token_ids) != s.num_cached_tokens + 1:
                raise AssertionError(
                    f"decode invariant broken for seq {s.seq_id}: {len(s.token_ids)} tokens, "
                    f"{s.num_cached_tokens} cached"
                )
            decodes.append(_entry(s, [s.last_token], True))
        prefills = []
        for s in self.prefills:
            lo = s.num_cached_tokens
            prefills.append(_entry(s, s.token_ids[lo: lo + s.num_scheduled_tokens], s.need_sample))
        return SchedulerOutput(prefills=prefills, decodes=decodes, released=list(self.released),
                               step_id=self.step_id)
