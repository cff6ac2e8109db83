"""Host-side state of one request (reference: src/data/sequence.py:20-141).

Nothing in ``data/`` imports torch: the ledger lives on the driver CPU, the KV tensors live
in ``runtime/kv_pool.py``, and block ids are the only key the two sides share.
"""

from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from enum import Enum, auto

import numpy as np

from ..sampling_params import SamplingParams

__all__ = ["Sequence", "SequenceStatus", "slots_for_range", "PENDING_TOKEN"]

# Stands in ``token_ids`` for a token that the device has sampled (or is about to) but the host has not read
# yet: the engine core may launch step n + 1 before it reads step n's samples.
PENDING_TOKEN = -1

_next_seq_id = itertools.count(1)


class SequenceStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    FINISHED = auto()


def slots_for_range(block_table, start: int, end: int, block_size: int) -> list[int]:
    """Physical KV slot of every token position in ``[start, end)``.

    Slot of position ``p`` is ``block_table[p // block_size] * block_size + p % block_size``.
    Computed with one vectorised gather instead of a per-token loop.
    """
    if end <= start:
        return []
    pos = np.arange(start, end, dtype=np.int64)
    table = np.asarray(block_table, dtype=np.int64)
    return (table[pos // block_size] * block_size + pos % block_size).tolist()


@dataclass
class Sequence:
    token_ids: list[int]
    block_size: int
    seq_id: int = 0
    status: SequenceStatus = SequenceStatus.WAITING
    block_table: list[int] = field(default_factory=list)
    num_cached_tokens: int = 0      # tokens whose KV is already in the cache
    num_scheduled_tokens: int = 0   # tokens scheduled for the step in flight
    need_sample: bool = False       # this step's prefill chunk reaches the end of the prompt
    is_prefill: bool = True
    num_prompt_tokens: int = 0
    temperature: float = 0.0
    top_p: float | None = None
    top_k: int | None = None
    min_p: float | None = None
    max_tokens: int = 128
    ignore_eos: bool = False
    last_token: int = 0
    # Leading block-table entries the workers already hold; the wire carries only the rest.
    bt_synced: int = 0
    # One-step-late scheduling: trailing entries of token_ids that are still PENDING_TOKEN, and whether the
    # sequence ends (max_tokens) as soon as the step in flight has been read.
    num_pending: int = 0
    finishing: bool = False
    # timing marks filled by the engine core (seconds, time.perf_counter)
    t_arrival: float = 0.0
    t_first_token: float = 0.0
    t_finished: float = 0.0

    @classmethod
    def from_prompt(cls, token_ids, *, block_size: int, sampling: SamplingParams | None = None) -> "Sequence":
        ids = list(token_ids)
        if not ids:
            raise ValueError("empty prompt")
        sp = sampling if sampling is not None else SamplingParams()
        return cls(
            token_ids=ids, block_size=block_size, seq_id=next(_next_seq_id),
            num_prompt_tokens=len(ids), last_token=ids[-1],
            temperature=sp.temperature, top_p=sp.top_p, top_k=sp.top_k, min_p=sp.min_p,
            max_tokens=sp.max_tokens, ignore_eos=sp.ignore_eos,
        )

    # --- sizes -----------------------------------------------------------------
    def __len__(self) -> int:
        return len(self.token_ids)

    def __getitem__(self, key):
        return self.token_ids[key]

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def is_finished(self) -> bool:
        return self.status is SequenceStatus.FINISHED

    @property
    def num_completion_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def num_known_completion_tokens(self) -> int:
        """Completion tokens whose value the host has read."""
        return len(self.token_ids) - self.num_prompt_tokens - self.num_pending

    @property
    def num_blocks(self) -> int:
        return -(-len(self.token_ids) // self.block_size)

    @property
    def last_block_num_tokens(self) -> int:
        n = len(self.token_ids)
        return 0 if n == 0 else n - (self.num_blocks - 1) * self.block_size

    def num_full_blocks(self) -> int:
        return len(self.token_ids) // self.block_size

    def block_token_ids(self, i: int) -> list[int]:
        if not 0 <= i < self.num_blocks:
            raise IndexError(i)
        lo = i * self.block_size
        return self.token_ids[lo: lo + self.block_size]

    def append_token(self, token_id: int) -> None:
        self.token_ids.append(token_id)
        self.last_token = token_id

    # --- block-table edits (keep bt_synced consistent) ----------------------------
    def bt_append(self, block_id: int) -> None:
        self.block_table.append(block_id)

    def bt_replace(self, index: int, block_id: int) -> None:
        self.block_table[index] = block_id
        if index < self.bt_synced:
            self.bt_synced = index

    def bt_clear(self) -> None:
        self.block_table.clear()
        self.bt_synced = 0
