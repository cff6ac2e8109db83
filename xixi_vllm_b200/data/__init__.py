"""CPU data plane: request state, wire messages, KV page ledger and prefix indexes."""

from .block_manager import BlockManager
from .kv import KVManager
from .sequence import Sequence, SequenceStatus, slots_for_range
from .wire import DecodeBatch, EngineCoreOutput, ScheduledBatch, SchedulerOutput, SeqSchedule

__all__ = [
    "BlockManager", "KVManager", "Sequence", "SequenceStatus", "slots_for_range",
    "DecodeBatch", "EngineCoreOutput", "ScheduledBatch", "SchedulerOutput", "SeqSchedule",
]
