"""Process groups for one engine replica (reference: src/distributed/parallel_state.py:23-259).

Rank layout is ``global = pp_rank * tp + tp_rank``. Every logical group carries a device
group (NCCL on GPUs, gloo on CPU) for tensors and a gloo group for control bytes and
barriers. With ``pp == 1`` the tensor-parallel group reuses the world communicators.
"""

from __future__ import annotations

import datetime
import logging
import os
from contextlib import contextmanager
from dataclasses import dataclass

import torch
import torch.distributed as dist

logger = logging.getLogger(__name__)

__all__ = [
    "Group", "get_world_group", "get_tp_group", "get_pp_group", "init_distributed_environment",
    "initialize_model_parallel", "destroy_model_parallel", "destroy_distributed_environment",
    "model_parallel_is_initialized", "graph_capture", "set_nccl_env", "single_process_groups",
]


@dataclass
class Group:
    ranks: list[int]            # global ranks, in group order
    rank: int                   # this process's global rank
    device_group: object | None  # ProcessGroup for tensors (None for a size-1 stand-in)
    cpu_group: object | None     # gloo ProcessGroup for bytes / barriers

    @property
    def size(self) -> int:
        return len(self.ranks)

    @property
    def group_rank(self) -> int:
        return self.ranks.index(self.rank)

    @property
    def is_first_rank(self) -> bool:
        return self.rank == self.ranks[0]

    @property
    def is_last_rank(self) -> bool:
        return self.rank == self.ranks[-1]

    @property
    def prev_rank(self) -> int:
        return self.ranks[(self.group_rank - 1) % self.size]

    @property
    def next_rank(self) -> int:
        return self.ranks[(self.group_rank + 1) % self.size]

    def barrier(self) -> None:
        if self.size > 1 and self.cpu_group is not None:
            dist.barrier(group=self.cpu_group)


_WORLD: Group | None = None
_TP: Group | None = None
_PP: Group | None = None
_OWNS_PG = False


def _solo() -> Group:
    return Group(ranks=[0], rank=0, device_group=None, cpu_group=None)


def single_process_groups() -> None:
    """Install size-1 groups without touching torch.distributed (tp=pp=1 engines, unit tests)."""
    global _WORLD, _TP, _PP
    _WORLD, _TP, _PP = _solo(), _solo(), _solo()


def get_world_group() -> Group:
    if _WORLD is None:
        single_process_groups()
    return _WORLD


def get_tp_group() -> Group:
    if _TP is None:
        single_process_groups()
    return _TP


def get_pp_group() -> Group:
    if _PP is None:
        single_process_groups()
    return _PP


def model_parallel_is_initialized() -> bool:
    return _TP is not None and _PP is not None


def set_nccl_env(ifname: str = "", disable_ib: bool = True) -> None:
    """NCCL defaults for a single NVLink node; ``setdefault`` so users can override
    (reference: src/distributed/parallel_state.py:247-259)."""
    env = os.environ
    if ifname:
        env.setdefault("NCCL_SOCKET_IFNAME", ifname)
        env.setdefault("GLOO_SOCKET_IFNAME", ifname)
    if disable_ib:
        env.setdefault("NCCL_IB_DISABLE", "1")
    env.setdefault("TORCH_NCCL_HEARTBEAT_TIMEOUT_SEC", "1800")
    env.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "1")


def init_distributed_environment(*, world_size: int, rank: int, local_rank: int = 0,
                                 backend: str = "nccl", init_method: str = "env://",
                                 timeout_s: float = 600.0) -> None:
    """Create the default process group (if absent) and the WORLD ``Group``."""
    global _WORLD, _OWNS_PG
    timeout = datetime.timedelta(seconds=timeout_s)
    if not dist.is_initialized():
        kwargs = dict(backend=backend, init_method=init_method, world_size=world_size, rank=rank,
                      timeout=timeout)
        if backend == "nccl":
            kwargs["device_id"] = torch.device(f"cuda:{local_rank}")
        dist.init_process_group(**kwargs)
        _OWNS_PG = True
        logger.info("process group up: rank %d/%d backend=%s", rank, world_size, backend)
    ranks = list(range(dist.get_world_size()))
    cpu = dist.group.WORLD if backend == "gloo" else dist.new_group(ranks, backend="gloo", timeout=timeout)
    _WORLD = Group(ranks=ranks, rank=dist.get_rank(), device_group=dist.group.WORLD, cpu_group=cpu)


def _make_group(rank_lists: list[list[int]], backend: str, reuse_world: bool) -> Group:
    """Collectively create one communicator pair per rank list; return the one holding this rank."""
    me = dist.get_rank()
    mine: Group | None = None
    for ranks in rank_lists:
        if reuse_world and ranks == _WORLD.ranks:
            g = Group(ranks=ranks, rank=me, device_group=_WORLD.device_group, cpu_group=_WORLD.cpu_group)
        else:
            dev = dist.new_group(ranks, backend=backend)
            cpu = dev if backend == "gloo" else dist.new_group(ranks, backend="gloo")
            g = Group(ranks=ranks, rank=me, device_group=dev, cpu_group=cpu)
        if me in ranks:
            mine = g
    assert mine is not None
    return mine


def initialize_model_parallel(tp_size: int, pp_size: int, tp_rank: int | None = None,
                              pp_rank: int | None = None, backend: str | None = None) -> None:
    global _TP, _PP
    if _WORLD is None:
        raise RuntimeError("init_distributed_environment must run first")
    world = _WORLD.size
    if tp_size * pp_size != world:
        raise ValueError(f"tp({tp_size}) * pp({pp_size}) != world size {world}")
    backend = backend or dist.get_backend()
    tp_lists = [list(range(p * tp_size, (p + 1) * tp_size)) for p in range(pp_size)]
    pp_lists = [list(range(t, world, tp_size)) for t in range(tp_size)]
    _TP = _make_group(tp_lists, backend, reuse_world=True)
    _PP = _make_group(pp_lists, backend, reuse_world=True)
    if tp_rank is not None and _TP.group_rank != tp_rank:
        raise RuntimeError(f"rank layout mismatch: tp_rank {tp_rank} vs {_TP.group_rank}")
    if pp_rank is not None and _PP.group_rank != pp_rank:
        raise RuntimeError(f"rank layout mismatch: pp_rank {pp_rank} vs {_PP.group_rank}")


def destroy_model_parallel() -> None:
    global _TP, _PP
    _TP = _PP = None


def destroy_distributed_environment() -> None:
    global _WORLD, _OWNS_PG
    _WORLD = None
    if _OWNS_PG and dist.is_initialized():
        try:
            dist.destroy_process_group()
        except Exception:  # a dead peer must not block teardown
            pass
    _OWNS_PG = False


@contextmanager
def graph_capture():
    """Barriers on both sides of CUDA-graph capture so every rank enters collectives in the
    same order (reference: src/distributed/parallel_state.py:234-244)."""
    world = get_world_group()
    world.barrier()
    try:
        yield
    finally:
        world.barrier()
