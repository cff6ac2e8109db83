"""One-process-per-GPU start-up under ``torchrun`` (reference: run_torchrun.py:110-199).

Every process builds a ``Worker`` from ``RANK`` / ``LOCAL_RANK`` / ``WORLD_SIZE`` with an
``env://`` rendezvous. Rank 0 wraps its worker in a ``MultiprocExecutor`` and gets an
``Engine``; the other ranks serve broadcast commands until the driver shuts them down.
"""

from __future__ import annotations

import os

from ..config import EngineConfig

__all__ = ["launch_from_env", "env_rank_info"]


def env_rank_info() -> tuple[int, int, int]:
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def launch_from_env(config: EngineConfig):
    """Returns an ``Engine`` on rank 0. On other ranks it blocks in the worker loop and
    returns ``None`` after the driver's shutdown command."""
    import torch.distributed as dist

    from ..parallel.groups import get_world_group
    from ..runtime.worker import Worker
    from .engine import Engine
    from .executor import MultiprocExecutor, worker_loop

    rank, local_rank, world = env_rank_info()
    if config.dp_size != 1:
        raise ValueError("the torchrun path runs one replica: dp_size must be 1")
    if config.tp_size * config.pp_size != world:
        raise ValueError(f"tp({config.tp_size}) * pp({config.pp_size}) must equal WORLD_SIZE={world}")
    if world == 1:
        return Engine(config)
    worker = Worker(config, rank, rank % config.tp_size, rank // config.tp_size, local_rank=local_rank)
    try:
        worker.init_environment(init_method="env://")
        worker.initialize()
        dist.barrier(group=get_world_group().cpu_group)
        if rank == 0:
            ex = MultiprocExecutor(config, worker.device, worker.dtype, worker=worker)
            engine = Engine(config, executor=ex)
            engine._torchrun_worker = worker
            return engine
        worker_loop(worker)
        return None
    finally:
        if rank != 0:
            worker.destroy_environment()


def shutdown_from_env(engine) -> None:
    """Driver side of the torchrun teardown: stop the other ranks, then free rank 0."""
    ex = engine._client.engine_core.executor
    worker = getattr(engine, "_torchrun_worker", None)
    try:
        ex.shutdown()
    finally:
        engine.destroy()
        if worker is not None:
            worker.destroy_environment()
