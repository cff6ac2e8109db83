"""Bridge between the engine core and the workers (reference: src/control/executor.py:29-467).

``tp*pp == 1``: ``UniprocExecutor`` calls the worker in-process. Otherwise
``MultiprocExecutor``: rank 0 is both driver and worker; each step's ``SchedulerOutput`` is
msgpack-encoded and broadcast over gloo, every rank runs the forward, and the sampler rank
(first rank of the last pipeline stage) sends the ids back when it is not rank 0.
"""

from __future__ import annotations

import multiprocessing as mp
import os
from abc import ABC, abstractmethod

import msgspec

from ..config import EngineConfig
from ..data import KVManager, ScheduledBatch, SchedulerOutput
from ..parallel.control_channel import ControlChannel
from ..parallel.groups import get_world_group

__all__ = ["ControlCommand", "Executor", "UniprocExecutor", "MultiprocExecutor", "create_executor",
           "worker_loop"]


def _sampler_rank(tp_size: int, pp_size: int) -> int:
    """Global rank that samples: tensor-parallel rank 0 of the last pipeline stage."""
    return (pp_size - 1) * tp_size


def _terminate_procs(procs: list) -> None:
    """SIGTERM, wait 3 s, SIGKILL, wait 5 s: a child stuck in a blocking call cannot keep the
    driver from exiting."""
    for p in procs:
        if p.is_alive():
            p.terminate()
    for p in procs:
        p.join(timeout=3)
    for p in procs:
        if p.is_alive():
            p.kill()
    for p in procs:
        p.join(timeout=5)
    procs.clear()


class ControlCommand(msgspec.Struct):
    op: str                                  # "execute" | "reset_kv" | "device_time" | "shutdown"
    sched: SchedulerOutput | None = None
    prefix_backend: str | None = None
    args: list[int] = []


class Executor(ABC):
    def __init__(self, config: EngineConfig, device=None, dtype=None) -> None:
        self.config, self.device, self.dtype = config, device, dtype
        self.sampler_rank = _sampler_rank(config.tp_size, config.pp_size)
        self.kv: KVManager | None = None

    def _kv_manager(self, num_blocks: int) -> KVManager:
        return KVManager(num_blocks=num_blocks, block_size=self.config.block_size,
                         prefix_backend=self.config.prefix_backend)

    @abstractmethod
    def init_kv(self) -> KVManager: ...

    @abstractmethod
    def reset_kv(self, prefix_backend: str | None = None) -> KVManager: ...

    @abstractmethod
    def run(self, sched: ScheduledBatch) -> tuple[int, int]: ...

    @abstractmethod
    def read_samples(self, n_p: int, n_d: int) -> tuple[list[int], list[int]]: ...

    @abstractmethod
    def destroy(self) -> None: ...

    def collective_rpc(self, op: str, **payload) -> object:
        raise ValueError(f"unknown control op: {op}")

    def shutdown(self) -> None:
        return None


def _spawn_worker(config: EngineConfig, rank: int, tp_rank: int, pp_rank: int, rdv_tag: str) -> None:
    import torch.distributed as dist

    from ..runtime.worker import Worker

    os.environ["XV_RDV_TAG"] = rdv_tag
    worker = Worker(config, rank, tp_rank, pp_rank)
    try:
        worker.init_environment()
        worker.initialize()
        dist.barrier(group=get_world_group().cpu_group)
        worker_loop(worker)
    finally:
        worker.destroy_environment()


def worker_loop(worker) -> None:
    """Ranks >= 1: wait for broadcast commands until ``shutdown``."""
    sampler_rank = _sampler_rank(worker.tp_size, worker.pp_size)
    channel = ControlChannel(get_world_group().cpu_group, reply_from=sampler_rank)
    enc = msgspec.msgpack.Encoder()
    dec = msgspec.msgpack.Decoder(ControlCommand)
    while True:
        cmd = dec.decode(channel.broadcast(None, src=0))
        if cmd.op == "shutdown":
            channel.close()
            return
        if cmd.op == "reset_kv":
            worker.reset_kv(cmd.prefix_backend)
            continue
        if cmd.op == "device_time":
            worker.device_time_ms(cmd.args[0], cmd.args[1])
            continue
        if cmd.op != "execute":
            raise ValueError(f"unknown control op: {cmd.op}")
        counts = worker.execute_model(cmd.sched)
        if worker.rank != sampler_rank:
            continue
        n_p, n_d = counts
        p_ids, d_ids = worker.read_samples(n_p, n_d)
        channel.send(enc.encode([[n_p, n_d], p_ids, d_ids]), dst=0)   # one message, not two


class UniprocExecutor(Executor):
    def __init__(self, config: EngineConfig, device=None, dtype=None) -> None:
        super().__init__(config, device, dtype)
        from ..runtime.worker import Worker

        self.worker = Worker(config, rank=0, tp_rank=0, pp_rank=0)
        self.worker.init_environment()
        self._ready = False

    def init_kv(self) -> KVManager:
        if not self._ready:
            self.worker.initialize()
            self._ready = True
        self.kv = self._kv_manager(self.worker.get_kv_cache_size())
        return self.kv

    def reset_kv(self, prefix_backend: str | None = None) -> KVManager:
        if prefix_backend is not None:
            self.config.prefix_backend = prefix_backend
        self.worker.reset_kv(prefix_backend)
        self.kv = self._kv_manager(self.worker.get_kv_cache_size())
        return self.kv

    def run(self, sched: ScheduledBatch) -> tuple[int, int]:
        return self.worker.execute_model(sched.to_wire())

    def read_samples(self, n_p: int, n_d: int):
        return self.worker.read_samples(n_p, n_d)

    def collective_rpc(self, op: str, **payload) -> object:
        if op == "reset_kv":
            self.worker.reset_kv(payload.get("prefix_backend"))
            return None
        return super().collective_rpc(op, **payload)

    def device_time_ms(self, lo: int, hi: int) -> float:
        return self.worker.device_time_ms(lo, hi)

    def destroy(self) -> None:
        self.kv = None
        self.worker.destroy_environment()


class MultiprocExecutor(Executor):
    """``worker=None``: spawn ranks 1.. and build rank 0 here (``run.py`` path).
    ``worker=<initialised Worker>``: processes were started externally (torchrun path)."""

    def __init__(self, config: EngineConfig, device=None, dtype=None, worker=None) -> None:
        super().__init__(config, device, dtype)
        self._enc = msgspec.msgpack.Encoder()
        self._dec_reply = msgspec.msgpack.Decoder(list[list[int]])
        self._procs: list = []
        self._owns_workers = worker is None
        self._pending_reply = None
        if worker is None:
            worker = self._spawn_world()
        self.worker = worker
        self.num_blocks = worker.get_kv_cache_size()
        self._channel = ControlChannel(get_world_group().cpu_group, reply_from=self.sampler_rank)

    def _spawn_world(self):
        import torch.distributed as dist

        from ..runtime.worker import Worker

        driver = None
        tag = f"{os.getpid()}_{id(self) & 0xFFFF}"
        os.environ["XV_RDV_TAG"] = tag
        try:
            ctx = mp.get_context("spawn")
            tp, pp = self.config.tp_size, self.config.pp_size
            for rank in range(1, tp * pp):
                p = ctx.Process(target=_spawn_worker, args=(self.config, rank, rank % tp, rank // tp, tag),
                                daemon=False)
                p.start()
                self._procs.append(p)
            driver = Worker(self.config, rank=0, tp_rank=0, pp_rank=0)
            driver.init_environment()
            driver.initialize()
            dist.barrier(group=get_world_group().cpu_group)
            return driver
        except BaseException:
            _terminate_procs(self._procs)
            if driver is not None:
                try:
                    driver.destroy_environment()
                except Exception:
                    pass
            raise

    def init_kv(self) -> KVManager:
        self.kv = self._kv_manager(self.num_blocks)
        return self.kv

    def reset_kv(self, prefix_backend: str | None = None) -> KVManager:
        if prefix_backend is not None:
            self.config.prefix_backend = prefix_backend
        self.collective_rpc("reset_kv", prefix_backend=prefix_backend)
        self.worker.reset_kv(prefix_backend)
        self.num_blocks = self.worker.get_kv_cache_size()
        self.kv = self._kv_manager(self.num_blocks)
        return self.kv

    def collective_rpc(self, op: str, **payload) -> object:
        cmd = ControlCommand(op=op, sched=payload.get("sched"), prefix_backend=payload.get("prefix_backend"),
                             args=list(payload.get("args", [])))
        self._channel.broadcast(self._enc.encode(cmd), src=0)
        return None

    def _check_children(self) -> None:
        for p in self._procs:
            if not p.is_alive():
                raise RuntimeError(f"worker process {p.pid} exited with code {p.exitcode}")

    def run(self, sched: ScheduledBatch) -> tuple[int, int]:
        self._check_children()
        wire = sched.to_wire()
        self.collective_rpc("execute", sched=wire)
        counts = self.worker.execute_model(wire)
        if self.sampler_rank == 0:
            return counts
        reply = self._dec_reply.decode(self._channel.recv(self.sampler_rank))
        self._pending_reply = reply
        return reply[0][0], reply[0][1]

    def read_samples(self, n_p: int, n_d: int):
        if self.sampler_rank == 0:
            return self.worker.read_samples(n_p, n_d)
        reply, self._pending_reply = self._pending_reply, None
        return reply[1], reply[2]

    def device_time_ms(self, lo: int, hi: int) -> float:
        self.collective_rpc("device_time", args=[lo, hi])
        return self.worker.device_time_ms(lo, hi)

    def shutdown(self) -> None:
        self.collective_rpc("shutdown")

    def destroy(self) -> None:
        if self._owns_workers:
            try:
                self.shutdown()
            except Exception:
                pass
            for p in self._procs:
                p.join(timeout=10)
            _terminate_procs(self._procs)
            self._channel.close()
            self.worker.destroy_environment()
        else:
            self._channel.close()      # ranks started externally: only the shared-memory ring is ours to drop
        self.kv = None


def create_executor(config: EngineConfig, device=None, dtype=None, *, rank0_worker=None) -> Executor:
    if config.tp_size == 1 and config.pp_size == 1:
        return UniprocExecutor(config, device, dtype)
    return MultiprocExecutor(config, device, dtype, worker=rank0_worker)
