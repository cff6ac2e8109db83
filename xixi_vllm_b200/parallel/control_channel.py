"""Control messages between the driver (rank 0) and the worker ranks.

Tensors travel on NCCL; scheduling messages and sampled ids travel here so control traffic never
queues behind GPU work. Point-to-point messages and the fallback broadcast are length-prefixed
bytes over a gloo group (reference: src/distributed/control_channel.py:22-55).

The per-step broadcast of the scheduler's output is on the critical path of every step (the GPUs
idle until the workers have it), and two gloo collectives cost 0.3-0.6 ms for 2-8 local ranks. When
all ranks share a host the broadcast therefore goes through a single-writer ring in shared memory
(a file under /dev/shm mapped by every rank): the driver copies the bytes into the next slot and
publishes a sequence number, the workers poll for it (busy first, then yielding, then sleeping, so
idle engines cost next to nothing) and acknowledge, which is what lets the driver reuse slots.
The rank that answers the driver every step (the sampler rank of a pipeline) gets a second ring of its
own towards rank 0. Messages larger than a slot, other point-to-point pairs, hosts without /dev/shm
and multi-node groups use the gloo path.
``XV_CTL_SHM=0`` disables the ring.
"""

from __future__ import annotations

import atexit
import mmap
import os
import socket
import struct
import threading
import time

import torch
import torch.distributed as dist

__all__ = ["ControlChannel"]

_SLOTS = 8
_SLOT_BYTES = 1 << 20              # payload capacity of a slot
_HDR = 16                          # per slot: sequence number, payload length
_ACK_OFF = 64                      # acknowledgements, one cache line per rank
_VIA_GLOO = (1 << 63)              # length marker: this message follows on the gloo path


class _ShmRing:
    """Single-writer, many-reader message ring in a shared mapping."""

    def __init__(self, path: str, world: int, rank: int, create: bool, writer: int = 0,
                 readers: list[int] | None = None) -> None:
        self.path, self.world, self.rank, self.owner = path, world, rank, create
        self.writer = writer
        self.readers = readers if readers is not None else [r for r in range(world) if r != writer]
        self.slots_off = _ACK_OFF + 64 * world
        size = self.slots_off + _SLOTS * (_HDR + _SLOT_BYTES)
        flags = os.O_RDWR | (os.O_CREAT | os.O_EXCL if create else 0)
        fd = os.open(path, flags, 0o600)
        try:
            if create:
                os.ftruncate(fd, size)
            self.map = mmap.mmap(fd, size)
        finally:
            os.close(fd)
        self.q = memoryview(self.map).cast("Q")          # 8-byte cells: headers and acknowledgements
        self.seq = 0                                     # last message written (driver) / read (worker)
        self._fence = threading.Lock()
        if create:
            atexit.register(self._unlink)            # a driver that exits without close() leaves no file behind
        if rank == writer:
            struct.pack_into("<Q", self.map, 0, os.getpid())          # lets readers notice a dead writer
        elif rank in self.readers:
            self.q[(_ACK_OFF + 64 * rank) // 8 + 1] = os.getpid()     # lets the writer notice a dead reader

    def _barrier(self) -> None:
        # a lock round trip orders this thread's earlier stores before its later ones on any CPU
        self._fence.acquire()
        self._fence.release()

    def _slot(self, seq: int) -> int:
        return self.slots_off + (seq % _SLOTS) * (_HDR + _SLOT_BYTES)

    def writer_pid(self) -> int:
        return struct.unpack_from("<Q", self.map, 0)[0]

    # --- driver ------------------------------------------------------------------------------
    def write(self, payload: bytes | None, marker: int = 0) -> None:
        seq = self.seq + 1
        if seq > _SLOTS:        # the slot's previous message must have been read by every worker
            need = seq - _SLOTS
            spins = 0
            checked = time.monotonic()
            while min(self.q[(_ACK_OFF + 64 * r) // 8] for r in self.readers) < need:
                spins += 1
                if spins > 2000:
                    time.sleep(0.0001)
                    if time.monotonic() - checked > 1.0:
                        checked = time.monotonic()
                        self._check_readers(need)
        off = self._slot(seq)
        if payload is not None:
            self.map[off + _HDR: off + _HDR + len(payload)] = payload
            self.q[(off + 8) // 8] = len(payload)
        else:
            self.q[(off + 8) // 8] = marker
        self._barrier()
        self.q[off // 8] = seq
        self.seq = seq

    def _check_readers(self, need: int) -> None:
        for r in self.readers:
            cell = (_ACK_OFF + 64 * r) // 8
            pid = self.q[cell + 1]
            if self.q[cell] < need and pid:
                try:
                    os.kill(pid, 0)
                except ProcessLookupError:
                    raise RuntimeError(f"rank {r} (pid {pid}) is gone with control messages unread") from None
                except PermissionError:
                    pass

    # --- workers -----------------------------------------------------------------------------
    def read(self) -> tuple[bytes | None, int]:
        """Next message: ``(payload, 0)``, or ``(None, marker)`` for one that follows on the gloo path."""
        seq = self.seq + 1
        off = self._slot(seq)
        cell = off // 8
        # Poll hot while the engine is busy (a step takes 5-30 ms and every rank's launch waits for this
        # message), yield the core between bursts, and back off to short sleeps only when nothing has come
        # for a while, so an idle engine costs next to nothing.
        q = self.q
        t0 = 0.0
        last_check = 0.0
        while q[cell] != seq:
            for _ in range(256):
                if q[cell] == seq:
                    break
            else:
                now = time.monotonic()
                if not t0:
                    t0 = last_check = now
                idle = now - t0
                if idle < 0.05:
                    os.sched_yield()
                elif idle < 2.0:
                    time.sleep(0.0002)
                else:
                    time.sleep(0.001)
                if now - last_check > 1.0:
                    last_check = now
                    pid = self.writer_pid()
                    try:
                        if pid:
                            os.kill(pid, 0)
                    except ProcessLookupError:
                        raise RuntimeError("the sending process is gone; leaving the control loop") from None
                    except PermissionError:
                        pass
        self._barrier()
        n = self.q[cell + 1]
        out = (None, n) if n & _VIA_GLOO else (bytes(self.map[off + _HDR: off + _HDR + n]), 0)
        self.seq = seq
        self.q[(_ACK_OFF + 64 * self.rank) // 8] = seq
        return out

    def close(self) -> None:
        try:
            self.q.release()
            self.map.close()
        except (BufferError, ValueError):
            pass
        if self.owner:
            self._unlink()

    def _unlink(self) -> None:
        try:
            os.unlink(self.path)
        except OSError:
            pass


class ControlChannel:
    def __init__(self, cpu_group, shm: bool | None = None, reply_from: int = 0) -> None:
        """Collective when shared memory is enabled: every rank of the group constructs its channel at
        the same point (the driver after its workers are up, the workers when they enter their loop).
        ``reply_from``: the rank whose ``send(..., dst=0)`` answers the driver every step (the sampler rank
        of a pipeline); it gets a ring of its own towards rank 0. 0 = no such rank."""
        self.group = cpu_group
        self.reply_from = reply_from
        self._ring: _ShmRing | None = None
        self._reply: _ShmRing | None = None
        if shm is None:
            shm = os.environ.get("XV_CTL_SHM", "1") != "0"
        world = dist.get_world_size(group=cpu_group)
        if shm and world > 1:
            self._setup_ring(world)

    def _setup_ring(self, world: int) -> None:
        me = dist.get_rank(group=self.group)
        info = [None]
        ring = reply = None
        rf = self.reply_from if 0 < self.reply_from < world else 0
        if me == 0:
            path = f"/dev/shm/xv_ctl_{os.getpid()}_{int(time.time() * 1e6) & 0xFFFFFFFF:x}"
            try:
                ring = _ShmRing(path, world, 0, create=True)
                if rf:
                    reply = _ShmRing(path + "_r", world, 0, create=True, writer=rf, readers=[0])
                info = [(path, socket.gethostname())]
            except OSError:
                if ring is not None:
                    ring.close()
                    ring = None
                info = [None]
        dist.broadcast_object_list(info, src=dist.get_global_rank(self.group, 0), group=self.group)
        ok = 1
        if info[0] is None:
            ok = 0
        elif me != 0:
            path, host = info[0]
            try:
                if host != socket.gethostname():
                    raise OSError("different host")
                ring = _ShmRing(path, world, me, create=False)
                if rf and me == rf:
                    reply = _ShmRing(path + "_r", world, me, create=False, writer=rf, readers=[0])
            except OSError:
                ok = 0
        flag = torch.tensor([ok], dtype=torch.int64)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 1:
            self._ring, self._reply = ring, reply
        else:
            for r in (ring, reply):
                if r is not None:
                    r.close()

    @property
    def uses_shared_memory(self) -> bool:
        return self._ring is not None

    def broadcast(self, payload: bytes | None, src: int = 0) -> bytes:
        """``src`` passes bytes, the others pass None; everyone returns the payload."""
        if self._ring is not None and src == 0:
            me = dist.get_rank(group=self.group)
            if me == 0:
                assert payload is not None
                if len(payload) <= _SLOT_BYTES:
                    self._ring.write(payload)
                    return payload
                self._ring.write(None, _VIA_GLOO | len(payload))
            else:
                data, marker = self._ring.read()
                if data is not None:
                    return data
        return self._broadcast_gloo(payload, src)

    def _broadcast_gloo(self, payload: bytes | None, src: int) -> bytes:
        me = dist.get_rank()
        if me == src:
            assert payload is not None
            n = torch.tensor([len(payload)], dtype=torch.int64)
        else:
            n = torch.zeros(1, dtype=torch.int64)
        dist.broadcast(n, src=src, group=self.group)
        size = int(n.item())
        if me == src:
            buf = torch.frombuffer(bytearray(payload), dtype=torch.uint8) if size else torch.empty(0, dtype=torch.uint8)
        else:
            buf = torch.empty(size, dtype=torch.uint8)
        if size:
            dist.broadcast(buf, src=src, group=self.group)
        return payload if me == src else bytes(buf.numpy())

    def send(self, payload: bytes, dst: int) -> None:
        if self._reply is not None and dst == 0 and dist.get_rank(group=self.group) == self.reply_from:
            if len(payload) <= _SLOT_BYTES:
                self._reply.write(payload)
                return
            self._reply.write(None, _VIA_GLOO | len(payload))
        dist.send(torch.tensor([len(payload)], dtype=torch.int64), dst=dst, group=self.group)
        if payload:
            dist.send(torch.frombuffer(bytearray(payload), dtype=torch.uint8), dst=dst, group=self.group)

    def recv(self, src: int) -> bytes:
        if self._reply is not None and src == self.reply_from and dist.get_rank(group=self.group) == 0:
            data, _ = self._reply.read()
            if data is not None:
                return data
        n = torch.zeros(1, dtype=torch.int64)
        dist.recv(n, src=src, group=self.group)
        size = int(n.item())
        if not size:
            return b""
        buf = torch.empty(size, dtype=torch.uint8)
        dist.recv(buf, src=src, group=self.group)
        return bytes(buf.numpy())

    def close(self) -> None:
        for ring in (self._ring, self._reply):
            if ring is not None:
                ring.close()
        self._ring = self._reply = None
