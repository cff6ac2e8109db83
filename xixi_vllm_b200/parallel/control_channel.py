"""Length-prefixed byte messages over a gloo group (reference:
src/distributed/control_channel.py:22-55). Tensors travel on NCCL; scheduling messages and
sampled ids travel here so control traffic never queues behind GPU work.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

__all__ = ["ControlChannel"]


class ControlChannel:
    def __init__(self, cpu_group) -> None:
        self.group = cpu_group

    def broadcast(self, payload: bytes | None, src: int = 0) -> bytes:
        """``src`` passes bytes, the others pass None; everyone returns the payload."""
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
        dist.send(torch.tensor([len(payload)], dtype=torch.int64), dst=dst, group=self.group)
        if payload:
            dist.send(torch.frombuffer(bytearray(payload), dtype=torch.uint8), dst=dst, group=self.group)

    def recv(self, src: int) -> bytes:
        n = torch.zeros(1, dtype=torch.int64)
        dist.recv(n, src=src, group=self.group)
        size = int(n.item())
        if not size:
            return b""
        buf = torch.empty(size, dtype=torch.uint8)
        dist.recv(buf, src=src, group=self.group)
        return bytes(buf.numpy())
