"""Tensor collectives over a ``Group`` (reference: src/distributed/communication_op.py:21-130).

These are the library (NCCL / gloo) forms. On GPUs the tensor-parallel hot paths use the
fused kernels in ``parallel/symm.py`` instead; the functions here serve pipeline p2p, CPU
runs, start-up, and as the baseline the fused kernels are checked against.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .groups import Group, get_pp_group, get_tp_group

__all__ = [
    "all_reduce", "all_gather", "reduce_scatter", "send_tensors", "recv_tensors",
    "tensor_model_parallel_all_reduce", "tensor_model_parallel_all_gather",
    "tensor_model_parallel_reduce_scatter",
]


def all_reduce(x: torch.Tensor, group: Group) -> torch.Tensor:
    """In-place sum over the group."""
    if group.size > 1:
        dist.all_reduce(x, group=group.device_group)
    return x


def all_gather(x: torch.Tensor, group: Group, dim: int = -1) -> torch.Tensor:
    """Concatenate every rank's ``x`` along ``dim``."""
    n = group.size
    if n == 1:
        return x
    dim = dim % x.dim()
    x = x.contiguous()
    flat = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(flat, x, group=group.device_group)
    out = flat.view((n,) + tuple(x.shape))
    if dim == 0:
        return out.reshape((n * x.shape[0],) + tuple(x.shape[1:]))
    out = out.movedim(0, dim)
    shape = list(x.shape)
    shape[dim] *= n
    return out.reshape(shape)


def reduce_scatter(x: torch.Tensor, group: Group, dim: int = 0) -> torch.Tensor:
    """Sum over the group, each rank keeping its ``1/size`` slice along ``dim``."""
    n = group.size
    if n == 1:
        return x
    dim = dim % x.dim()
    if x.shape[dim] % n:
        raise ValueError(f"dim {dim} of size {x.shape[dim]} not divisible by {n}")
    xt = x.movedim(dim, 0).contiguous()
    out = torch.empty((xt.shape[0] // n,) + tuple(xt.shape[1:]), dtype=x.dtype, device=x.device)
    if dist.get_backend(group.device_group) == "gloo":
        # gloo has no reduce_scatter: reduce then slice
        full = xt.clone()
        dist.all_reduce(full, group=group.device_group)
        out.copy_(full.chunk(n, 0)[group.group_rank])
    else:
        dist.reduce_scatter_tensor(out, xt, group=group.device_group)
    return out.movedim(0, dim)


def tensor_model_parallel_all_reduce(x: torch.Tensor) -> torch.Tensor:
    return all_reduce(x, get_tp_group())


def tensor_model_parallel_all_gather(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    return all_gather(x, get_tp_group(), dim)


def tensor_model_parallel_reduce_scatter(x: torch.Tensor, dim: int = 0) -> torch.Tensor:
    return reduce_scatter(x, get_tp_group(), dim)


def send_tensors(tensors: list[torch.Tensor], dst: int | None = None, group: Group | None = None):
    """Batched non-blocking sends to the next pipeline stage; returns the work handles."""
    group = group or get_pp_group()
    dst = group.next_rank if dst is None else dst
    ops = [dist.P2POp(dist.isend, t.contiguous(), dst, group=group.device_group) for t in tensors]
    return dist.batch_isend_irecv(ops) if ops else []


def recv_tensors(tensors: list[torch.Tensor], src: int | None = None, group: Group | None = None,
                 wait: bool = True):
    """Batched receives into preallocated tensors from the previous pipeline stage."""
    group = group or get_pp_group()
    src = group.prev_rank if src is None else src
    ops = [dist.P2POp(dist.irecv, t, src, group=group.device_group) for t in tensors]
    works = dist.batch_isend_irecv(ops) if ops else []
    if wait:
        for w in works:
            w.wait()
    return works
