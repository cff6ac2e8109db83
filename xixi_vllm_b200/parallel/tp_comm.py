"""Tensor-parallel reduction points of the decoder, behind one small interface so the model
code is identical for the library path (NCCL / gloo all-reduce followed by separate ops)
and the fused path (one kernel that exchanges partials over NVLink peer memory, adds the
residual and normalises; see ``parallel/symm.py``).

In the reference these are an NCCL all-reduce inside ``RowParallelLinear.forward`` followed
by a separate fused add+RMSNorm kernel (reference: src/compute/layers/linear.py:141-154,
src/compute/layers/layernorm.py:16-20).
"""

from __future__ import annotations

import torch

from ..ops import dispatch as ops
from . import collectives as coll
from .groups import Group

__all__ = ["TPComm", "LibraryTPComm", "make_tp_comm"]


class TPComm:
    group: Group

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def begin_forward(self) -> None:
        """Called once at the start of every model forward."""

    def alloc_partial(self, tokens: int, final: bool = False) -> torch.Tensor | None:
        """Where the producer of the next partial should write (None = allocate normally).
        ``final`` marks the last reduction of a forward."""
        return None

    def row_linear(self, proj, x: torch.Tensor, final: bool = False):
        """Runs (or defers) a RowParallelLinear whose output goes to the next reduction point."""
        return proj(x, reduce=False, out=self.alloc_partial(x.shape[0], final), defer=True)

    def reduce_add_rmsnorm(self, partial: torch.Tensor, residual: torch.Tensor | None,
                           w: torch.Tensor, eps: float):
        """Sum ``partial`` over the TP group, add it to ``residual`` (or start the residual
        stream when it is None), and return ``(rmsnorm(residual) * w, residual)``."""
        raise NotImplementedError


class LibraryTPComm(TPComm):
    def __init__(self, group: Group) -> None:
        self.group = group

    def all_reduce(self, x):
        if not isinstance(x, torch.Tensor):
            x = x.materialize()
        return coll.all_reduce(x, self.group)

    def reduce_add_rmsnorm(self, partial, residual, w, eps):
        if not isinstance(partial, torch.Tensor):
            # unreduced split-K planes from the GEMM: with one rank the add+norm kernel sums them
            if self.group.size == 1 and residual is not None:
                return ops.add_rmsnorm(partial, residual, w, eps), residual
            partial = partial.materialize()
        x = coll.all_reduce(partial, self.group)
        if residual is None:
            return ops.rmsnorm(x, w, eps), x
        return ops.add_rmsnorm(x, residual, w, eps), residual


def make_tp_comm(group: Group, mode: str, device, hidden_size: int, max_tokens: int, dtype,
                 logits_rows: int = 0, logits_local_cols: int = 0) -> TPComm:
    """``mode``: "nccl" forces the library path; "fused" requires the peer-memory kernels;
    "auto" uses them when running on GPUs with more than one rank. ``logits_rows`` x
    ``logits_local_cols`` sizes the symmetric matrix in which the fused path gathers full logits
    for sampled requests (0 = that gather stays on the library collective)."""
    if group.size == 1 or mode == "nccl" or torch.device(device).type != "cuda":
        return LibraryTPComm(group)
    try:
        from .symm import FusedTPComm

        return FusedTPComm(group, device, hidden_size, max_tokens, dtype, logits_rows, logits_local_cols)
    except Exception:
        if mode == "fused":
            raise
        import logging

        logging.getLogger(__name__).exception("fused TP path unavailable; using NCCL")
        return LibraryTPComm(group)
