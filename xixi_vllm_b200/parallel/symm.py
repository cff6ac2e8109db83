"""Symmetric peer-memory buffers and the fused tensor-parallel reduction path.

Each rank allocates the same buffer through PyTorch's symmetric-memory allocator (CUDA VMM
allocations whose handles are exchanged over the process group), which yields every peer's
mapping of the buffer and, on NVSwitch systems, a multicast address. The hand-written
kernels in ``csrc/kernels/tp_fused.cu`` read peers' partial results straight from those
mappings (or let the switch add them with ``multimem.ld_reduce``) and finish with the
residual add and RMSNorm, so the decoder issues no NCCL call and no separate add+norm kernel.
The reference does an NCCL all-reduce followed by a FlashInfer fused add+norm kernel at
each of these points (reference: src/compute/layers/linear.py:141-154).

Buffer rotation: a forward's reductions use buffers A, B, A, B, ... and the last one uses C,
so no buffer is written for two consecutive reductions, also across forwards and across
CUDA-graph replays (see the reuse rule in tp_fused.cu).

Environment: ``XV_TP_NVLS=0`` disables the multicast path (plain peer loads are used).
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import cuda
from .groups import Group
from .tp_comm import TPComm

__all__ = ["SymmetricBuffer", "FusedTPComm", "DeferredRowGemm"]


class DeferredRowGemm:
    """A row-parallel projection whose GEMM has not run yet: the communicator launches it
    together with the reduction that consumes it (one kernel)."""

    __slots__ = ("x", "weight", "final")

    def __init__(self, x: torch.Tensor, weight: torch.Tensor, final: bool) -> None:
        self.x, self.weight, self.final = x, weight, final

    @property
    def shape(self):
        return (self.x.shape[0], self.weight.shape[0])

FLAG_BYTES = 4096          # epoch flags (three channels x 8 ranks) and the push protocol's arrival counters
SPIN_LIMIT = 2_000_000     # microseconds a kernel waits for a peer before it reports and returns


class SymmetricBuffer:
    """A byte buffer that exists on every rank of ``group`` and is mapped on all of them."""

    def __init__(self, nbytes: int, group: Group, device: torch.device) -> None:
        import torch.distributed._symmetric_memory as symm

        self.group, self.device, self.nbytes = group, device, nbytes
        self.local = symm.empty(nbytes, dtype=torch.uint8, device=device)
        self.local.zero_()
        torch.cuda.synchronize(device)
        self.handle = symm.rendezvous(self.local, group.device_group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.rank, self.world = int(self.handle.rank), int(self.handle.world_size)
        use_mc = os.environ.get("XV_TP_NVLS", "1") != "0"
        self.multicast_ptr = int(self.handle.multicast_ptr) if (use_mc and self.handle.has_multicast_support) else 0
        dist.barrier(group=group.cpu_group)      # every rank has zeroed and mapped before first use

    def ptr_array(self, offset: int = 0):
        return (ctypes.c_void_p * self.world)(*[p + offset for p in self.ptrs])


class FusedTPComm(TPComm):
    def __init__(self, group: Group, device, hidden_size: int, max_tokens: int, dtype,
                 logits_rows: int = 0, logits_local_cols: int = 0) -> None:
        if dtype != torch.bfloat16:
            raise TypeError("the fused tensor-parallel path runs bfloat16")
        self.group = group
        self.device = torch.device(device)
        self.hidden = hidden_size
        self.max_tokens = max_tokens
        # room for the push protocol's slot array: world sources x ceil(tokens / world) rows
        self.buf_bytes = -(-(max_tokens + group.size) * hidden_size * 2 // 4096) * 4096
        self.slot_bytes = -(-group.size * max_tokens * 8 // 4096) * 4096
        # optional [logits_rows, world * logits_local_cols] matrix for gathering sampled rows' logits
        self._logit_rows, self._logit_cols = logits_rows, logits_local_cols * group.size
        logit_bytes = -(-logits_rows * self._logit_cols * 2 // 4096) * 4096
        self.logits_off = 4 * self.buf_bytes + self.slot_bytes + FLAG_BYTES
        # exchange region of the sharded sampler (row maxima, selection histograms, candidates): XV_TP_SAMPLE=0
        # samples from the gathered logits instead
        self.sample_rows = logits_rows if os.environ.get("XV_TP_SAMPLE", "1") != "0" else 0
        self.sample_off = self.logits_off + logit_bytes
        total = self.sample_off + (cuda.tp_sample_region_bytes(self.sample_rows, group.size) if self.sample_rows else 0)
        self.symm = SymmetricBuffer(total, group, self.device)
        self.rank, self.world = self.symm.rank, self.symm.world
        self.h_off = 3 * self.buf_bytes              # activation buffer the row-sharded reductions broadcast into
        self.slots_off = 4 * self.buf_bytes
        self.flags_off = 4 * self.buf_bytes + self.slot_bytes
        # The native forward uses the row-sharded (two-shot) reduction from 4 ranks up: its traffic per GPU
        # does not grow with the rank count, at the price of a second barrier (measured slower at 2 ranks).
        # XV_TP_SHARDED=0/1 forces the choice.
        env = os.environ.get("XV_TP_SHARDED", "")
        self.sharded_reduce = (env == "1") if env in ("0", "1") else group.size >= 4
        self._bufs = self.symm.ptr_array(0)
        self._flags = self.symm.ptr_array(self.flags_off)
        self.mc_ptr = self.symm.multicast_ptr
        self.epoch = torch.zeros(32, dtype=torch.int32, device=self.device)   # [0] epoch, the rest: counter history
        self.epoch[0] = 1
        self.status = cuda.device_status(self.epoch)
        # The row-parallel GEMM and its reduction can run as ONE kernel (tiles pushed from the GEMM epilogue into
        # the reducing ranks' slots, XV_TP_PUSH=1). It is off by default: at 2 and 4 ranks the GEMM followed by
        # the reduction kernel that pulls measured faster at every batch size (the pushing GEMM keeps few CTAs
        # busy and pays a system-scope release per tile). This module-by-module path (tests, stages driven from
        # Python) reduces every row on every rank, which costs NVLink traffic proportional to the rank count,
        # so with XV_TP_PUSH=1 it is used up to XV_TP_FUSE_GEMM_MAX_T tokens.
        self.fuse_gemm = os.environ.get("XV_TP_PUSH", "0") == "1"
        self.fuse_gemm_max_tokens = int(os.environ.get("XV_TP_FUSE_GEMM_MAX_T", "256"))
        # native executor: forwards of at most push_max_tokens run the one-kernel projection, of those the ones
        # of at most one_shot_max_tokens in the form where every rank reduces every row
        self.push_max_tokens = int(os.environ.get("XV_TP_PUSH_MAX_T", "256"))
        # all-gather -> GEMM: after a two-shot one-kernel projection the GEMM that reads the activation waits for
        # the rows the other ranks broadcast (in its TMA producer), instead of the projection kernel itself
        self.defer_row_wait = os.environ.get("XV_TP_DEFER_ROW_WAIT", "1") != "0"
        # the same hand-over after the row-sharded reduction kernel (the kernel ends once its own rows are
        # broadcast). Token-equal on 2 GPUs, no time gained there and not timed on more ranks: opt-in.
        self.pull_defer_row_wait = os.environ.get("XV_TP_PULL_DEFER", "0") == "1"
        self.one_shot_max_tokens = int(os.environ.get("XV_TP_ONE_SHOT_MAX_T", "64"))
        self._idx = 0
        self._logits_view = None
        if logit_bytes:
            self._logit_bufs = self.symm.ptr_array(self.logits_off)
            self._logit_mc = self.mc_ptr + self.logits_off if self.mc_ptr else 0
            n = logits_rows * self._logit_cols * 2
            self._logits_view = self.symm.local[self.logits_off:self.logits_off + n].view(torch.bfloat16).view(
                logits_rows, self._logit_cols)
        self._base = self.symm.local.data_ptr()
        self._views = [self.symm.local[i * self.buf_bytes:(i + 1) * self.buf_bytes].view(torch.bfloat16)
                       for i in range(3)]
        self.h_view = self.symm.local[self.h_off: self.h_off + self.buf_bytes].view(torch.bfloat16)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group.cpu_group)
        if self.rank == 0:
            print(f"[tp] fused peer-memory reductions: world={self.world} "
                  f"nvls_multicast={'yes' if self.mc_ptr else 'no'}", flush=True)

    # --- buffer rotation ------------------------------------------------------------------
    def begin_forward(self) -> None:
        self._idx = 0

    def alloc_partial(self, tokens: int, final: bool = False) -> torch.Tensor:
        if tokens > self.max_tokens:
            raise RuntimeError(f"{tokens} tokens exceed the symmetric buffer ({self.max_tokens})")
        which = 2 if final else self._idx % 2
        self._idx += 1
        return self._views[which][: tokens * self.hidden].view(tokens, self.hidden)

    def _offset_of(self, partial: torch.Tensor) -> int:
        off = partial.data_ptr() - self._base
        if 0 <= off < 3 * self.buf_bytes and partial.is_contiguous():
            return off
        # produced elsewhere: stage it through the next buffer
        buf = self.alloc_partial(partial.shape[0])
        buf.copy_(partial)
        return buf.data_ptr() - self._base

    def row_linear(self, proj, x: torch.Tensor, final: bool = False):
        """Output of a RowParallelLinear as something ``reduce_add_rmsnorm`` / ``all_reduce`` accept."""
        T = x.shape[0]
        if (self.fuse_gemm and proj.bias is None and 0 < T <= self.fuse_gemm_max_tokens and self.hidden <= 6144
                and self.world * T * self.hidden * 2 <= self.buf_bytes):
            return DeferredRowGemm(x, proj.weight, final)
        return proj(x, reduce=False, out=self.alloc_partial(x.shape[0], final))

    def _fused(self, d: DeferredRowGemm, residual, w, eps, mode):
        T = d.x.shape[0]
        buf = self.alloc_partial(T, d.final)
        off = buf.data_ptr() - self._base
        y = torch.empty((T, self.hidden), dtype=torch.bfloat16, device=self.device)
        res_out = None
        if mode == 0:
            res_out = residual if residual is not None else torch.empty_like(y)
        cuda.gemm_tp_fused(d.x, d.weight, self._bufs, self._flags, self.mc_ptr, self.epoch, self.rank, self.world,
                           off, self.buf_bytes, False, 0, residual, res_out, w, y, eps, mode, SPIN_LIMIT)
        return y, res_out

    def gemm_reduce_norm(self, x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor | None,
                         w: torch.Tensor | None, eps: float, *, two_shot: bool, final: bool = False,
                         first: bool = False, mode: int = 0, defer_row_wait: bool = False):
        """Row-parallel projection, cross-rank sum, residual add and RMSNorm as one kernel.

        ``two_shot``: rank r reduces rows r, r + world, ...; ``residual`` is a local [T, H] buffer of which
        only those rows are read and written (``first`` starts the stream instead of adding), and the
        result is the view of the symmetric activation buffer every rank's rows were broadcast into.
        Otherwise every rank reduces all rows and gets a fresh [T, H] tensor.
        ``defer_row_wait`` (two-shot): the kernel ends without waiting for the other ranks' rows; the caller
        must run ``await_rows()`` right before the GEMM that reads ``y``.
        Returns ``(y, residual)``."""
        T = x.shape[0]
        buf = self.alloc_partial(T, final)
        off = buf.data_ptr() - self._base
        if two_shot:
            y = self.h_view[: T * self.hidden].view(T, self.hidden)
        else:
            y = torch.empty((T, self.hidden), dtype=torch.bfloat16, device=self.device)
        res_out = None
        if mode == 0:
            res_out = residual if residual is not None else torch.empty((T, self.hidden), dtype=torch.bfloat16,
                                                                        device=self.device)
        cuda.gemm_tp_fused(x, weight, self._bufs, self._flags, self.mc_ptr, self.epoch, self.rank, self.world,
                           off, self.buf_bytes, two_shot, self.h_off, None if first else residual, res_out, w,
                           None if two_shot else y, eps, mode, SPIN_LIMIT, defer_row_wait=defer_row_wait)
        return y, res_out

    def await_rows(self) -> None:
        """The next GEMM launched from this thread waits (in its loader) for the rows that the last two-shot
        projection with ``defer_row_wait`` has the other ranks broadcast."""
        L = cuda.lib()
        L.xv_gemm_wait_for_rows.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_uint]
        L.xv_gemm_wait_for_rows.restype = None
        flags = self.symm.ptrs[self.rank] + self.flags_off + 4 * L.xv_tp_bcast_word()
        targets = self.epoch.data_ptr() + 4 * L.xv_tp_bcast_base_word()
        L.xv_gemm_wait_for_rows(flags, targets, self.world, SPIN_LIMIT)

    # --- reductions -----------------------------------------------------------------------------
    def reduce_add_rmsnorm(self, partial, residual, w, eps):
        if isinstance(partial, DeferredRowGemm):
            return self._fused(partial, residual, w, eps, 0)
        T = partial.shape[0]
        off = self._offset_of(partial)
        y = torch.empty((T, self.hidden), dtype=torch.bfloat16, device=self.device)
        res_out = residual if residual is not None else torch.empty_like(y)
        cuda.tp_reduce_norm(self._bufs, self._flags, self.mc_ptr, self.epoch, self.rank, self.world, off,
                            residual, res_out, w, y, T, self.hidden, eps, 0, SPIN_LIMIT, self.status)
        return y, res_out

    def all_reduce(self, x):
        if isinstance(x, DeferredRowGemm):
            return self._fused(x, None, None, 0.0, 1)[0]
        T = x.shape[0]
        off = self._offset_of(x)
        y = torch.empty((T, self.hidden), dtype=torch.bfloat16, device=self.device)
        cuda.tp_reduce_norm(self._bufs, self._flags, self.mc_ptr, self.epoch, self.rank, self.world, off,
                            None, None, None, y, T, self.hidden, 0.0, 1, SPIN_LIMIT, self.status)
        return y

    def argmax(self, local_logits: torch.Tensor, valid_vocab: int, vocab_start: int) -> torch.Tensor:
        rows = local_logits.shape[0]
        out = torch.empty(rows, dtype=torch.int64, device=self.device)
        cuda.tp_argmax(self._bufs, self._flags, self.epoch, self.rank, self.world, self.slots_off, local_logits,
                       local_logits.shape[1], valid_vocab, vocab_start, out, SPIN_LIMIT, self.status)
        return out

    def sample(self, local_logits: torch.Tensor, valid_vocab: int, vocab_start: int, total_vocab: int,
               temperature, top_k, top_p, min_p, rng) -> torch.Tensor | None:
        """Tokens drawn from the vocabulary-sharded logits without gathering them, the same on every rank; None
        when no exchange region was reserved for this many rows (the caller gathers the logits instead)."""
        if local_logits.shape[0] > self.sample_rows:
            return None
        return cuda.tp_sample(self._bufs, self._flags, self.epoch, self.rank, self.world, self.sample_off,
                              self.sample_rows, local_logits, valid_vocab, vocab_start, total_vocab, temperature,
                              top_k, top_p, min_p, rng, SPIN_LIMIT, self.status)

    # --- full logits for sampled requests ------------------------------------------------------
    def gather_logits(self, local_logits: torch.Tensor) -> torch.Tensor | None:
        """All ranks' vocabulary shards side by side, or None when no matching matrix was reserved
        (the caller then uses the library collective). The result aliases the symmetric buffer and
        stays valid until the next call."""
        rows, cols = local_logits.shape
        if self._logits_view is None or rows > self._logit_rows or cols * self.world != self._logit_cols:
            return None
        cuda.tp_allgather_cols(self._logit_bufs, self._flags, self._logit_mc, self.epoch, self.rank, self.world,
                               local_logits, self._logit_cols, SPIN_LIMIT, self.status)
        return self._logits_view[:rows]

    def destroy(self) -> None:
        self._views = []
        self._logits_view = None
        self.symm = None
