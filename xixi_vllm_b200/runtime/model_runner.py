"""Runs one scheduled step on this rank (reference: src/compute/model_runner.py:22-361).

A step is ONE forward over the packed batch (decode rows then prefill chunks). Pure-decode
steps replay a CUDA graph when graphs are enabled. Pipeline hand-off tensors move with NCCL
p2p outside the graphs. Sampled ids leave the device on a side stream into pinned memory;
``read_samples`` is the only point that waits.
"""

from __future__ import annotations

import os
from collections import deque

import torch

from ..ops import dispatch as ops
from ..parallel.collectives import recv_tensors, send_tensors
from ..parallel.groups import get_pp_group, get_tp_group
from ..parallel.pp import IntermediateTensors
from ..utils.nvtx import nvtx_range
from .graphs import CUDAGraphRunner, make_bs_list
from .kv_pool import KVPool
from .sampler import Sampler
from .staging import BatchStager, split_forward_batch

__all__ = ["ModelRunner"]


class ModelRunner:
    def __init__(self, model, kv: KVPool, sampler: Sampler, *, config, device) -> None:
        self.model, self.kv, self.sampler, self.config = model, kv, sampler, config
        self.device = torch.device(device)
        self.is_cuda = self.device.type == "cuda"
        self.block_size = kv.block_size
        self.hidden_size = config.hf_config.hidden_size
        pp, tp = get_pp_group(), get_tp_group()
        self._pp = pp
        self.is_first_pp, self.is_last_pp = pp.is_first_rank, pp.is_last_rank
        self.is_driver = self.is_last_pp and tp.group_rank == 0
        self.max_bs = config.max_num_seqs
        self.max_tokens = max(config.max_num_batched_tokens, self.max_bs)
        self.max_blocks = -(-config.context_len // self.block_size)
        self.pp_microbatches = max(1, int(getattr(config, "pp_microbatches", 1)))
        self.stager = BatchStager(max_seqs=self.max_bs, max_tokens=self.max_tokens,
                                  max_blocks=self.max_blocks, block_size=self.block_size, device=self.device,
                                  seed=getattr(config, "seed", 0))
        self._pp_buf = None
        if not self.is_first_pp:
            shape = (self.max_tokens, self.hidden_size)
            self._pp_buf = (torch.empty(shape, dtype=kv.dtype, device=self.device),
                            torch.empty(shape, dtype=kv.dtype, device=self.device))
        self._copy_stream = torch.cuda.Stream(device=self.device) if self.is_cuda else None
        # Two read-back slots used in turn: with one-step-late scheduling step n + 1 is launched before step n's
        # samples have been read. ``_unread`` lists the launched steps whose samples are still to be read.
        self._sample_events = [torch.cuda.Event() for _ in range(2)] if self.is_cuda else [None, None]
        self._host_samples = [torch.zeros(self.max_bs, dtype=torch.int64, pin_memory=self.is_cuda) for _ in range(2)]
        self._host_statuses = [torch.zeros(1, dtype=torch.int32, pin_memory=self.is_cuda) for _ in range(2)]
        self._slot = 0
        self._unread: deque = deque()
        self._dev_status = None
        if self.is_cuda:
            from ..ops import cuda as _cuda

            self._dev_status = _cuda.device_status(self._host_samples[0].to(self.device))
        self._dev_samples: torch.Tensor | None = None
        self._n_samples = 0
        self._last: tuple[int, int, list[bool]] = (0, 0, [])
        # per-step device time (CUDA events around the forward), kept for the last few thousand steps
        self.time_steps = self.is_cuda and os.environ.get("XV_TIME_STEPS", "0") == "1"
        self._step_events: dict[int, tuple] = {}
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        # GPU models run through the native executor: one C call launches a pipeline stage's whole forward
        self.native = None
        if self.is_cuda and os.environ.get("XV_NATIVE_FORWARD", "1") != "0":
            from .native_forward import NativeForward

            tp = get_tp_group()
            if tp.size == 1 or hasattr(model.comm, "symm"):
                self.native = NativeForward(model, kv, max_tokens=self.max_tokens, max_samples=self.max_bs)
        self.graphs: CUDAGraphRunner | None = None
        if self.is_cuda and not config.enforce_eager:
            self._capture_graphs()

    # --- forward --------------------------------------------------------------------------
    def _forward(self, batch, intermediate=None):
        if self.native is not None:
            out = self.native.forward(batch)      # a stage that is not the first reads what _recv put in the arena
            if not self.is_last_pp:
                return IntermediateTensors(hidden_states=out[0], residual=out[1])
            if batch.all_greedy:
                return out
            return self._sample_local(out, batch)
        out = self.model.forward(batch.input_ids, batch, self.kv, intermediate)
        if not self.is_last_pp:
            return out
        if batch.num_samples == 0:      # only a mid-prompt chunk: the forward wrote its KV, nothing to sample
            return torch.empty(0, dtype=torch.int64, device=self.device)
        hidden = ops.gather_rows(out, batch.sample_rows)
        if batch.all_greedy:
            return self.model.greedy_tokens(hidden)
        head = self.model.lm_head
        if getattr(head, "tp", None) is not None and head.tp.size > 1 and hasattr(self.model.comm, "sample"):
            return self._sample_local(head.local_logits(hidden), batch)
        logits = self.model.compute_logits(hidden)
        return self.sampler(logits, batch.temperature, batch.top_k, batch.top_p, batch.min_p, rng=batch.rng)

    def _sample_local(self, logits, batch):
        """Draws from this rank's logits: under tensor parallelism they are a vocabulary shard, sampled across the
        ranks without gathering it (or gathered first when the communicator has no exchange region for it)."""
        head = self.model.lm_head
        if head.tp.size > 1:
            comm = self.model.comm
            if hasattr(comm, "sample"):
                valid = max(0, min(head.per_rank, head.num_embeddings - head.vocab_start))
                tokens = comm.sample(logits, valid, head.vocab_start, head.num_embeddings, batch.temperature,
                                     batch.top_k, batch.top_p, batch.min_p, batch.rng)
                if tokens is not None:
                    self.sampler.step += 1
                    return tokens
            gathered = self._gather_logits(logits)
            if gathered is None:
                from ..parallel import collectives as coll

                gathered = coll.all_gather(logits, head.tp, dim=-1)
            logits = gathered
        logits = logits[..., : head.num_embeddings]
        return self.sampler(logits, batch.temperature, batch.top_k, batch.top_p, batch.min_p, rng=batch.rng)

    def _gather_logits(self, local_logits):
        comm = self.model.comm
        return comm.gather_logits(local_logits) if hasattr(comm, "gather_logits") else None

    def _recv(self, n_tokens: int) -> IntermediateTensors:
        """Receives the previous stage's hidden states and residual stream for a whole step: straight into
        the native executor's arena when it runs this stage, else into the runner's own pair."""
        if self.native is not None:
            h, r = self.native.stage_inputs(n_tokens)
        else:
            h, r = self._pp_buf[0][:n_tokens], self._pp_buf[1][:n_tokens]
        recv_tensors([h, r], group=self._pp)
        return IntermediateTensors(hidden_states=h, residual=r)

    def _send(self, inter: IntermediateTensors) -> None:
        for w in send_tensors([inter["hidden_states"], inter["residual"]], group=self._pp):
            w.wait()

    def _forward_microbatched(self, batch):
        """Pipeline stages work on several pieces of the step in turn: while this stage computes piece k+1,
        its output for piece k is already on its way and the next stage is computing it. Sends are not waited
        for until every piece has been launched; receives land in disjoint row ranges of the hand-off buffers.
        (The reference runs its stages in lockstep on the whole step.)"""
        pending, pieces = [], []
        for sub, t0, t1 in split_forward_batch(batch, self.pp_microbatches):
            inter = None
            if not self.is_first_pp:
                h, r = self._pp_buf[0][t0:t1], self._pp_buf[1][t0:t1]
                recv_tensors([h, r], group=self._pp)
                inter = IntermediateTensors(hidden_states=h, residual=r)
                if self.native is not None:
                    # the native executor reads a stage's input at the start of its arena; the pieces land in
                    # disjoint rows of the runner's pair so that a receive never waits for the piece before it
                    ah, ar = self.native.stage_inputs(t1 - t0)
                    ah.copy_(h)
                    ar.copy_(r)
            with nvtx_range("forward"):
                out = self._forward(sub, inter)
            if self.native is not None and self.is_last_pp and isinstance(out, torch.Tensor):
                out = out.clone()       # the executor's output buffer is reused by the next piece
            if not self.is_last_pp:
                hs, rs = out["hidden_states"], out["residual"]
                if self.native is not None:
                    hs, rs = hs.clone(), rs.clone()    # the next piece overwrites the arena while this one travels
                pending.extend(send_tensors([hs, rs], group=self._pp))
            elif sub.num_samples:
                pieces.append(out)
        for w in pending:
            w.wait()
        if not self.is_last_pp:
            return None
        return torch.cat(pieces) if len(pieces) != 1 else pieces[0]

    def run_forward(self, sched) -> tuple[int, int]:
        """Launches the step (no host wait). Returns (#prefill sequences, #decode sequences)."""
        n_p, n_d = len(sched.prefills), len(sched.decodes)
        use_graph = self.graphs is not None and n_p == 0 and 0 < n_d <= self.graphs.max_bs
        ev = None
        if self.time_steps:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        with torch.no_grad():
            if use_graph:
                bucket = self.graphs.pad_bs(n_d)
                with nvtx_range("stage"):
                    batch = self.stager.build(sched, pad_to=bucket, fixed_blocks=True)
                    self._resolve_token_refs(batch)
                greedy = batch.all_greedy if self.is_last_pp else True
                if not self.is_first_pp:
                    self._recv(bucket)             # outside the graph, into the buffers the graph reads
                with nvtx_range("decode_graph"):
                    tokens = self.graphs.replay(bucket, greedy)
                if not self.is_last_pp:
                    self._send(tokens)
                    tokens = None
            else:
                with nvtx_range("stage"):
                    batch = self.stager.build(sched)
                    self._resolve_token_refs(batch)
                if self.pp_microbatches > 1 and not (self.is_first_pp and self.is_last_pp):
                    tokens = self._forward_microbatched(batch)
                else:
                    inter = None if self.is_first_pp else self._recv(batch.num_tokens)
                    with nvtx_range("forward"):
                        tokens = self._forward(batch, inter)
                    if not self.is_last_pp:
                        self._send(tokens)
                        tokens = None
        self._last = (n_p, n_d, batch.prefill_sampled)
        self.h2d_bytes = self.stager.last_h2d_bytes
        if ev is not None:
            ev[1].record()
            self._step_events[sched.step_id] = ev
            if len(self._step_events) > 8192:
                for k in sorted(self._step_events)[:4096]:
                    del self._step_events[k]
        if tokens is not None:
            self._stage_samples(tokens, batch.num_samples)
            self.d2h_bytes = batch.num_samples * 8
        return n_p, n_d

    def device_time_ms(self, lo: int, hi: int) -> float:
        """Sum of forward device time of the steps with ``lo <= step_id < hi``."""
        torch.cuda.synchronize(self.device)
        return float(sum(e0.elapsed_time(e1) for sid, (e0, e1) in self._step_events.items() if lo <= sid < hi))

    def _resolve_token_refs(self, batch) -> None:
        """Decode rows whose input token the host did not know when it scheduled them (their sequence sampled
        it in the step launched just before) take it from that step's sample buffer, on the device."""
        if batch.num_token_refs:
            if self._dev_samples is None:
                raise RuntimeError("a step refers to the previous step's samples but none were kept")
            ops.resolve_token_refs(batch.input_ids[: batch.num_token_refs], self._dev_samples)

    def _stage_samples(self, tokens: torch.Tensor, n: int) -> None:
        slot = self._slot
        self._slot ^= 1
        self._unread.append((slot, n, self._last))
        if len(self._unread) > 2:          # a rank whose samples nobody reads keeps the newest two only
            self._unread.popleft()
        self._dev_samples = tokens
        if not self.is_cuda:
            self._host_samples[slot][:n].copy_(tokens[:n])
            return
        cur = torch.cuda.current_stream(self.device)
        self._copy_stream.wait_stream(cur)
        with torch.cuda.stream(self._copy_stream):
            self._host_samples[slot][:n].copy_(tokens[:n], non_blocking=True)
            self._host_statuses[slot].copy_(self._dev_status, non_blocking=True)
            self._sample_events[slot].record(self._copy_stream)
        # the next forward may overwrite the buffer `tokens` lives in: it starts after this copy
        cur.wait_event(self._sample_events[slot])

    def read_samples(self, n_p: int, n_d: int) -> tuple[list[int], list[int]]:
        """Blocks until the ids of the oldest launched step that has not been read are on the host. Prefill
        entries that did not sample are -1."""
        slot, n, last = self._unread.popleft()
        if self.is_cuda:
            self._sample_events[slot].synchronize()
            code = int(self._host_statuses[slot][0])
            if code:
                self._dev_status.zero_()
                raise RuntimeError(
                    f"GPU kernel {code >> 16} reported status {code & 0xFFFF} (1-3: pipeline wait ran out, "
                    "4: a tensor-parallel peer did not arrive in time, 5: index out of range)")
        flat = self._host_samples[slot][:n].tolist()
        _, _, sampled = last
        d_ids = flat[:n_d]
        p_ids, k = [], n_d
        for s in sampled:
            if s:
                p_ids.append(flat[k])
                k += 1
            else:
                p_ids.append(-1)
        return p_ids, d_ids

    # --- CUDA graphs ---------------------------------------------------------------------------
    def _capture_graphs(self) -> None:
        from ..data.wire import DecodeBatch, SchedulerOutput

        single_stage = self.is_first_pp and self.is_last_pp
        if not single_stage and (self.native is None or self.pp_microbatches > 1):
            return   # a stage body is one graph only when one native call runs it on the whole step
        runner = CUDAGraphRunner(make_bs_list(min(self.max_bs, 512)))

        def make_inputs(bs: int, greedy: bool):
            self.stager.reset()
            batch = self.stager.build(SchedulerOutput(decodes=DecodeBatch.of([(-1, 0, 0, 0, [0])])), pad_to=bs,
                                      fixed_blocks=True)
            batch.slots.fill_(-1)      # capture must not write real KV slots
            batch.all_greedy = greedy
            return batch

        # the p2p hand-off between stages stays outside the graphs (the reference does the same:
        # src/compute/model_runner.py:62-66,178-192); stages without the sampler need one variant only
        runner.capture((True, False) if self.is_last_pp else (True,), make_inputs, self._forward)
        self.stager.reset()
        self.graphs = runner

    def destroy(self) -> None:
        if self.graphs is not None:
            self.graphs.destroy()
        self.graphs = None
        self._dev_samples = None
