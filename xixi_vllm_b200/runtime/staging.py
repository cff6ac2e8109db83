"""Per-step forward inputs (reference: src/compute/batch.py:37-251).

A step's decode tokens and prefill chunks are packed into ONE varlen batch (decodes first),
so the weights stream once per step instead of once per phase. All integer and float
metadata of the step lives in one pinned host buffer and reaches the device with a single
copy; device-side views into that buffer are what kernels read.

Workers keep each live sequence's block table in a persistent host array and receive only
the new tail entries from the driver (see ``data/wire.py``).
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np
import torch

from ..ops import hostlib

__all__ = ["AttnBatch", "ForwardBatch", "BatchStager", "split_forward_batch"]


@dataclass
class AttnBatch:
    cu_q: torch.Tensor          # [B+1] int32, query row ranges
    kv_lens: torch.Tensor       # [B]   int32, KV length including this step's tokens
    block_tables: torch.Tensor  # [B, max_blocks] int32
    num_seqs: int
    num_decode: int             # the first num_decode sequences have exactly one query row
    max_q_len: int
    max_kv_len: int
    num_tokens: int
    # host copies for launch-shape decisions (never read inside CUDA graphs)
    cu_q_host: np.ndarray | None = None
    kv_lens_host: np.ndarray | None = None


@dataclass
class ForwardBatch:
    input_ids: torch.Tensor     # [T] int32
    positions: torch.Tensor     # [T] int32
    slots: torch.Tensor         # [T] int32, -1 = do not store KV (padding rows)
    attn: AttnBatch
    sample_rows: torch.Tensor   # [S] int32 rows of the hidden states that need logits
    temperature: torch.Tensor   # [S] f32
    top_k: torch.Tensor         # [S] int32 (0 = off)
    top_p: torch.Tensor         # [S] f32 (1 = off)
    min_p: torch.Tensor         # [S] f32 (0 = off)
    rng: torch.Tensor           # [2] int32 on the device: seed, step counter
    num_tokens: int
    num_samples: int
    all_greedy: bool
    n_prefill: int
    n_decode: int
    prefill_sampled: list[bool]
    # leading rows of input_ids among which some are references into the previous step's samples (ids < 0,
    # one-step-late scheduling); 0 = none
    num_token_refs: int = 0


def split_forward_batch(batch: ForwardBatch, parts: int) -> list[tuple[ForwardBatch, int, int]]:
    """Cuts a staged batch into at most ``parts`` micro-batches of whole sequences with about equal token
    counts, for pipeline stages that want several pieces of a step in flight. Returns ``(sub, t0, t1)``
    triples: ``sub`` views rows ``t0:t1`` of the packed token arrays and the matching sequence range, with
    its query offsets and sample rows rebased to the piece. Concatenating the pieces' samples in order gives
    the full batch's sample order (decodes first, then the prefills that finish their prompt)."""
    a = batch.attn
    B = a.num_seqs
    cu = a.cu_q_host
    if parts <= 1 or B < 2 or cu is None:
        return [(batch, 0, batch.num_tokens)]
    parts = min(parts, B)
    T = int(cu[B])
    bounds = [0]
    for k in range(1, parts):
        s = int(np.searchsorted(cu[1:B + 1], T * k / parts, side="left")) + 1     # first boundary at/after the target
        s = min(max(s, bounds[-1] + 1), B - (parts - k))                           # every piece keeps a sequence
        bounds.append(s)
    bounds.append(B)
    n_d = a.num_decode
    # samples before each sequence: every decode row samples, a prefill only when it finishes its prompt
    flags = [1] * n_d + [1 if f else 0 for f in batch.prefill_sampled]
    flags += [0] * (B - len(flags))
    before = np.concatenate(([0], np.cumsum(flags)))
    out: list[tuple[ForwardBatch, int, int]] = []
    kv_host = a.kv_lens_host
    for s0, s1 in zip(bounds[:-1], bounds[1:]):
        if s1 <= s0:
            continue
        t0, t1 = int(cu[s0]), int(cu[s1])
        r0, r1 = int(before[s0]), min(int(before[s1]), batch.num_samples)
        q_lens = np.diff(cu[s0:s1 + 1])
        sub_attn = AttnBatch(cu_q=a.cu_q[s0:s1 + 1] - t0, kv_lens=a.kv_lens[s0:s1], block_tables=a.block_tables[s0:s1],
                             num_seqs=s1 - s0, num_decode=max(0, min(n_d, s1) - s0),
                             max_q_len=int(q_lens.max()) if q_lens.size else 1,
                             max_kv_len=int(kv_host[s0:s1].max()) if kv_host is not None else a.max_kv_len,
                             num_tokens=t1 - t0, cu_q_host=cu[s0:s1 + 1] - t0,
                             kv_lens_host=kv_host[s0:s1] if kv_host is not None else None)
        n_dec = sub_attn.num_decode
        sub = ForwardBatch(input_ids=batch.input_ids[t0:t1], positions=batch.positions[t0:t1], slots=batch.slots[t0:t1],
                           attn=sub_attn, sample_rows=batch.sample_rows[r0:r1] - t0,
                           temperature=batch.temperature[r0:r1], top_k=batch.top_k[r0:r1], top_p=batch.top_p[r0:r1],
                           min_p=batch.min_p[r0:r1], rng=batch.rng, num_tokens=t1 - t0, num_samples=r1 - r0,
                           all_greedy=batch.all_greedy, n_prefill=(s1 - s0) - n_dec, n_decode=n_dec,
                           prefill_sampled=batch.prefill_sampled[max(0, s0 - n_d):max(0, s1 - n_d)])
        out.append((sub, t0, t1))
    return out


class BatchStager:
    """Owns the host/device staging buffers and the per-sequence block-table rows."""

    def __init__(self, *, max_seqs: int, max_tokens: int, max_blocks: int, block_size: int, device,
                 seed: int = 0) -> None:
        self.seed, self.step_counter = int(seed) & 0x7FFFFFFF, 0
        self.max_seqs, self.max_tokens, self.max_blocks = max_seqs, max_tokens, max_blocks
        self.block_size = block_size
        self.device = torch.device(device)
        self._lib = hostlib.get()
        cuda = self.device.type == "cuda"
        # persistent block-table rows, one per live sequence (+ headroom for the step in which
        # rows are released and reassigned)
        self.num_rows = max_seqs * 2 + 8
        self.tables = np.zeros((self.num_rows, max_blocks), dtype=np.int32)
        self.row_of: dict[int, int] = {}
        # sampling parameters remembered per row (decode messages do not repeat them)
        self.row_temp = np.zeros(self.num_rows, dtype=np.float32)
        self.row_topk = np.zeros(self.num_rows, dtype=np.int32)
        self.row_topp = np.ones(self.num_rows, dtype=np.float32)
        self.row_minp = np.zeros(self.num_rows, dtype=np.float32)
        self.free_rows = list(range(self.num_rows - 1, -1, -1))
        cap = 3 * max_tokens + 8 * (max_seqs + 1) + max_seqs * max_blocks + 64
        # Two pinned buffers used in turn: with one-step-late scheduling the host packs step n + 1 while the
        # copy of step n's buffer may still be queued behind the forward before it.
        self._hosts = [torch.zeros(cap, dtype=torch.int32, pin_memory=cuda) for _ in range(2 if cuda else 1)]
        self._hosts_np = [h.numpy() for h in self._hosts]
        self._host_idx = 0
        self.host = self._hosts[0]
        self.host_np = self._hosts_np[0]
        self.dev = torch.zeros(cap, dtype=torch.int32, device=self.device) if cuda else self.host
        self.last_h2d_bytes = 0
        self._rows_tmp = np.zeros(max_seqs, dtype=np.int32)
        self._cached_tmp = np.zeros(max_seqs, dtype=np.int32)

    # --- block-table rows ------------------------------------------------------------------
    def release(self, seq_ids) -> None:
        for sid in seq_ids:
            row = self.row_of.pop(sid, None)
            if row is not None:
                self.free_rows.append(row)

    def reset(self) -> None:
        self.row_of.clear()
        self.free_rows = list(range(self.num_rows - 1, -1, -1))

    def _row(self, entry) -> int:
        row = self.row_of.get(entry.seq_id)
        if row is None:
            if not self.free_rows:
                raise RuntimeError("out of block-table rows: more live sequences than 2*max_num_seqs")
            row = self.free_rows.pop()
            self.row_of[entry.seq_id] = row
            if entry.bt_from != 0:
                raise RuntimeError(f"sequence {entry.seq_id}: first message must carry the whole block table")
        tail = entry.bt_tail
        if tail:
            end = entry.bt_from + len(tail)
            if end > self.max_blocks:
                raise RuntimeError(f"sequence {entry.seq_id} needs {end} pages > max_blocks={self.max_blocks}")
            self.tables[row, entry.bt_from:end] = tail
        self.row_temp[row] = entry.temperature
        self.row_topk[row] = entry.top_k if entry.top_k is not None and entry.top_k > 0 else 0
        self.row_topp[row] = entry.top_p if entry.top_p is not None else 1.0
        self.row_minp[row] = entry.min_p if entry.min_p is not None else 0.0
        return row

    def _decode_rows(self, dec) -> np.ndarray:
        """Rows of the decode batch's sequences, after applying its sparse block-table updates."""
        n = len(dec.seq_ids)
        rows = self._rows_tmp[:n]
        row_of = self.row_of
        try:
            rows[:] = [row_of[sid] for sid in dec.seq_ids]
        except KeyError:
            # first sight of a sequence in a decode message (no prefill seen by this worker)
            for i, sid in enumerate(dec.seq_ids):
                r = row_of.get(sid)
                if r is None:
                    if not self.free_rows:
                        raise RuntimeError("out of block-table rows: more live sequences than 2*max_num_seqs")
                    r = row_of[sid] = self.free_rows.pop()
                    self.row_temp[r], self.row_topk[r], self.row_topp[r], self.row_minp[r] = 0.0, 0, 1.0, 0.0
                rows[i] = r
        off = 0
        for i, start, cnt in zip(dec.bt_index, dec.bt_from, dec.bt_count):
            end = start + cnt
            if end > self.max_blocks:
                raise RuntimeError(f"sequence {dec.seq_ids[i]} needs {end} pages > max_blocks={self.max_blocks}")
            self.tables[rows[i], start:end] = dec.bt_vals[off:off + cnt]
            off += cnt
        return rows

    # --- packing -----------------------------------------------------------------------------
    def build(self, sched, *, pad_to: int | None = None, fixed_blocks: bool = False) -> ForwardBatch:
        """Pack ``sched`` (a ``SchedulerOutput``). ``pad_to`` pads a pure-decode batch with inert
        rows up to a CUDA-graph bucket; ``fixed_blocks`` makes the block-table width
        ``max_blocks`` regardless of content (graph replay needs fixed strides)."""
        self.release(sched.released)
        decodes, prefills = sched.decodes, sched.prefills
        n_d, n_p = len(decodes), len(prefills)
        bsz = self.block_size
        B_real = n_d + n_p
        B = max(B_real, pad_to or 0)
        T_real = n_d + sum(len(e.token_ids) for e in prefills)
        rows_d = self._decode_rows(decodes) if n_d else None
        T = T_real + (B - B_real)
        if T > self.max_tokens or B > self.max_seqs:
            raise RuntimeError(f"batch of {T} tokens / {B} sequences exceeds staging capacity")

        rows_p = [self._row(e) for e in prefills]
        max_kv = 1
        if n_d:
            cached = self._cached_tmp[:n_d]
            cached[:] = decodes.cached
            max_kv = int(cached.max()) + 1
        for e in prefills:
            max_kv = max(max_kv, e.num_cached_tokens + len(e.token_ids))
        nblk = self.max_blocks if fixed_blocks else max(1, -(-max_kv // bsz))

        if len(self._hosts) > 1:
            self._host_idx ^= 1
            self.host = self._hosts[self._host_idx]
            self.host_np = self._hosts_np[self._host_idx]
        h = self.host_np
        o = 0
        ids = h[o:o + T]; o += T
        pos = h[o:o + T]; o += T
        slots = h[o:o + T]; o += T
        cu_q = h[o:o + B + 1]; o += B + 1
        kv_lens = h[o:o + B]; o += B
        srows = h[o:o + B]; o += B
        temp = h[o:o + B].view(np.float32); o += B
        topk = h[o:o + B]; o += B
        topp = h[o:o + B].view(np.float32); o += B
        minp = h[o:o + B].view(np.float32); o += B
        bt = h[o:o + B * nblk].reshape(B, nblk); o += B * nblk
        rng = h[o:o + 2]; o += 2
        self.step_counter += 1
        rng[0] = self.seed
        rng[1] = self.step_counter & 0x7FFFFFFF
        used = o

        # decode rows
        n_refs = 0
        if n_d:
            ids[:n_d] = decodes.tokens
            if int(ids[:n_d].min()) < 0:
                n_refs = n_d
            if self._lib is not None:
                p = lambda a: a.ctypes.data_as(ctypes.c_void_p)  # noqa: E731
                self._lib.xv_fill_decode(n_d, p(rows_d), p(cached), p(self.tables), self.max_blocks, bsz,
                                         p(pos), p(slots), p(kv_lens), p(bt), nblk)
            else:
                pos[:n_d] = cached
                kv_lens[:n_d] = cached + 1
                t = self.tables[rows_d]
                slots[:n_d] = t[np.arange(n_d), cached // bsz] * bsz + cached % bsz
                w = min(nblk, self.max_blocks)
                bt[:n_d, :w] = t[:, :w]
            cu_q[:n_d + 1] = np.arange(n_d + 1, dtype=np.int32)
        else:
            cu_q[0] = 0

        # prefill chunks
        t_off = n_d
        max_q = 1 if n_d else 0
        n_s = n_d
        srows[:n_d] = np.arange(n_d, dtype=np.int32)
        prefill_sampled: list[bool] = []
        for j, e in enumerate(prefills):
            b = n_d + j
            n = len(e.token_ids)
            c = e.num_cached_tokens
            ids[t_off:t_off + n] = e.token_ids
            p_arr = np.arange(c, c + n, dtype=np.int32)
            pos[t_off:t_off + n] = p_arr
            trow = self.tables[rows_p[j]]
            slots[t_off:t_off + n] = trow[p_arr // bsz] * bsz + p_arr % bsz
            kv_lens[b] = c + n
            cu_q[b + 1] = t_off + n
            nb = -(-(c + n) // bsz)
            bt[b, :nb] = trow[:nb]
            bt[b, nb:] = 0
            if e.need_sample:
                srows[n_s] = t_off + n - 1
                n_s += 1
            prefill_sampled.append(bool(e.need_sample))
            max_q = max(max_q, n)
            t_off += n

        # inert padding rows (graph buckets): one token, no KV write, empty context
        for b in range(B_real, B):
            ids[t_off] = 0
            pos[t_off] = 0
            slots[t_off] = -1
            kv_lens[b] = 0
            cu_q[b + 1] = t_off + 1
            bt[b, :] = 0
            t_off += 1

        # sampling parameters, in sample-row order (decodes, then prefills that finish)
        greedy = True
        k = n_d
        if n_d:
            temp[:n_d] = self.row_temp[rows_d]
            greedy = bool((temp[:n_d] <= 1e-5).all())
            if greedy:
                topk[:n_d] = 0
                topp[:n_d] = 1.0
                minp[:n_d] = 0.0
            else:
                topk[:n_d] = self.row_topk[rows_d]
                topp[:n_d] = self.row_topp[rows_d]
                minp[:n_d] = self.row_minp[rows_d]
        for e in prefills:
            if e.need_sample:
                greedy &= self._put_sampling(e, k, temp, topk, topp, minp)
                k += 1
        if pad_to and n_s < B:     # padded rows still produce (ignored) samples in graph mode
            if n_p:
                raise RuntimeError("only pure-decode batches can be padded to a graph bucket")
            srows[n_s:B] = np.arange(n_s, B, dtype=np.int32)
            temp[n_s:B] = 0.0
            topk[n_s:B] = 0
            topp[n_s:B] = 1.0
            minp[n_s:B] = 0.0
        S = B if pad_to else n_s

        self.last_h2d_bytes = used * 4
        if self.dev is not self.host:
            self.dev[:used].copy_(self.host[:used], non_blocking=True)
        d = self.dev
        o = 0
        def take(n):  # noqa: E306
            nonlocal o
            v = d[o:o + n]
            o += n
            return v
        d_ids, d_pos, d_slots = take(T), take(T), take(T)
        d_cu, d_kv, d_srows = take(B + 1), take(B), take(B)
        d_temp, d_topk = take(B).view(torch.float32), take(B)
        d_topp, d_minp = take(B).view(torch.float32), take(B).view(torch.float32)
        d_bt = take(B * nblk).view(B, nblk)
        d_rng = take(2)
        attn = AttnBatch(cu_q=d_cu, kv_lens=d_kv, block_tables=d_bt, num_seqs=B, num_decode=n_d + (B - B_real),
                         max_q_len=max(max_q, 1), max_kv_len=max_kv, num_tokens=T,
                         cu_q_host=cu_q.copy(), kv_lens_host=kv_lens.copy())
        return ForwardBatch(input_ids=d_ids, positions=d_pos, slots=d_slots, attn=attn,
                            sample_rows=d_srows[:S], temperature=d_temp[:S], top_k=d_topk[:S],
                            top_p=d_topp[:S], min_p=d_minp[:S], rng=d_rng, num_tokens=T, num_samples=S,
                            all_greedy=greedy, n_prefill=n_p, n_decode=n_d, prefill_sampled=prefill_sampled,
                            num_token_refs=n_refs)

    @staticmethod
    def _put_sampling(e, k: int, temp, topk, topp, minp) -> bool:
        t = float(e.temperature)
        temp[k] = t
        topk[k] = int(e.top_k) if e.top_k is not None and e.top_k > 0 else 0
        topp[k] = float(e.top_p) if e.top_p is not None else 1.0
        minp[k] = float(e.min_p) if e.min_p is not None else 0.0
        return t <= 1e-5
