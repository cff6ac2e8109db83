"""Python side of the native forward executor (``csrc/kernels/forward.cu``).

Describes the model (weights, caches, tensor-parallel communicator) and a preallocated
activation arena to the C library once; each step then fills a small batch struct and makes
ONE call that launches the whole forward of this pipeline stage. The module-by-module Python
forward stays as the CPU path. A stage that is not the first finds its inputs (normalised hidden
states and the residual stream) in the arena, where the model runner received them; a stage that
is not the last leaves its outputs there for the runner to send.
"""

from __future__ import annotations

import ctypes
import os

import torch

from ..ops import cuda

_vp, _i32, _i64, _f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float

__all__ = ["NativeForward"]


class LayerWeights(ctypes.Structure):
    _fields_ = [(n, _vp) for n in ("input_norm", "qkv", "q_norm", "k_norm", "o", "post_norm", "gate_up", "down",
                                   "k_cache", "v_cache")]


class ModelDesc(ctypes.Structure):
    _fields_ = [(n, _i32) for n in ("num_layers", "hidden", "hq", "hkv", "head_dim", "inter_local", "qkv_rows",
                                    "block_size")] + \
               [("eps", _f32), ("attn_scale", _f32), ("gate_up_interleaved", _i32), ("vocab_start", _i32),
                ("vocab_rows", _i32), ("lm_head_rows", _i32), ("lm_valid", _i32), ("embed", _vp), ("final_norm", _vp),
                ("lm_head", _vp), ("cos_sin", _vp), ("layers", ctypes.POINTER(LayerWeights)), ("tp_rank", _i32),
                ("tp_world", _i32), ("peer_bufs", _vp), ("peer_flags", _vp), ("mc_buf", _vp), ("epoch", _vp),
                ("h_offset", _i64), ("buf_bytes", _i64), ("slots_offset", _i64), ("spin_us", ctypes.c_uint),
                ("num_kv_blocks", _i32), ("prefill_tc", _i32), ("tp_push", _i32), ("tp_push_max", _i32),
                ("tp_one_shot_max", _i32), ("tp_pull_two_shot", _i32), ("tp_defer_row_wait", _i32), ("is_first", _i32),
                ("is_last", _i32)]


class BatchDesc(ctypes.Structure):
    _fields_ = [(n, _i32) for n in ("num_tokens", "num_seqs", "num_decode", "max_q_len", "max_blocks", "num_samples",
                                    "all_greedy")] + \
               [(n, _vp) for n in ("input_ids", "positions", "slots", "cu_q", "kv_lens", "block_tables", "sample_rows")]


class Arena(ctypes.Structure):
    _fields_ = [(n, _vp) for n in ("h", "qkv", "q", "attn", "act", "gu", "residual", "partial", "hidden_out", "logits",
                                   "tokens", "gemm_ws")] + \
               [("gemm_ws_bytes", _i64), ("attn_ws", _vp), ("attn_ws_bytes", _i64), ("status", _vp), ("num_sms", _i32)]


class NativeForward:
    def __init__(self, model, kv, *, max_tokens: int, max_samples: int) -> None:
        L = cuda.lib()
        L.xv_qwen3_forward.argtypes = [ctypes.POINTER(ModelDesc), ctypes.POINTER(BatchDesc), ctypes.POINTER(Arena), _vp]
        L.xv_forward_failed_op.restype = _i32
        L.xv_forward_launch_calls.restype = _i64
        self._lib = L
        m = model.model
        cfg = model.cfg
        dev = model.device
        if not m.layers:
            raise ValueError("the native forward needs at least one decoder layer per stage")
        self.is_first, self.is_last = bool(m.is_first), bool(m.is_last)
        first = m.layers[0]
        attn0 = first.self_attn
        self.hidden = cfg.hidden_size
        self.max_tokens, self.max_samples = max_tokens, max_samples
        self.layers = (LayerWeights * len(m.layers))()
        self._keep = [model, kv]
        for i, layer in enumerate(m.layers):
            a, f = layer.self_attn, layer.mlp
            lw = self.layers[i]
            lw.input_norm = layer.input_layernorm.weight.data_ptr()
            lw.qkv = a.qkv_proj.weight.data_ptr()
            lw.q_norm = a.q_norm.weight.data_ptr()
            lw.k_norm = a.k_norm.weight.data_ptr()
            lw.o = a.o_proj.weight.data_ptr()
            lw.post_norm = layer.post_attention_layernorm.weight.data_ptr()
            lw.gate_up = f.gate_up_proj.weight.data_ptr()
            lw.down = f.down_proj.weight.data_ptr()
            lw.k_cache = kv.k_cache(i).data_ptr()
            lw.v_cache = kv.v_cache(i).data_ptr()
            if a.qkv_proj.bias is not None:
                raise ValueError("the native forward does not apply QKV bias")
        head = model.lm_head if self.is_last else None
        d = ModelDesc()
        d.is_first, d.is_last = int(self.is_first), int(self.is_last)
        d.num_layers, d.hidden = len(m.layers), cfg.hidden_size
        d.hq, d.hkv, d.head_dim = attn0.num_heads, attn0.num_kv_heads, attn0.head_dim
        d.inter_local = first.mlp.down_proj.in_local
        d.qkv_rows = attn0.qkv_proj.weight.shape[0]
        d.block_size = kv.block_size
        d.num_kv_blocks = kv.k_cache(0).shape[0]
        d.prefill_tc = int(os.environ.get("XV_ATTN_PREFILL", "tc") != "mma")
        d.eps, d.attn_scale = float(cfg.rms_norm_eps), float(attn0.scale)
        d.gate_up_interleaved = 1 if first.mlp.gate_up_proj.interleave else 0
        if self.is_first:
            d.vocab_start, d.vocab_rows = m.embed_tokens.vocab_start, m.embed_tokens.weight.shape[0]
            d.embed = m.embed_tokens.weight.data_ptr()
        if self.is_last:
            d.lm_head_rows = head.weight.shape[0]
            d.lm_valid = max(0, min(head.per_rank, head.num_embeddings - head.vocab_start))
            d.final_norm = m.norm.weight.data_ptr()
            d.lm_head = head.weight.data_ptr()
        else:
            d.final_norm = m.boundary_norm.weight.data_ptr()    # the next stage's first input norm
        d.cos_sin = attn0.rotary.cos_sin.data_ptr()
        d.layers = ctypes.cast(self.layers, ctypes.POINTER(LayerWeights))
        comm = model.comm
        self.comm = comm
        if comm.group.size > 1:
            if not hasattr(comm, "symm"):
                raise ValueError("tensor-parallel native forward needs the fused peer-memory communicator")
            d.tp_rank, d.tp_world = comm.rank, comm.world
            d.peer_bufs = ctypes.cast(comm._bufs, _vp)
            d.peer_flags = ctypes.cast(comm._flags, _vp)
            d.mc_buf = comm.mc_ptr or None
            d.epoch = comm.epoch.data_ptr()
            d.buf_bytes, d.slots_offset = comm.buf_bytes, comm.slots_off
            d.h_offset = comm.h_off
            d.tp_pull_two_shot = 1 if comm.sharded_reduce else 0
            d.tp_push = 1 if comm.fuse_gemm else 0
            d.tp_push_max = comm.push_max_tokens
            d.tp_one_shot_max = comm.one_shot_max_tokens
            d.tp_defer_row_wait = (1 if comm.defer_row_wait else 0) | (2 if comm.pull_defer_row_wait else 0)
            from ..parallel.symm import SPIN_LIMIT

            d.spin_us = SPIN_LIMIT
        else:
            d.tp_rank, d.tp_world = 0, 1
            d.h_offset = -1
        self.desc = d
        self.vocab_local = d.lm_head_rows
        lm_rows = max(d.lm_head_rows, 8)

        def buf(rows, cols, dtype=torch.bfloat16):
            return torch.empty((rows, cols), dtype=dtype, device=dev)

        T, S, H = max_tokens, max_samples, cfg.hidden_size
        q_cols = d.hq * d.head_dim
        if d.tp_world > 1:
            if T > comm.max_tokens:
                raise ValueError("arena larger than the communicator's symmetric buffers")
            h_buf = comm.h_view[: T * H].view(T, H)        # broadcast target of the row-sharded reductions
        else:
            h_buf = buf(T, H)
        self.t = dict(h=h_buf, qkv=buf(T, d.qkv_rows), q=buf(T, q_cols), attn=buf(T, q_cols),
                      act=buf(T, d.inter_local), residual=buf(T, H), partial=buf(T, H), hidden_out=buf(S, H),
                      logits=buf(S, lm_rows), tokens=torch.zeros(S, dtype=torch.int64, device=dev))
        if not d.gate_up_interleaved:
            self.t["gu"] = buf(T, 2 * d.inter_local)
        st = cuda._state(self.t["h"])
        need = L.xv_attn_decode_workspace_bytes(max_samples, d.hq, d.head_dim, 16)
        if need > st.attn_ws.numel():
            st.attn_ws = torch.empty(need, dtype=torch.uint8, device=dev)
        self._state = st
        a = Arena()
        for name in ("h", "qkv", "q", "attn", "act", "residual", "partial", "hidden_out", "logits", "tokens"):
            setattr(a, name, self.t[name].data_ptr())
        a.gu = self.t["gu"].data_ptr() if "gu" in self.t else None
        a.gemm_ws, a.gemm_ws_bytes = st.gemm_ws.data_ptr(), st.gemm_ws.numel()
        a.attn_ws, a.attn_ws_bytes = st.attn_ws.data_ptr(), st.attn_ws.numel()
        a.status, a.num_sms = st.status.data_ptr(), st.num_sms
        self.arena = a
        self.launches_per_call = 0

    def stage_inputs(self, n_tokens: int):
        """Where a stage that is not the first receives (hidden states, residual stream)."""
        return self.t["h"][:n_tokens], self.t["residual"][:n_tokens]

    def forward(self, batch):
        """Launches the stage. On the last stage returns the int64 token tensor for greedy batches, else the
        local logits; on other stages the (hidden states, residual stream) pair to hand on."""
        if batch.num_tokens > self.max_tokens or batch.num_samples > self.max_samples:
            raise RuntimeError("batch exceeds the native forward's arena")
        at = batch.attn
        b = BatchDesc()
        b.num_tokens, b.num_seqs, b.num_decode = batch.num_tokens, at.num_seqs, at.num_decode
        b.max_q_len, b.max_blocks = at.max_q_len, at.block_tables.shape[1]
        b.num_samples, b.all_greedy = batch.num_samples, 1 if batch.all_greedy else 0
        b.input_ids, b.positions, b.slots = batch.input_ids.data_ptr(), batch.positions.data_ptr(), batch.slots.data_ptr()
        b.cu_q, b.kv_lens, b.block_tables = at.cu_q.data_ptr(), at.kv_lens.data_ptr(), at.block_tables.data_ptr()
        b.sample_rows = batch.sample_rows.data_ptr()
        before = self._lib.xv_forward_launch_calls()
        rc = self._lib.xv_qwen3_forward(ctypes.byref(self.desc), ctypes.byref(b), ctypes.byref(self.arena),
                                        torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"native forward failed at step {self._lib.xv_forward_failed_op()}: "
                               f"{cuda.ERRORS.get(rc, rc)}")
        cuda.launch_count += self._lib.xv_forward_launch_calls() - before
        if not self.is_last:
            return self.stage_inputs(batch.num_tokens)
        if batch.all_greedy:
            return self.t["tokens"][: batch.num_samples]
        return self.t["logits"][: batch.num_samples]
