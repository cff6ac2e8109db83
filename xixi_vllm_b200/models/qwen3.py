"""Dense Qwen3 decoder (reference: src/compute/models/qwen3.py:28-314).

Pre-norm decoder with a running residual stream, per-head RMSNorm on q and k, NeoX rotary
embedding, GQA, SwiGLU MLP. The tensor-parallel reductions after o_proj and down_proj are
*deferred*: a layer hands its unreduced partial to the next normalisation point, where one
call reduces across ranks, adds the residual and normalises. Pipeline stages own a
contiguous layer range; the first holds the embedding, the last the final norm and LM head.
"""

from __future__ import annotations

import torch

from ..ops import dispatch as ops
from ..parallel.groups import get_pp_group, get_tp_group
from ..parallel.pp import IntermediateTensors, PPMissingLayer, get_pp_indices
from ..parallel.tp_comm import LibraryTPComm, TPComm
from .layers import (MergedColumnParallelLinear, ParallelLMHead, QKVParallelLinear, RMSNorm,
                     RotaryEmbedding, RowParallelLinear, VocabParallelEmbedding)

__all__ = ["Qwen3ForCausalLM", "Qwen3Model", "Qwen3DecoderLayer", "Qwen3Attention", "Qwen3MLP"]


class Qwen3MLP:
    def __init__(self, cfg, dtype, device) -> None:
        on_gpu = torch.device(device).type == "cuda"
        self.gate_up_proj = MergedColumnParallelLinear(cfg.hidden_size, [cfg.intermediate_size] * 2,
                                                       dtype=dtype, device=device, interleave=8 if on_gpu else 0)
        self.down_proj = RowParallelLinear(cfg.intermediate_size, cfg.hidden_size, dtype=dtype, device=device)

    def forward(self, x: torch.Tensor, comm: TPComm, final: bool = False):
        """Returns this rank's partial sum of the MLP output (possibly not computed yet: the
        communicator may run the down projection inside the kernel that reduces it)."""
        return comm.row_linear(self.down_proj, self.gate_up_proj.forward_act(x), final)


class Qwen3Attention:
    def __init__(self, cfg, layer_idx: int, dtype, device) -> None:
        self.layer_idx = layer_idx
        self.head_dim = cfg.head_dim
        self.qkv_proj = QKVParallelLinear(cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads,
                                          cfg.num_key_value_heads, bias=bool(cfg.get("attention_bias", False)),
                                          dtype=dtype, device=device)
        self.o_proj = RowParallelLinear(cfg.num_attention_heads * cfg.head_dim, cfg.hidden_size,
                                        dtype=dtype, device=device)
        self.q_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.k_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.rotary = RotaryEmbedding(cfg.head_dim, cfg.max_position_embeddings, cfg.rope_theta, device)
        self.num_heads = self.qkv_proj.num_heads
        self.num_kv_heads = self.qkv_proj.num_kv_heads
        self.scale = cfg.head_dim ** -0.5

    def forward(self, x: torch.Tensor, batch, k_cache: torch.Tensor, v_cache: torch.Tensor, comm: TPComm):
        qkv = self.qkv_proj(x, defer=True)      # split-K partials are summed inside the next kernel
        q = ops.qk_norm_rope_cache(qkv, self.q_norm.weight, self.k_norm.weight, self.q_norm.eps,
                                   self.rotary.cos_sin, batch.positions, batch.slots, k_cache, v_cache,
                                   self.num_heads, self.num_kv_heads, self.head_dim,
                                   prefill_begin=batch.attn.num_decode)
        o = ops.paged_attention(q, k_cache, v_cache, batch.attn, self.scale, self.num_heads,
                                self.num_kv_heads, self.head_dim)
        return comm.row_linear(self.o_proj, o)


class Qwen3DecoderLayer:
    def __init__(self, cfg, layer_idx: int, dtype, device) -> None:
        self.layer_idx = layer_idx
        self.self_attn = Qwen3Attention(cfg, layer_idx, dtype, device)
        self.mlp = Qwen3MLP(cfg, dtype, device)
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device)

    def forward(self, partial, residual, batch, k_cache, v_cache, comm: TPComm, last: bool = False):
        """``partial`` is the previous block's unreduced output (or the embedding partial).
        ``last`` marks the layer whose MLP output feeds the forward's final reduction."""
        ln = self.input_layernorm
        h, residual = comm.reduce_add_rmsnorm(partial, residual, ln.weight, ln.eps)
        attn_partial = self.self_attn.forward(h, batch, k_cache, v_cache, comm)
        ln = self.post_attention_layernorm
        h, residual = comm.reduce_add_rmsnorm(attn_partial, residual, ln.weight, ln.eps)
        return self.mlp.forward(h, comm, final=last), residual


class Qwen3Model:
    def __init__(self, cfg, dtype, device) -> None:
        pp = get_pp_group()
        self.cfg = cfg
        self.start_layer, self.end_layer = get_pp_indices(cfg.num_hidden_layers, pp.group_rank, pp.size)
        self.is_first, self.is_last = pp.is_first_rank, pp.is_last_rank
        self.embed_tokens = (VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device)
                             if self.is_first else PPMissingLayer())
        self.layers = [Qwen3DecoderLayer(cfg, i, dtype, device) for i in range(self.start_layer, self.end_layer)]
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device) if self.is_last else PPMissingLayer()
        # A stage that hands over to another one keeps a copy of that stage's first input norm: the native
        # executor ends the stage with "reduce + residual add + that norm", so the receiver starts at its QKV GEMM.
        self.boundary_norm = (None if self.is_last else
                              RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device))

    def forward(self, input_ids, batch, kv, comm: TPComm, intermediate: IntermediateTensors | None = None):
        """Returns final-normed hidden states on the last stage, else ``IntermediateTensors``."""
        comm.begin_forward()
        if self.is_first:
            out = comm.alloc_partial(input_ids.shape[0], final=not self.layers)
            partial, residual = self.embed_tokens(input_ids, reduce=False, out=out), None
        else:
            # the previous stage sends its last partial already reduced
            partial, residual = intermediate["hidden_states"], intermediate["residual"]
            comm = _NoReduceOnce(comm)
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            partial, residual = layer.forward(partial, residual, batch, kv.k_cache(i), kv.v_cache(i), comm,
                                              last=i == n - 1)
        if not self.is_last:
            return IntermediateTensors(hidden_states=comm.all_reduce(partial), residual=residual)
        h, _ = comm.reduce_add_rmsnorm(partial, residual, self.norm.weight, self.norm.eps)
        return h


class _NoReduceOnce(TPComm):
    """First normalisation point of a non-first stage: its input was reduced by the sender."""

    def __init__(self, inner: TPComm) -> None:
        self.inner, self.group, self._first = inner, inner.group, True

    def all_reduce(self, x):
        return self.inner.all_reduce(x)

    def begin_forward(self):
        self.inner.begin_forward()

    def alloc_partial(self, tokens, final=False):
        return self.inner.alloc_partial(tokens, final)

    def row_linear(self, proj, x, final=False):
        return self.inner.row_linear(proj, x, final)

    def reduce_add_rmsnorm(self, partial, residual, w, eps):
        if self._first:
            self._first = False
            if residual is None:
                return ops.rmsnorm(partial, w, eps), partial
            return ops.add_rmsnorm(partial, residual, w, eps), residual
        return self.inner.reduce_add_rmsnorm(partial, residual, w, eps)


# HF checkpoint name fragment -> (fused parameter, shard id)
_STACKED = {
    "q_proj": ("qkv_proj", "q"), "k_proj": ("qkv_proj", "k"), "v_proj": ("qkv_proj", "v"),
    "gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", 1),
}


class Qwen3ForCausalLM:
    def __init__(self, cfg, dtype=torch.bfloat16, device="cpu") -> None:
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.model = Qwen3Model(cfg, dtype, device)
        self.is_last = self.model.is_last
        self.lm_head = (ParallelLMHead(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device)
                        if self.is_last else PPMissingLayer())
        self.comm: TPComm = LibraryTPComm(get_tp_group())
        self.tied = bool(cfg.get("tie_word_embeddings", False))

    # --- forward -------------------------------------------------------------------------
    def forward(self, input_ids, batch, kv, intermediate=None):
        return self.model.forward(input_ids, batch, kv, self.comm, intermediate)

    __call__ = forward

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.lm_head(hidden)

    def greedy_tokens(self, hidden: torch.Tensor) -> torch.Tensor:
        fused = getattr(self.comm, "argmax", None)
        if fused is not None:
            head = self.lm_head
            valid = max(0, min(head.per_rank, head.num_embeddings - head.vocab_start))
            return fused(head.local_logits(hidden), valid, head.vocab_start)
        return self.lm_head.argmax(hidden)

    # --- weights ---------------------------------------------------------------------------
    def named_parameters(self):
        """(name, tensor) for every local parameter, HF-style names with fused projections."""
        m = self.model
        if m.is_first:
            yield "model.embed_tokens.weight", m.embed_tokens.weight
        for layer in m.layers:
            p = f"model.layers.{layer.layer_idx}."
            a, f = layer.self_attn, layer.mlp
            yield p + "self_attn.qkv_proj.weight", a.qkv_proj.weight
            if a.qkv_proj.bias is not None:
                yield p + "self_attn.qkv_proj.bias", a.qkv_proj.bias
            yield p + "self_attn.o_proj.weight", a.o_proj.weight
            yield p + "self_attn.q_norm.weight", a.q_norm.weight
            yield p + "self_attn.k_norm.weight", a.k_norm.weight
            yield p + "mlp.gate_up_proj.weight", f.gate_up_proj.weight
            yield p + "mlp.down_proj.weight", f.down_proj.weight
            yield p + "input_layernorm.weight", layer.input_layernorm.weight
            yield p + "post_attention_layernorm.weight", layer.post_attention_layernorm.weight
        if m.boundary_norm is not None:
            yield "model.boundary_norm.weight", m.boundary_norm.weight
        if m.is_last:
            yield "model.norm.weight", m.norm.weight
            yield "lm_head.weight", self.lm_head.weight

    def num_parameter_bytes(self) -> int:
        seen, total = set(), 0
        for _, t in self.named_parameters():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    def _target(self, name: str):
        """Resolve an HF tensor name to (layer object, loader method name, shard id) or None."""
        m = self.model
        if name == "model.embed_tokens.weight":
            return (m.embed_tokens, "load", None) if m.is_first else None
        if name == "model.norm.weight":
            return (m.norm, "load", None) if m.is_last else None
        if name == "lm_head.weight":
            return (self.lm_head, "load", None) if m.is_last else None
        parts = name.split(".")
        if len(parts) < 5 or parts[0] != "model" or parts[1] != "layers":
            return None
        idx = int(parts[2])
        if idx == m.end_layer and m.boundary_norm is not None and parts[3] == "input_layernorm":
            return m.boundary_norm, "load", None
        if not m.start_layer <= idx < m.end_layer:
            return None
        layer = m.layers[idx - m.start_layer]
        block, leaf, kind = parts[3], parts[4], parts[-1]
        if block in ("input_layernorm", "post_attention_layernorm"):
            return getattr(layer, block), "load", None
        owner = layer.self_attn if block == "self_attn" else layer.mlp if block == "mlp" else None
        if owner is None:
            return None
        method = "load" if kind == "weight" else "load_bias"
        if leaf in _STACKED:
            fused, shard = _STACKED[leaf]
            return getattr(owner, fused), method, shard
        if leaf == "qkv_proj":
            return owner.qkv_proj, "load_merged" if kind == "weight" else "load_bias", None
        if hasattr(owner, leaf):
            return getattr(owner, leaf), method, None
        return None

    def load_weights(self, src) -> dict:
        """Fill parameters from a weight source; returns ``{"loaded": n, "skipped": [...]}``.

        Names outside this stage's layer range are ignored; ``lm_head`` falls back to the
        embedding matrix when the checkpoint ties them or omits it.
        """
        loaded, skipped, saw_head = 0, [], False
        for name in src.names():
            if "rotary_emb.inv_freq" in name:
                continue
            tgt = self._target(name)
            if tgt is None:
                skipped.append(name)
                continue
            obj, method, shard = tgt
            if method == "load_merged":
                obj.load_merged(src, name)
            else:
                getattr(obj, method)(src, name, shard)
            saw_head |= name == "lm_head.weight"
            loaded += 1
        if self.is_last and not saw_head:
            if self.model.is_first:
                self.lm_head.tie(self.model.embed_tokens)
            elif src.has("model.embed_tokens.weight"):
                self.lm_head.load(src, "model.embed_tokens.weight")
            else:
                raise RuntimeError("checkpoint has neither lm_head.weight nor model.embed_tokens.weight")
        return {"loaded": loaded, "skipped": skipped}

    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        """Random weights generated on the device: N(0, std) matrices, unit norms. Every TP
        rank draws from its own stream, so shards are independent (fine for synthetic
        benchmarks; use a checkpoint when ranks must agree on a reference)."""
        dev = self.device
        gen = torch.Generator(device=dev)
        tp, pp = get_tp_group(), get_pp_group()
        gen.manual_seed(seed * 1000003 + tp.group_rank * 1009 + pp.group_rank * 17 + 1)
        for name, t in self.named_parameters():
            if name.endswith("norm.weight") or "layernorm" in name:
                t.fill_(1.0)
            elif name == "lm_head.weight" and self.tied and self.model.is_first:
                continue
            else:
                t.normal_(0.0, std, generator=gen)
        if self.tied and self.is_last and self.model.is_first:
            self.lm_head.tie(self.model.embed_tokens)
