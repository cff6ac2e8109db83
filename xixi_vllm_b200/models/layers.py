"""Tensor-parallel building blocks for dense Qwen3 (reference: src/compute/layers/*.py).

Layers are thin parameter holders whose ``forward`` calls ``ops.dispatch``; parameters are
created directly on the target device, already sharded, and filled by ``load`` from a
*weight source* that can read sub-blocks of a checkpoint tensor, so a rank touches only
the bytes it owns (the reference reads every tensor in full on every rank and narrows
afterwards, reference: src/compute/layers/linear.py:27-42).

Megatron layout: QKV and gate/up are column-parallel (no gather), o_proj and down_proj are
row-parallel (partial sums need a reduction), embedding and LM head are vocab-parallel.
Row-parallel layers can return the *unreduced* partial so the caller can fuse the
reduction with the residual add and RMSNorm that follow.
"""

from __future__ import annotations

import torch

from ..ops import dispatch as ops
from ..parallel import collectives as coll
from ..parallel.groups import get_tp_group
from ..parallel.pp import divide

__all__ = [
    "ColumnParallelLinear", "RowParallelLinear", "QKVParallelLinear", "MergedColumnParallelLinear",
    "VocabParallelEmbedding", "ParallelLMHead", "RMSNorm", "RotaryEmbedding", "SiluAndMul",
    "pad_vocab_size", "TensorSource",
]


class TensorSource:
    """Weight source over in-memory tensors (tests, random init). ``read`` returns a sub-block."""

    def __init__(self, tensors: dict[str, torch.Tensor]) -> None:
        self.tensors = tensors

    def names(self):
        return list(self.tensors)

    def has(self, name: str) -> bool:
        return name in self.tensors

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.tensors[name].shape)

    def read(self, name: str, row0: int = 0, nrows: int | None = None, col0: int = 0,
             ncols: int | None = None) -> torch.Tensor:
        t = self.tensors[name]
        if t.dim() == 1:
            return t[row0: None if nrows is None else row0 + nrows]
        r1 = t.shape[0] if nrows is None else row0 + nrows
        c1 = t.shape[1] if ncols is None else col0 + ncols
        return t[row0:r1, col0:c1]


def _empty(shape, dtype, device) -> torch.Tensor:
    return torch.empty(shape, dtype=dtype, device=device)


class _Linear:
    def __init__(self, out_local: int, in_local: int, bias: bool, dtype, device) -> None:
        self.weight = _empty((out_local, in_local), dtype, device)
        self.bias = _empty((out_local,), dtype, device) if bias else None
        self.tp = get_tp_group()

    def _copy_rows(self, dst_row0: int, block: torch.Tensor) -> None:
        self.weight[dst_row0: dst_row0 + block.shape[0]].copy_(block)


class ColumnParallelLinear(_Linear):
    """``y = x W^T`` with W's output rows split across ranks; optional gather of the outputs."""

    def __init__(self, in_features: int, out_features: int, *, bias: bool = False,
                 gather_output: bool = False, dtype=torch.bfloat16, device="cpu") -> None:
        tp = get_tp_group()
        self.in_features, self.out_features = in_features, out_features
        self.out_local = divide(out_features, tp.size)
        self.gather_output = gather_output
        super().__init__(self.out_local, in_features, bias, dtype, device)

    def load(self, src, name: str, shard_id=None) -> None:
        r0 = self.tp.group_rank * self.out_local
        self.weight.copy_(src.read(name, r0, self.out_local))

    def load_bias(self, src, name: str, shard_id=None) -> None:
        r0 = self.tp.group_rank * self.out_local
        self.bias.copy_(src.read(name, r0, self.out_local))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = ops.linear(x, self.weight, self.bias)
        return coll.all_gather(y, self.tp, dim=-1) if self.gather_output else y

    __call__ = forward


class MergedColumnParallelLinear(_Linear):
    """Several column-parallel projections stacked on the output axis (gate | up).

    ``interleave=8`` (two equal projections only) stores the rows as repeating groups of
    [8 of the first | 8 of the second], the layout the GPU GEMM's fused SiLU-mul epilogue
    expects; ``forward_act`` then returns ``silu(gate) * up`` directly."""

    def __init__(self, in_features: int, output_sizes: list[int], *, bias: bool = False,
                 dtype=torch.bfloat16, device="cpu", interleave: int = 0) -> None:
        tp = get_tp_group()
        self.in_features = in_features
        self.output_sizes = list(output_sizes)
        self.local_sizes = [divide(s, tp.size) for s in output_sizes]
        self.interleave = interleave
        if interleave:
            if len(output_sizes) != 2 or self.local_sizes[0] != self.local_sizes[1] or self.local_sizes[0] % interleave:
                raise ValueError("interleaving needs two equal projections whose local size divides by the group")
        super().__init__(sum(self.local_sizes), in_features, bias, dtype, device)

    def load(self, src, name: str, shard_id: int = 0) -> None:
        n = self.local_sizes[shard_id]
        block = src.read(name, self.tp.group_rank * n, n)
        if self.interleave:
            g = self.interleave
            self.weight.view(n // g, 2, g, self.in_features)[:, shard_id].copy_(block.reshape(n // g, g, -1))
        else:
            self._copy_rows(sum(self.local_sizes[:shard_id]), block)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias)

    __call__ = forward

    def forward_act(self, x: torch.Tensor) -> torch.Tensor:
        """``silu(gate(x)) * up(x)``."""
        if self.interleave and self.bias is None:
            return ops.linear_silu_mul(x, self.weight)
        return ops.silu_mul(self.forward(x))


class QKVParallelLinear(_Linear):
    """Fused q|k|v projection split by heads. With more ranks than KV heads each KV head is
    replicated on ``tp / kv_heads`` consecutive ranks (reference: src/compute/layers/linear.py:157-268)."""

    def __init__(self, hidden_size: int, head_dim: int, num_heads: int, num_kv_heads: int, *,
                 bias: bool = False, dtype=torch.bfloat16, device="cpu") -> None:
        tp = get_tp_group()
        self.hidden_size, self.head_dim = hidden_size, head_dim
        self.total_heads, self.total_kv_heads = num_heads, num_kv_heads
        self.num_heads = divide(num_heads, tp.size)
        if tp.size >= num_kv_heads:
            self.num_kv_heads, self.kv_replicas = 1, divide(tp.size, num_kv_heads)
        else:
            self.num_kv_heads, self.kv_replicas = divide(num_kv_heads, tp.size), 1
        self.q_size = self.num_heads * head_dim
        self.kv_size = self.num_kv_heads * head_dim
        super().__init__(self.q_size + 2 * self.kv_size, hidden_size, bias, dtype, device)

    def _range(self, shard_id: str) -> tuple[int, int, int]:
        """(source row0, rows, destination row0) for shard 'q' | 'k' | 'v'."""
        r = self.tp.group_rank
        if shard_id == "q":
            return r * self.q_size, self.q_size, 0
        src0 = (r // self.kv_replicas) * self.kv_size
        dst0 = self.q_size + (0 if shard_id == "k" else self.kv_size)
        return src0, self.kv_size, dst0

    def load(self, src, name: str, shard_id: str = "q") -> None:
        s0, n, d0 = self._range(shard_id)
        self._copy_rows(d0, src.read(name, s0, n))

    def load_bias(self, src, name: str, shard_id: str = "q") -> None:
        s0, n, d0 = self._range(shard_id)
        self.bias[d0:d0 + n].copy_(src.read(name, s0, n))

    def load_merged(self, src, name: str) -> None:
        """Checkpoint stores one fused [q|k|v] tensor with all heads."""
        full_q = self.total_heads * self.head_dim
        full_kv = self.total_kv_heads * self.head_dim
        for shard, base in (("q", 0), ("k", full_q), ("v", full_q + full_kv)):
            s0, n, d0 = self._range(shard)
            self._copy_rows(d0, src.read(name, base + s0, n))

    def forward(self, x: torch.Tensor, defer: bool = False) -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias, None, defer and self.bias is None)

    __call__ = forward


class RowParallelLinear(_Linear):
    """``y = x W^T`` with W's input columns split across ranks: each rank's product is a
    partial sum. ``forward(x, reduce=False)`` returns the partial so the reduction can be
    fused with what follows; bias (full size) is added once, after the reduction."""

    def __init__(self, in_features: int, out_features: int, *, bias: bool = False,
                 dtype=torch.bfloat16, device="cpu") -> None:
        tp = get_tp_group()
        self.in_features, self.out_features = in_features, out_features
        self.in_local = divide(in_features, tp.size)
        super().__init__(out_features, self.in_local, bias, dtype, device)

    def load(self, src, name: str, shard_id=None) -> None:
        self.weight.copy_(src.read(name, 0, None, self.tp.group_rank * self.in_local, self.in_local))

    def load_bias(self, src, name: str, shard_id=None) -> None:
        self.bias.copy_(src.read(name))

    def forward(self, x: torch.Tensor, reduce: bool = True, out: torch.Tensor | None = None,
                defer: bool = False) -> torch.Tensor:
        y = ops.linear(x, self.weight, None, out if not reduce else None, defer and not reduce and out is None)
        if not reduce:
            return y
        y = coll.all_reduce(y, self.tp)
        return y + self.bias if self.bias is not None else y

    __call__ = forward


def pad_vocab_size(vocab_size: int, tp_size: int, multiple: int = 16) -> int:
    """Smallest size >= vocab whose per-rank share is a multiple of ``multiple``."""
    per = -(-vocab_size // tp_size)
    per = -(-per // multiple) * multiple
    return per * tp_size


class _VocabShard:
    def __init__(self, num_embeddings: int, embedding_dim: int, dtype, device) -> None:
        self.tp = get_tp_group()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.padded = pad_vocab_size(num_embeddings, self.tp.size)
        self.per_rank = self.padded // self.tp.size
        self.vocab_start = self.per_rank * self.tp.group_rank
        self.vocab_end = self.vocab_start + self.per_rank
        self.weight = _empty((self.per_rank, embedding_dim), dtype, device)

    def load(self, src, name: str, shard_id=None) -> None:
        rows = src.shape(name)[0]
        n = max(0, min(self.per_rank, rows - self.vocab_start))
        if n:
            self.weight[:n].copy_(src.read(name, self.vocab_start, n))
        if n < self.per_rank:
            self.weight[n:].zero_()


class VocabParallelEmbedding(_VocabShard):
    """Each rank looks up the ids it owns and contributes zeros for the rest; the sum over
    ranks is the embedding. ``forward(ids, reduce=False)`` returns the partial."""

    def __init__(self, num_embeddings: int, embedding_dim: int, *, dtype=torch.bfloat16, device="cpu"):
        super().__init__(num_embeddings, embedding_dim, dtype, device)

    def forward(self, ids: torch.Tensor, reduce: bool = True, out: torch.Tensor | None = None) -> torch.Tensor:
        y = ops.embedding(ids, self.weight, self.vocab_start, out if not reduce else None)
        if reduce and self.tp.size > 1:
            y = coll.all_reduce(y, self.tp)
        return y

    __call__ = forward


class ParallelLMHead(_VocabShard):
    """Vocab-parallel output projection. ``forward`` gathers full logits (padding removed);
    ``argmax`` finds the best token with two tiny gathers instead of moving logits
    (reference: src/compute/layers/vocab_parallel.py:171-216)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, *, dtype=torch.bfloat16, device="cpu"):
        super().__init__(num_embeddings, embedding_dim, dtype, device)

    def tie(self, embedding: VocabParallelEmbedding) -> None:
        self.weight = embedding.weight

    def local_logits(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = self.local_logits(x)
        if self.tp.size > 1:
            logits = coll.all_gather(logits, self.tp, dim=-1)
        return logits[..., : self.num_embeddings]

    __call__ = forward

    def argmax(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp.size == 1:
            return ops.argmax(self.local_logits(x)[..., : self.num_embeddings])
        logits = self.local_logits(x).float()
        n_valid = max(0, min(self.per_rank, self.num_embeddings - self.vocab_start))
        if n_valid < self.per_rank:
            logits[..., n_valid:] = float("-inf")
        val, idx = logits.max(dim=-1)
        idx = idx + self.vocab_start
        if self.tp.size == 1:
            return idx
        vals = coll.all_gather(val.unsqueeze(-1), self.tp, dim=-1)     # [bs, tp]
        idxs = coll.all_gather(idx.unsqueeze(-1), self.tp, dim=-1)
        # ties resolve to the lowest rank, i.e. the lowest token id, like a global argmax
        best = vals.argmax(dim=-1, keepdim=True)
        return idxs.gather(-1, best).squeeze(-1)


class RMSNorm:
    """Returns ``(normed, residual)``; with a residual it is the fused in-place add + norm
    (reference: src/compute/layers/layernorm.py:10-20)."""

    def __init__(self, hidden_size: int, eps: float = 1e-6, *, dtype=torch.bfloat16, device="cpu") -> None:
        self.weight = torch.ones(hidden_size, dtype=dtype, device=device)
        self.eps = eps

    def load(self, src, name: str, shard_id=None) -> None:
        self.weight.copy_(src.read(name))

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        if residual is None:
            return ops.rmsnorm(x, self.weight, self.eps), x
        return ops.add_rmsnorm(x, residual, self.weight, self.eps), residual

    __call__ = forward


class RotaryEmbedding:
    """One fp32 ``[max_pos, head_dim]`` cos|sin table shared by every layer (the reference
    builds one per layer, reference: src/compute/layers/rotary.py:37-39)."""

    _tables: dict[tuple, torch.Tensor] = {}

    def __init__(self, head_dim: int, max_position: int, theta: float, device="cpu") -> None:
        key = (head_dim, max_position, float(theta), str(device))
        if key not in self._tables:
            self._tables[key] = ops.build_cos_sin_cache(head_dim, max_position, theta, device)
        self.cos_sin = self._tables[key]
        self.head_dim = head_dim


class SiluAndMul:
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.silu_mul(x)

    __call__ = forward
