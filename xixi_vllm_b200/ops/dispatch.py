"""Entry points used by model code. A CUDA tensor goes to the sm_100a kernels, a CPU tensor
to the PyTorch oracle. There is exactly one GPU implementation per op; if the CUDA library
is missing on a machine with a GPU the call raises instead of falling back.
"""

from __future__ import annotations

import torch

from . import cpu_ref

__all__ = [
    "rmsnorm", "add_rmsnorm", "linear", "linear_silu_mul", "silu_mul", "embedding", "qk_norm_rope_cache",
    "paged_attention", "sample", "argmax", "build_cos_sin_cache", "gather_rows",
    "resolve_token_refs",
]

build_cos_sin_cache = cpu_ref.build_cos_sin_cache


def _cuda():
    from . import cuda

    return cuda


def rmsnorm(x, w, eps):
    return _cuda().rmsnorm(x, w, eps) if x.is_cuda else cpu_ref.rmsnorm(x, w, eps)


def add_rmsnorm(x, residual, w, eps):
    return _cuda().add_rmsnorm(x, residual, w, eps) if x.is_cuda else cpu_ref.add_rmsnorm(x, residual, w, eps)


def linear(x, w, bias=None, out=None, defer=False):
    """``defer=True`` lets the GPU GEMM hand back unreduced split-K partials; only pass the result
    to ``add_rmsnorm`` or ``qk_norm_rope_cache`` (they sum the partials themselves)."""
    if x.is_cuda:
        return _cuda().linear(x, w, bias, out, defer)
    y = cpu_ref.linear(x, w, bias)
    if out is not None:
        out.copy_(y)
        return out
    return y


def linear_silu_mul(x, w):
    """GPU only: fused gate/up projection + SiLU-mul over an interleaved weight (see ops.cuda)."""
    return _cuda().linear_silu_mul(x, w)


def silu_mul(x):
    return _cuda().silu_mul(x) if x.is_cuda else cpu_ref.silu_mul(x)


def embedding(ids, w, vocab_start=0, out=None):
    if w.is_cuda:
        return _cuda().embedding(ids, w, vocab_start, out)
    y = cpu_ref.embedding(ids, w, vocab_start)
    if out is not None:
        out.copy_(y)
        return out
    return y


def qk_norm_rope_cache(qkv, q_w, k_w, eps, cos_sin, positions, slots, k_cache, v_cache,
                       num_q_heads, num_kv_heads, head_dim, prefill_begin: int = 0):
    """``prefill_begin``: index of the first prefill row of the packed batch (decode rows come first).
    The GPU kernel clears the V rows that follow a prefill chunk's last row inside its page."""
    if qkv.is_cuda:
        return _cuda().qk_norm_rope_cache(qkv, q_w, k_w, eps, cos_sin, positions, slots, k_cache, v_cache,
                                          num_q_heads, num_kv_heads, head_dim, prefill_begin)
    return cpu_ref.qk_norm_rope_cache(qkv, q_w, k_w, eps, cos_sin, positions, slots, k_cache, v_cache,
                                      num_q_heads, num_kv_heads, head_dim)


def paged_attention(q, k_cache, v_cache, attn, scale, num_q_heads, num_kv_heads, head_dim):
    """``attn`` is a ``runtime.staging.AttnBatch`` (cu_q, kv_lens, block_tables, decode split)."""
    if q.is_cuda:
        return _cuda().paged_attention(q, k_cache, v_cache, attn, scale, num_q_heads, num_kv_heads, head_dim)
    return cpu_ref.paged_attention(q, k_cache, v_cache, attn.cu_q, attn.kv_lens, attn.block_tables,
                                   scale, num_q_heads, num_kv_heads, head_dim)


def argmax(logits):
    return _cuda().argmax(logits) if logits.is_cuda else cpu_ref.argmax(logits)


def sample(logits, temperature, top_k, top_p, min_p, *, rng=None, generator=None):
    """``rng``: device int32 ``[seed, step]`` (GPU path); ``generator``: torch generator (CPU path)."""
    if logits.is_cuda:
        return _cuda().sample(logits, temperature, top_k, top_p, min_p, rng)
    return cpu_ref.sample(logits, temperature, top_k, top_p, min_p, generator)


def resolve_token_refs(ids, prev) -> None:
    """In place: input ids < 0 name rows of the previous step's sample buffer (``-(row) - 1``)."""
    if ids.is_cuda:
        _cuda().resolve_token_refs(ids, prev)
        return
    neg = ids < 0
    if bool(neg.any()):
        ids[neg] = prev[(-ids[neg] - 1).long()].to(ids.dtype)


def gather_rows(x, rows):
    """``x[rows]`` for int32 row indices."""
    if x.is_cuda:
        return _cuda().gather_rows(x, rows)
    return x.index_select(0, rows.long())
