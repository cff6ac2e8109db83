"""Plain-PyTorch implementations of every model op.

Two roles: the numerical oracle each CUDA kernel is tested against (run them in fp32), and
the execution backend for CPU/gloo runs, where the whole engine works without a GPU. The
reference cannot do the latter because its op wrappers import CUDA-only libraries at module
import (reference: src/compute/layers/ops.py:14-17, src/compute/layers/attention.py:9).

KV cache layout per layer: ``k_cache, v_cache: [num_blocks, kv_heads, block_size, head_dim]``
(head-major inside a page, so one page of one head is a contiguous run). Slot ``s`` is
page ``s // block_size``, offset ``s % block_size``.
"""

from __future__ import annotations


import torch

__all__ = [
    "rmsnorm", "add_rmsnorm", "linear", "silu_mul", "embedding", "build_cos_sin_cache",
    "qk_norm_rope_cache", "paged_attention", "sample", "argmax",
]


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * w.float()).to(x.dtype)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """``residual += x`` in place (rounded to its dtype), returns ``rmsnorm(residual)``."""
    residual.copy_((residual.float() + x.float()).to(residual.dtype))
    return rmsnorm(residual, w, eps)


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x[M,K] @ w[N,K]^T`` with fp32 accumulation."""
    if x.dtype in (torch.float32, torch.float64):
        y = x @ w.t()
        return y + bias if bias is not None else y
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def silu_mul(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    g, u = x[..., :d].float(), x[..., d:].float()
    return (g * torch.sigmoid(g) * u).to(x.dtype)


def embedding(ids: torch.Tensor, w: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    """Rows of ``w`` for ids inside ``[vocab_start, vocab_start + rows)``, zeros elsewhere."""
    local = ids.long() - vocab_start
    ok = (local >= 0) & (local < w.shape[0])
    out = w[local.clamp(0, w.shape[0] - 1)]
    return out * ok.unsqueeze(-1).to(out.dtype)


def build_cos_sin_cache(head_dim: int, max_pos: int, theta: float, device=None) -> torch.Tensor:
    """fp32 ``[max_pos, head_dim]``: cos in the first half of each row, sin in the second."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=-1).to(torch.float32).to(device)


def _rope_neox(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    # x: [T, heads, D] fp32; cos/sin: [T, D/2]
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def qk_norm_rope_cache(qkv: torch.Tensor, q_w: torch.Tensor, k_w: torch.Tensor, eps: float,
                       cos_sin: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                       k_cache: torch.Tensor, v_cache: torch.Tensor, num_q_heads: int,
                       num_kv_heads: int, head_dim: int) -> torch.Tensor:
    """Per-head RMSNorm of q and k, NeoX rotary embedding, and KV-cache append.

    Returns q ``[T, num_q_heads*head_dim]``. Rows whose slot is negative are not stored.
    """
    T = qkv.shape[0]
    D = head_dim
    nq, nk = num_q_heads * D, num_kv_heads * D
    q = qkv[:, :nq].reshape(T, num_q_heads, D).float()
    k = qkv[:, nq:nq + nk].reshape(T, num_kv_heads, D).float()
    v = qkv[:, nq + nk:nq + 2 * nk].reshape(T, num_kv_heads, D)
    q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_w.float()
    k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_w.float()
    cs = cos_sin[positions.long()].float()
    cos, sin = cs[:, : D // 2], cs[:, D // 2:]
    q = _rope_neox(q, cos, sin).to(qkv.dtype)
    k = _rope_neox(k, cos, sin).to(qkv.dtype)
    bs = k_cache.shape[2]
    keep = slots >= 0
    if bool(keep.any()):
        s = slots[keep].long()
        blk, off = s // bs, s % bs
        k_cache[blk, :, off, :] = k[keep].to(k_cache.dtype)
        v_cache[blk, :, off, :] = v[keep].to(v_cache.dtype)
    return q.reshape(T, nq)


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    cu_q: torch.Tensor, kv_lens: torch.Tensor, block_tables: torch.Tensor,
                    scale: float, num_q_heads: int, num_kv_heads: int, head_dim: int) -> torch.Tensor:
    """Causal GQA attention of packed queries against the paged cache.

    ``cu_q[b]..cu_q[b+1]`` are sequence b's query rows; they are the *last* ``q_len``
    positions of its ``kv_lens[b]`` cached tokens (the new tokens' KV is already appended).
    """
    T = q.shape[0]
    D = head_dim
    bs = k_cache.shape[2]
    group = num_q_heads // num_kv_heads
    out = torch.zeros(T, num_q_heads * D, dtype=q.dtype, device=q.device)
    cu = cu_q.tolist()
    lens = kv_lens.tolist()
    for b in range(len(lens)):
        q0, q1, L = cu[b], cu[b + 1], lens[b]
        n = q1 - q0
        if n == 0 or L == 0:
            continue
        nb = -(-L // bs)
        blocks = block_tables[b, :nb].long()
        k = k_cache[blocks].permute(1, 0, 2, 3).reshape(num_kv_heads, nb * bs, D)[:, :L].float()
        v = v_cache[blocks].permute(1, 0, 2, 3).reshape(num_kv_heads, nb * bs, D)[:, :L].float()
        qb = q[q0:q1].reshape(n, num_kv_heads, group, D).permute(1, 2, 0, 3).float()   # [Hkv,G,n,D]
        s = torch.einsum("hgnd,hld->hgnl", qb, k) * scale
        qpos = torch.arange(L - n, L, device=q.device)[:, None]
        kpos = torch.arange(L, device=q.device)[None, :]
        s = s.masked_fill(kpos > qpos, float("-inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("hgnl,hld->hgnd", p, v)                                        # [Hkv,G,n,D]
        out[q0:q1] = o.permute(2, 0, 1, 3).reshape(n, num_q_heads * D).to(q.dtype)
    return out


def argmax(logits: torch.Tensor) -> torch.Tensor:
    return logits.float().argmax(dim=-1)


def filtered_probs(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
                   top_p: torch.Tensor, min_p: torch.Tensor) -> torch.Tensor:
    """Distribution each non-greedy row is sampled from (reference: src/compute/sampler.py:27-118).

    Order: temperature, top-k, softmax over the survivors, top-p (a token stays if the mass
    strictly before it, in descending order, is <= top_p), min-p relative to the best
    survivor, renormalise. ``top_k <= 0``, ``top_p >= 1`` and ``min_p <= 0`` disable a filter.
    """
    B, V = logits.shape
    t = torch.where(temperature <= 1e-5, torch.ones_like(temperature), temperature).float()
    scaled = logits.float() / t[:, None]
    vals, idx = torch.sort(scaled, dim=-1, descending=True)
    rank = torch.arange(V, device=logits.device)[None, :]
    k = torch.where(top_k <= 0, torch.full_like(top_k, V), top_k).clamp(max=V)
    vals = vals.masked_fill(rank >= k[:, None], float("-inf"))
    p = torch.softmax(vals, dim=-1)
    drop = (p.cumsum(-1) - p) > top_p.float()[:, None]
    drop |= p < (min_p.float()[:, None] * p[:, :1])
    drop[:, 0] = False
    p = p.masked_fill(drop, 0.0)
    p = p / p.sum(-1, keepdim=True)
    out = torch.zeros_like(p)
    out.scatter_(1, idx, p)
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, min_p: torch.Tensor, generator: torch.Generator | None = None) -> torch.Tensor:
    """One token id per row; rows with temperature ~0 are greedy."""
    greedy = temperature <= 1e-5
    best = argmax(logits)
    if bool(greedy.all()):
        return best
    probs = filtered_probs(logits, temperature, top_k, top_p, min_p)
    drawn = torch.multinomial(probs, 1, generator=generator).squeeze(1)
    return torch.where(greedy, best, drawn)
