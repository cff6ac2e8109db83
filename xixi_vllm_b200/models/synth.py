"""Synthetic model directories: ``config.json`` plus seed-0 random safetensors shards of a
named Qwen3 architecture. Benchmarks use them because no checkpoints can be downloaded;
the reference engine needs such a directory on disk to start at all
(reference: src/config.py:61-74, src/compute/models/loader.py:56-58).

    python -m xixi_vllm_b200.models.synth --arch Qwen3-8B --out /tmp/q3-8b [--no-weights]
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from ..config import qwen3_arch_config
from .loader import write_safetensors

__all__ = ["make_model_dir", "hf_tensor_shapes"]


def hf_tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    """Every tensor of the unfused Hugging Face layout with its shape."""
    H, D = cfg["hidden_size"], cfg["head_dim"]
    nq, nkv, I, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"], cfg["vocab_size"]
    out: dict[str, tuple[int, ...]] = {"model.embed_tokens.weight": (V, H)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        out[p + "input_layernorm.weight"] = (H,)
        out[p + "post_attention_layernorm.weight"] = (H,)
        out[p + "self_attn.q_proj.weight"] = (nq * D, H)
        out[p + "self_attn.k_proj.weight"] = (nkv * D, H)
        out[p + "self_attn.v_proj.weight"] = (nkv * D, H)
        out[p + "self_attn.o_proj.weight"] = (H, nq * D)
        out[p + "self_attn.q_norm.weight"] = (D,)
        out[p + "self_attn.k_norm.weight"] = (D,)
        out[p + "mlp.gate_proj.weight"] = (I, H)
        out[p + "mlp.up_proj.weight"] = (I, H)
        out[p + "mlp.down_proj.weight"] = (H, I)
    out["model.norm.weight"] = (H,)
    if not cfg.get("tie_word_embeddings", False):
        out["lm_head.weight"] = (V, H)
    return out


def make_model_dir(out_dir: str, arch: str = "tiny", *, weights: bool = True, seed: int = 0,
                   std: float = 0.02, shard_bytes: int = 4 << 30, dtype: torch.dtype | None = None,
                   **overrides) -> str:
    cfg = qwen3_arch_config(arch, **overrides)
    os.makedirs(out_dir, exist_ok=True)
    # written under a temporary name and renamed, so a concurrent reader (another rank of the same
    # launch) sees either no file or the complete one
    tmp = os.path.join(out_dir, f".config.json.{os.getpid()}")
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=1)
    os.replace(tmp, os.path.join(out_dir, "config.json"))
    if not weights:
        return out_dir
    dtype = dtype or getattr(torch, cfg["torch_dtype"])
    gen = torch.Generator().manual_seed(seed)
    shard: dict[str, torch.Tensor] = {}
    used, idx = 0, 0

    def flush():
        nonlocal shard, used, idx
        if shard:
            idx += 1
            write_safetensors(os.path.join(out_dir, f"model-{idx:05d}.safetensors"), shard, {"format": "pt"})
            shard, used = {}, 0

    for name, shape in hf_tensor_shapes(cfg).items():
        if name.endswith("norm.weight"):
            t = torch.ones(shape, dtype=dtype)
        else:
            t = (torch.randn(shape, generator=gen, dtype=torch.float32) * std).to(dtype)
        nbytes = t.numel() * t.element_size()
        if used and used + nbytes > shard_bytes:
            flush()
        shard[name] = t
        used += nbytes
    flush()
    return out_dir


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--arch", default="tiny")
    ap.add_argument("--out", required=True)
    ap.add_argument("--no-weights", action="store_true", help="write config.json only (use load_format=dummy)")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    print(make_model_dir(a.out, a.arch, weights=not a.no_weights, seed=a.seed))


if __name__ == "__main__":
    main()
