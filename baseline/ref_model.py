"""Writes the model directory the reference engine needs on disk: ``config.json``, a small
word-level tokenizer (requests are fed as token ids, the tokenizer only has to load and name
an EOS id), and seed-0 random bf16 safetensors of the named Qwen3 architecture
(reference: src/config.py:61-74, src/control/engine.py:86-93, src/compute/models/loader.py:56-58).
"""

from __future__ import annotations

import json
import os

import torch

from xixi_vllm_b200.config import qwen3_arch_config
from xixi_vllm_b200.models.loader import write_safetensors
from xixi_vllm_b200.models.synth import hf_tensor_shapes


def write_tokenizer(out_dir: str, size: int = 1024) -> None:
    from tokenizers import Tokenizer, models, pre_tokenizers

    vocab = {f"<t{i}>": i for i in range(size)}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<t0>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(os.path.join(out_dir, "tokenizer.json"))
    with open(os.path.join(out_dir, "tokenizer_config.json"), "w", encoding="utf-8") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "<t1>", "pad_token": "<t1>",
                   "unk_token": "<t0>", "model_max_length": 1 << 20}, f)
    with open(os.path.join(out_dir, "special_tokens_map.json"), "w", encoding="utf-8") as f:
        json.dump({"eos_token": "<t1>", "pad_token": "<t1>", "unk_token": "<t0>"}, f)


def make_reference_model_dir(out_dir: str, arch: str, seed: int = 0, std: float = 0.02,
                             shard_bytes: int = 4 << 30) -> str:
    """Idempotent: a finished directory (marker file present) is reused."""
    marker = os.path.join(out_dir, ".complete")
    if os.path.isfile(marker):
        return out_dir
    os.makedirs(out_dir, exist_ok=True)
    cfg = qwen3_arch_config(arch)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=1)
    write_tokenizer(out_dir)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    gen = torch.Generator(device=dev).manual_seed(seed)
    shard, used, idx = {}, 0, 0

    def flush():
        nonlocal shard, used, idx
        if shard:
            idx += 1
            write_safetensors(os.path.join(out_dir, f"model-{idx:05d}.safetensors"), shard, {"format": "pt"})
            shard, used = {}, 0

    for name, shape in hf_tensor_shapes(cfg).items():
        if name.endswith("norm.weight"):
            t = torch.ones(shape, dtype=torch.bfloat16)
        else:
            t = (torch.randn(shape, generator=gen, device=dev, dtype=torch.float32) * std).to(torch.bfloat16).cpu()
        n = t.numel() * 2
        if used and used + n > shard_bytes:
            flush()
        shard[name] = t
        used += n
    flush()
    open(marker, "w").close()
    return out_dir
