"""Engine configuration (reference: src/config.py:9-92).

Field names and defaults follow the reference so its YAML files and call sites keep
working. Differences, all deliberate:

* ``kvcache_block_size`` defaults to 16 and accepts any multiple of 16 (the reference
  requires a multiple of 256 because of its attention library).
* ``load_format="dummy"`` builds random-initialised weights on the device without
  touching disk (benchmarks with synthetic weights); ``"auto"`` reads safetensors.
* ``device="cpu"`` runs the pure-PyTorch oracle ops on gloo; it is what the CPU tests use.
* The model configuration is read from ``config.json`` directly, so importing this
  module does not import ``transformers``.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from types import SimpleNamespace
from typing import Any

__all__ = ["EngineConfig", "ModelConfig", "load_model_config", "QWEN3_ARCHS"]

PREFIX_BACKENDS = ("none", "hash", "radix")


class ModelConfig(SimpleNamespace):
    """Attribute view over a Hugging Face ``config.json`` for dense Qwen3."""

    def get(self, key: str, default: Any = None) -> Any:
        return getattr(self, key, default)

    def to_dict(self) -> dict:
        return dict(self.__dict__)


_QWEN3_DEFAULTS = dict(
    model_type="qwen3",
    architectures=["Qwen3ForCausalLM"],
    hidden_act="silu",
    rms_norm_eps=1e-6,
    rope_theta=1000000.0,
    max_position_embeddings=40960,
    tie_word_embeddings=False,
    attention_bias=False,
    torch_dtype="bfloat16",
    vocab_size=151936,
    head_dim=128,
)

# Architectures named by the benchmark configs; weights are random for synthetic runs.
QWEN3_ARCHS: dict[str, dict] = {
    "tiny": dict(num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
                 head_dim=64, intermediate_size=768, vocab_size=1024, tie_word_embeddings=True,
                 max_position_embeddings=4096, torch_dtype="float32"),
    "Qwen3-0.6B": dict(num_hidden_layers=28, hidden_size=1024, num_attention_heads=16,
                       num_key_value_heads=8, intermediate_size=3072, tie_word_embeddings=True),
    "Qwen3-1.7B": dict(num_hidden_layers=28, hidden_size=2048, num_attention_heads=16,
                       num_key_value_heads=8, intermediate_size=6144, tie_word_embeddings=True),
    "Qwen3-4B": dict(num_hidden_layers=36, hidden_size=2560, num_attention_heads=32,
                     num_key_value_heads=8, intermediate_size=9728, tie_word_embeddings=True),
    "Qwen3-8B": dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32,
                     num_key_value_heads=8, intermediate_size=12288),
    "Qwen3-14B": dict(num_hidden_layers=40, hidden_size=5120, num_attention_heads=40,
                      num_key_value_heads=8, intermediate_size=17408),
    "Qwen3-32B": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
                      num_key_value_heads=8, intermediate_size=25600),
}


def qwen3_arch_config(name: str, **overrides: Any) -> dict:
    """Full ``config.json`` dictionary for a named Qwen3 architecture."""
    if name not in QWEN3_ARCHS:
        raise KeyError(f"unknown Qwen3 architecture {name!r}; known: {sorted(QWEN3_ARCHS)}")
    cfg = dict(_QWEN3_DEFAULTS)
    cfg.update(QWEN3_ARCHS[name])
    cfg.update(overrides)
    return cfg


def load_model_config(model_dir: str) -> ModelConfig:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{path} not found: a model directory needs a config.json")
    with open(path, encoding="utf-8") as f:
        raw = json.load(f)
    merged = dict(_QWEN3_DEFAULTS)
    merged.update(raw)
    if "head_dim" not in raw or raw["head_dim"] is None:
        merged["head_dim"] = merged["hidden_size"] // merged["num_attention_heads"]
    if "dtype" in raw and "torch_dtype" not in raw:  # newer HF writers use "dtype"
        merged["torch_dtype"] = raw["dtype"]
    rope = raw.get("rope_parameters") or {}
    if "rope_theta" not in raw and "rope_theta" in rope:
        merged["rope_theta"] = rope["rope_theta"]
    return ModelConfig(**merged)


@dataclass
class EngineConfig:
    """All engine knobs. ``dp_size`` replicas each own a ``tp_size * pp_size`` rank world."""

    model: str

    # scheduler
    context_len: int = 4096
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 8192
    mix_prefill_decode: bool = True

    # memory
    kvcache_block_size: int = 16
    gpu_memory_utilization: float = 0.9
    num_kvcache_blocks: int = 0
    prefix_backend: str = "hash"

    # execution
    enforce_eager: bool = True       # False: decode steps replay CUDA graphs
    torch_compile: bool = False      # accepted for CLI compatibility; no compiler is used
    compile_mode: str = "reduce-overhead"
    compile_dynamic: bool = True
    dtype: str = "auto"

    # parallelism
    tp_size: int = 1
    pp_size: int = 1
    dp_size: int = 1
    nccl_port: int = 29500
    master_addr: str = "127.0.0.1"
    master_port: int = 29500
    device_ids: list[int] | None = None
    nccl_ifname: str = ""
    pp_layer_counts: list[int] | None = None

    # additions over the reference
    load_format: str = "auto"        # "auto" = safetensors, "dummy" = random init on device
    device: str = "cuda"             # "cpu" runs the oracle ops over gloo
    seed: int = 0
    tp_comm: str = "auto"            # "auto" | "fused" | "nccl": tensor-parallel reduction path
    dp_ready_timeout_s: float = 0.0  # 0 = scale with model size
    pp_microbatches: int = 1         # pipeline stages work on this many pieces of a step in turn (1 = lockstep)
    # "on": step n + 1 is scheduled, staged and launched before step n's samples are read (the host's work
    # overlaps the GPU's; outputs arrive one step() call later). "auto": on for CUDA without pipeline stages.
    async_scheduling: str = "auto"

    hf_config: ModelConfig = field(init=False, repr=False)

    @property
    def one_step_late(self) -> bool:
        env = os.environ.get("XV_ASYNC_SCHEDULING", "")
        if env in ("0", "1") and self.pp_size == 1:
            return env == "1"
        if self.async_scheduling == "auto":
            return self.device == "cuda" and self.pp_size == 1
        return self.async_scheduling == "on"

    def __post_init__(self) -> None:
        self.model = os.path.expanduser(self.model)
        if not os.path.isdir(self.model):
            raise FileNotFoundError(
                f"Model path not found: {self.model}. Use a local directory that holds config.json."
            )
        if self.kvcache_block_size < 16 or self.kvcache_block_size % 16 != 0:
            raise ValueError("kvcache_block_size must be a positive multiple of 16")
        if self.prefix_backend not in PREFIX_BACKENDS:
            raise ValueError(f"prefix_backend must be none|hash|radix, got {self.prefix_backend!r}")
        if self.tp_size < 1 or self.pp_size < 1 or self.dp_size < 1:
            raise ValueError("tp_size / pp_size / dp_size must be >= 1")
        if self.max_num_seqs < 1 or self.max_num_batched_tokens < 1 or self.context_len < 1:
            raise ValueError("max_num_seqs / max_num_batched_tokens / context_len must be >= 1")
        if self.load_format not in ("auto", "dummy"):
            raise ValueError(f"load_format must be auto|dummy, got {self.load_format!r}")
        if self.device not in ("cuda", "cpu"):
            raise ValueError(f"device must be cuda|cpu, got {self.device!r}")
        if self.tp_comm not in ("auto", "fused", "nccl"):
            raise ValueError(f"tp_comm must be auto|fused|nccl, got {self.tp_comm!r}")
        if self.pp_microbatches < 1:
            raise ValueError("pp_microbatches must be >= 1")
        if self.async_scheduling not in ("auto", "on", "off"):
            raise ValueError(f"async_scheduling must be auto|on|off, got {self.async_scheduling!r}")
        if self.async_scheduling == "on" and self.pp_size > 1:
            raise ValueError("async_scheduling=on needs pp_size == 1: the first pipeline stage gets its input "
                             "tokens from the host")
        self.hf_config = load_model_config(self.model)
        if self.pp_layer_counts is not None:
            if len(self.pp_layer_counts) != self.pp_size:
                raise ValueError("pp_layer_counts needs one entry per pipeline stage")
            if sum(self.pp_layer_counts) != self.hf_config.num_hidden_layers:
                raise ValueError("pp_layer_counts must sum to the model's layer count")
        self.context_len = min(
            self.context_len, int(self.hf_config.get("max_position_embeddings", self.context_len))
        )

    @property
    def world_size(self) -> int:
        """Ranks inside one engine replica."""
        return self.tp_size * self.pp_size

    @property
    def num_gpus(self) -> int:
        return self.dp_size * self.tp_size * self.pp_size

    @property
    def block_size(self) -> int:
        return self.kvcache_block_size
