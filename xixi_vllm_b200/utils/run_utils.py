"""Helpers shared by the command-line entry points (reference: src/utils/run_utils.py:26-125).

Defaults live in ONE dictionary used by both CLIs (the reference keeps two copies whose
values drifted apart). Precedence, lowest to highest: ``DEFAULTS``, the YAML file, CLI flags.
"""

from __future__ import annotations

import time
from collections.abc import Callable
from pathlib import Path
from typing import Any

__all__ = ["DEFAULTS", "cuda_sync", "drain_engine", "dummy_token_ids", "engine_config_from", "handle_hub_cli",
           "load_config", "merge_cli", "print_bench_report", "warmup_engine"]

_WARMUP_ITERS = 3

DEFAULTS: dict[str, Any] = {
    "model": "Qwen3-0.6B", "prompt": "Hello, my name is", "max_new_tokens": 200, "temperature": 0.9,
    "top_p": 0.95, "top_k": 20, "enforce_eager": True, "torch_compile": False,
    "compile_mode": "reduce-overhead", "compile_dynamic": True, "dtype": "auto", "context_len": 4096,
    "max_num_seqs": 256, "max_num_batched_tokens": 8192, "mix_prefill_decode": True,
    "kvcache_block_size": 16, "prefix_backend": "hash", "gpu_memory_utilization": 0.9,
    "num_kvcache_blocks": 0, "tp_size": 1, "pp_size": 1, "dp_size": 1, "pp_layer_counts": None,
    "device_ids": None, "nccl_port": 29500, "master_addr": "127.0.0.1", "master_port": 29500,
    "nccl_ifname": "", "load_format": "auto", "device": "cuda", "tp_comm": "auto", "seed": 0, "pp_microbatches": 1,
    "async_scheduling": "auto",
}

_ENGINE_KEYS = ("enforce_eager", "torch_compile", "compile_mode", "compile_dynamic", "dtype", "context_len",
                "max_num_seqs", "max_num_batched_tokens", "mix_prefill_decode", "kvcache_block_size",
                "prefix_backend", "gpu_memory_utilization", "num_kvcache_blocks", "tp_size", "pp_size",
                "dp_size", "pp_layer_counts", "device_ids", "nccl_port", "master_addr", "master_port",
                "nccl_ifname", "load_format", "device", "tp_comm", "seed", "pp_microbatches", "async_scheduling")


def load_config(path: Path, defaults: dict | None = None) -> dict:
    """YAML values for keys that exist in ``defaults``; unknown keys are ignored."""
    defaults = DEFAULTS if defaults is None else defaults
    cfg: dict = {}
    if Path(path).is_file():
        import yaml

        with open(path, encoding="utf-8") as f:
            cfg = yaml.safe_load(f) or {}
    return {k: cfg.get(k, v) for k, v in defaults.items()}


def merge_cli(cfg: dict, args: Any, keys: tuple[str, ...]) -> None:
    for key in keys:
        v = getattr(args, key, None)
        if v is not None:
            cfg[key] = v


def engine_config_from(cfg: dict, model_path: str):
    from ..config import EngineConfig

    return EngineConfig(model=str(model_path), **{k: cfg[k] for k in _ENGINE_KEYS if k in cfg})


def handle_hub_cli(args: Any) -> bool:
    """``--list`` / ``--download``; True when the command was handled."""
    if not getattr(args, "list", False) and not getattr(args, "download", False):
        return False
    from ..model_hub import (DEFAULT_CACHE_DIR, QWEN3_REGISTRY, download_models, gpu_memory_gb,
                             select_models_for_vram)

    if args.list:
        vram = gpu_memory_gb() or 180.0
        print(f"Cache: {DEFAULT_CACHE_DIR}")
        print(f"VRAM:  {vram:.1f} GB")
        print(f"All:   {', '.join(s.local_name for s in QWEN3_REGISTRY)}")
        print(f"Fit:   {', '.join(s.local_name for s in select_models_for_vram(vram))}")
        return True
    print(f"Downloading to {DEFAULT_CACHE_DIR} ...")
    download_models(getattr(args, "download_specs", None))
    print("Done.")
    return True


def cuda_sync() -> None:
    import torch

    if torch.cuda.is_available():
        torch.cuda.synchronize()


def dummy_token_ids(n: int, salt: int = 0) -> list[int]:
    """Deterministic pseudo-random ids (same formula as the reference, so workloads line up)."""
    n = max(1, n)
    return [((i * 7919 + 10007 + salt * 97) % 100000) + 100 for i in range(n)]


def drain_engine(is_finished: Callable[[], bool], step: Callable[[], Any]) -> None:
    while not is_finished():
        step()


def warmup_engine(prompt_lens: list[int], *, add_request: Callable, drain: Callable[[], None],
                  sync: Callable[[], None], sampling_params: Any, iters: int = _WARMUP_ITERS,
                  vocab_size: int | None = None) -> float:
    """Runs ``iters`` rounds of dummy prompts of the given lengths; returns the seconds spent."""
    sync()
    t0 = time.perf_counter()
    for it in range(iters):
        for n in prompt_lens:
            ids = dummy_token_ids(n, salt=it * 31 + n)
            if vocab_size:
                ids = [i % vocab_size for i in ids]
            add_request(ids, sampling_params)
        drain()
    sync()
    return time.perf_counter() - t0


def print_bench_report(ttft_s: float | None, n: int, e2e_s: float, *, decode_s: float | None = None,
                       warmup_s: float | None = None) -> None:
    print()
    if warmup_s is not None:
        print(f"Warmup: {warmup_s:.2f}s  (graph capture and first launches, excluded)")
    if ttft_s is not None:
        print(f"TTFT:   {ttft_s * 1000:.1f} ms")
    n_dec = max(0, n - 1)
    if decode_s is not None and decode_s > 0 and n_dec > 0:
        print(f"Decode: {n_dec} tokens in {decode_s:.3f}s ({n_dec / decode_s:.1f} tok/s)")
    elif n_dec == 0:
        print("Decode: (no tokens after the first; raise max_new_tokens)")
    if e2e_s > 0:
        print(f"E2E:    {n} tokens in {e2e_s:.3f}s ({n / e2e_s:.1f} tok/s)")
