"""Single-node entry point (reference: run.py:36-292).

    python run.py                       # one prompt, settings from config.yaml
    python run.py --cg                  # decode with CUDA graphs
    python run.py --batch               # four-prompt batch demo
    python run.py --tp 4 --dp 2         # tensor / pipeline / data parallel
    python run.py --prefix-backend radix
"""

from __future__ import annotations

import argparse
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
if str(HERE) not in sys.path:
    sys.path.insert(0, str(HERE))

from xixi_vllm_b200 import Engine, SamplingParams  # noqa: E402
from xixi_vllm_b200.model_hub import resolve_model_path  # noqa: E402
from xixi_vllm_b200.utils.run_utils import (DEFAULTS, cuda_sync, drain_engine, engine_config_from,  # noqa: E402
                                            handle_hub_cli, load_config, merge_cli, print_bench_report,
                                            warmup_engine)

BATCH_PROMPTS = ["Hello, my name is", "Once upon a time", "The capital of France is", "In machine learning,"]


def _make_engine(cfg: dict) -> Engine:
    model_path = resolve_model_path(cfg["model"])
    print(f"Loading {model_path} ...")
    return Engine(engine_config_from(cfg, model_path))


def _warmup(engine: Engine, prompt_lens: list[int]) -> float:
    sp = SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True)
    return warmup_engine(prompt_lens, add_request=engine.add_request,
                         drain=lambda: drain_engine(lambda: not engine.has_unfinished(), engine.step),
                         sync=cuda_sync, sampling_params=sp,
                         vocab_size=getattr(getattr(engine, "config", None), "hf_config", None)
                         and engine.config.hf_config.vocab_size)


def _timed_run(engine: Engine, seqs) -> tuple[float | None, float, float | None]:
    cuda_sync()
    t0 = time.perf_counter()
    t_first = None
    while any(not s.is_finished for s in seqs):
        engine.step()
        if t_first is None and any(s.num_known_completion_tokens > 0 for s in seqs):
            cuda_sync()
            t_first = time.perf_counter()
    cuda_sync()
    t_end = time.perf_counter()
    ttft = None if t_first is None else t_first - t0
    return ttft, t_end - t0, None if t_first is None else t_end - t_first


def run_single(cfg: dict) -> None:
    engine = _make_engine(cfg)
    try:
        prompt = cfg["prompt"]
        ids = list(prompt) if isinstance(prompt, list) else engine.tokenizer.encode(prompt)
        warmup_s = _warmup(engine, [len(ids)])
        sp = SamplingParams(temperature=cfg["temperature"], top_p=cfg["top_p"], top_k=cfg["top_k"],
                            max_tokens=cfg["max_new_tokens"])
        seq = engine.add_request(ids, sp)
        ttft, e2e, decode_s = _timed_run(engine, [seq])
        completion = seq.token_ids[seq.num_prompt_tokens:]
        print(f"Prompt: {prompt}")
        print(f"{prompt}{engine.tokenizer.decode(completion)}")
        print_bench_report(ttft, len(completion), e2e, decode_s=decode_s, warmup_s=warmup_s)
    finally:
        engine.destroy()


def run_batch(cfg: dict) -> None:
    engine = _make_engine(cfg)
    try:
        encoded = [engine.tokenizer.encode(p) for p in BATCH_PROMPTS]
        warmup_s = _warmup(engine, [len(e) for e in encoded])
        sp = SamplingParams(temperature=0.0, max_tokens=cfg["max_new_tokens"])
        seqs = [engine.add_request(e, sp) for e in encoded]
        ttft, e2e, decode_s = _timed_run(engine, seqs)
        n = 0
        for p, s in zip(BATCH_PROMPTS, seqs):
            ids = s.token_ids[s.num_prompt_tokens:]
            n += len(ids)
            print(f"\n>>> {p}\n{engine.tokenizer.decode(ids)}")
        print_bench_report(ttft, n, e2e, decode_s=decode_s, warmup_s=warmup_s)
        print(f"Batch:  {len(BATCH_PROMPTS)} reqs, {n} completion tokens")
    finally:
        engine.destroy()


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="B200-native Qwen3 engine: paged attention, CUDA graphs, continuous batching")
    p.add_argument("--config", default=None, help="YAML file (default: config.yaml next to this script)")
    p.add_argument("--model", default=None)
    p.add_argument("--prompt", default=None)
    p.add_argument("--max-new-tokens", type=int, default=None)
    p.add_argument("--temperature", type=float, default=None)
    p.add_argument("--top-p", type=float, default=None)
    p.add_argument("--top-k", type=int, default=None)
    g = p.add_mutually_exclusive_group()
    g.add_argument("--cg", action="store_true", help="decode with CUDA graphs")
    g.add_argument("--eager", action="store_true", help="no CUDA graphs")
    g = p.add_mutually_exclusive_group()
    g.add_argument("--compile", action="store_true", help="accepted for compatibility (no compiler on the hot path)")
    g.add_argument("--no-compile", action="store_true")
    p.add_argument("--compile-mode", choices=("default", "reduce-overhead", "max-autotune"), default=None)
    p.add_argument("--compile-dynamic", action="store_true")
    p.add_argument("--no-compile-dynamic", action="store_true")
    p.add_argument("--prefix-backend", choices=("none", "hash", "radix"), default=None)
    p.add_argument("--max-num-seqs", type=int, default=None)
    p.add_argument("--tp", type=int, default=None, help="tensor-parallel degree")
    p.add_argument("--pp", type=int, default=None, help="pipeline-parallel degree")
    p.add_argument("--dp", type=int, default=None, help="data-parallel replicas")
    p.add_argument("--pp-layer-counts", type=str, default=None, help="layers per stage, comma separated")
    p.add_argument("--pp-microbatches", type=int, default=None,
                   help="pipeline stages work on this many pieces of a step in turn (default 1: lockstep)")
    p.add_argument("--device-ids", type=str, default=None, help="GPU ids, comma separated (dp*tp*pp entries)")
    p.add_argument("--load-format", choices=("auto", "dummy"), default=None)
    p.add_argument("--device", choices=("cuda", "cpu"), default=None)
    p.add_argument("--tp-comm", choices=("auto", "fused", "nccl"), default=None)
    p.add_argument("--async-scheduling", choices=("auto", "on", "off"), default=None,
                   help="launch step n+1 before step n's samples are read (auto: on for CUDA without pipeline stages)")
    p.add_argument("--batch", action="store_true", help="run the four-prompt batch demo")
    p.add_argument("--download", action="store_true")
    p.add_argument("--list", action="store_true")
    return p


def config_from_args(args) -> dict:
    path = Path(args.config) if args.config else HERE / "config.yaml"
    cfg = load_config(path, DEFAULTS)
    merge_cli(cfg, args, ("model", "prompt", "max_new_tokens", "temperature", "top_p", "top_k", "prefix_backend",
                          "max_num_seqs", "load_format", "device", "tp_comm", "async_scheduling"))
    for flag, key in (("tp", "tp_size"), ("pp", "pp_size"), ("dp", "dp_size")):
        if getattr(args, flag) is not None:
            cfg[key] = getattr(args, flag)
    if args.pp_layer_counts is not None:
        cfg["pp_layer_counts"] = [int(x) for x in args.pp_layer_counts.split(",")]
    if args.pp_microbatches is not None:
        cfg["pp_microbatches"] = args.pp_microbatches
    if args.device_ids is not None:
        cfg["device_ids"] = [int(x) for x in args.device_ids.split(",")]
    if args.cg:
        cfg["enforce_eager"] = False
    if args.eager:
        cfg["enforce_eager"] = True
    if args.compile:
        cfg["torch_compile"] = True
    if args.no_compile:
        cfg["torch_compile"] = False
    if args.compile_mode:
        cfg["compile_mode"] = args.compile_mode
    if args.compile_dynamic:
        cfg["compile_dynamic"] = True
    if args.no_compile_dynamic:
        cfg["compile_dynamic"] = False
    return cfg


def main(argv=None) -> None:
    args = build_parser().parse_args(argv)
    if handle_hub_cli(args):
        return
    cfg = config_from_args(args)
    (run_batch if args.batch else run_single)(cfg)


if __name__ == "__main__":
    main()
