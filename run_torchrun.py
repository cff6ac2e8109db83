"""torchrun entry point: one process per GPU, tensor x pipeline parallel, single or multi node
(reference: run_torchrun.py:37-199).

    torchrun --nproc_per_node 8 --master-addr 127.0.0.1 run_torchrun.py --tp 8 --cg
    torchrun --nnodes 2 --nproc_per_node 8 ... run_torchrun.py --tp 8 --pp 2

Rank 0 drives the engine; the other ranks serve broadcast commands until shutdown.
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
if str(HERE) not in sys.path:
    sys.path.insert(0, str(HERE))

from xixi_vllm_b200 import SamplingParams  # noqa: E402
from xixi_vllm_b200.control.torchrun import env_rank_info, launch_from_env, shutdown_from_env  # noqa: E402
from xixi_vllm_b200.model_hub import resolve_model_path  # noqa: E402
from xixi_vllm_b200.utils.run_utils import DEFAULTS, engine_config_from, load_config, merge_cli  # noqa: E402


def _run_driver(engine, cfg: dict) -> None:
    prompt = cfg["prompt"]
    sp = SamplingParams(temperature=cfg["temperature"], top_p=cfg["top_p"], top_k=cfg["top_k"],
                        max_tokens=cfg["max_new_tokens"])
    seq = engine.add_request(prompt, sp)
    while not seq.is_finished:
        engine.step()
    print(f"Prompt: {prompt}")
    print(f"{prompt}{engine.tokenizer.decode(seq.token_ids[seq.num_prompt_tokens:])}")


def main(argv=None) -> None:
    p = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    p.add_argument("--config", default=None)
    p.add_argument("--model", default=None)
    p.add_argument("--tp", type=int, default=None)
    p.add_argument("--pp", type=int, default=None)
    p.add_argument("--prompt", default=None)
    p.add_argument("--max-new-tokens", type=int, default=None)
    p.add_argument("--temperature", type=float, default=None)
    p.add_argument("--top-p", type=float, default=None)
    p.add_argument("--top-k", type=int, default=None)
    p.add_argument("--cg", action="store_true")
    p.add_argument("--compile", action="store_true", help="accepted for compatibility")
    p.add_argument("--pp-layer-counts", type=str, default=None)
    p.add_argument("--pp-microbatches", type=int, default=None,
                   help="pipeline stages work on this many pieces of a step in turn (default 1: lockstep)")
    p.add_argument("--device-ids", type=str, default=None)
    p.add_argument("--load-format", choices=("auto", "dummy"), default=None)
    p.add_argument("--device", choices=("cuda", "cpu"), default=None)
    p.add_argument("--tp-comm", choices=("auto", "fused", "nccl"), default=None)
    p.add_argument("--async-scheduling", choices=("auto", "on", "off"), default=None,
                   help="launch step n+1 before step n's samples are read (auto: on for CUDA without pipeline stages)")
    args = p.parse_args(argv)

    cfg = load_config(Path(args.config) if args.config else HERE / "config.yaml", DEFAULTS)
    merge_cli(cfg, args, ("model", "prompt", "max_new_tokens", "temperature", "top_p", "top_k", "load_format",
                          "device", "tp_comm", "async_scheduling"))
    rank, _, world = env_rank_info()
    cfg["tp_size"] = args.tp if args.tp is not None else cfg["tp_size"]
    cfg["pp_size"] = args.pp if args.pp is not None else cfg["pp_size"]
    cfg["dp_size"] = 1
    if cfg["tp_size"] * cfg["pp_size"] != world:
        raise SystemExit(f"tp({cfg['tp_size']}) * pp({cfg['pp_size']}) must equal WORLD_SIZE={world}")
    if args.cg:
        cfg["enforce_eager"] = False
    if args.compile:
        cfg["torch_compile"] = True
    if args.pp_layer_counts is not None:
        cfg["pp_layer_counts"] = [int(x) for x in args.pp_layer_counts.split(",")]
    if args.pp_microbatches is not None:
        cfg["pp_microbatches"] = args.pp_microbatches
    if args.device_ids is not None:
        cfg["device_ids"] = [int(x) for x in args.device_ids.split(",")]
    engine = launch_from_env(engine_config_from(cfg, resolve_model_path(cfg["model"])))
    if engine is None:
        return
    try:
        _run_driver(engine, cfg)
    finally:
        if world > 1:
            shutdown_from_env(engine)
        else:
            engine.destroy()


if __name__ == "__main__":
    main()
