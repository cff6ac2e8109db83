"""Drives the reference engine through its own public API (``Engine`` / ``EngineConfig`` /
``SamplingParams`` of the package installed at ``baseline/_ref``) on the benchmark workload.
Nothing of this repository's engine, models or kernels is on that path; only the synthetic
model directory writer and the workload generator are shared.

Device time per step is taken by wrapping the in-process rank-0 ``ModelRunner.run_forward``
with CUDA events from the outside (the reference exposes host timing only).
"""

from __future__ import annotations

import os
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))


def run(args, Workload, ClockSampler, flush_l2, run_to_completion=None, run_decode_only=None) -> dict:
    import torch

    if HERE not in sys.path:
        sys.path.insert(0, HERE)
    env_dir = os.path.join(HERE, "ref_env")
    os.environ["PYTHONPATH"] = os.pathsep.join([env_dir, HERE, os.path.dirname(HERE), os.environ.get("PYTHONPATH", "")])
    # the same aliases ref_env/sitecustomize.py installs in the spawned workers
    import torch.distributed as dist

    if not hasattr(dist, "all_gather_single"):
        dist.all_gather_single = dist.all_gather_into_tensor
    if not hasattr(dist, "reduce_scatter_single"):
        dist.reduce_scatter_single = dist.reduce_scatter_tensor
    import _ref  # the reference package, unmodified

    from baseline.ref_model import make_reference_model_dir

    model_dir = make_reference_model_dir(
        os.path.join(tempfile.gettempdir(), f"xv_ref_{args.model}_{os.getuid()}"), args.model, seed=args.seed)
    context = args.prompt_max + args.out_tokens
    if getattr(args, "mode", "steady") == "decode":
        context = -(-(args.decode_context + args.steps + args.warmup + 16) // 256) * 256
        args.max_num_seqs = max(8, args.decode_batch)     # the reference engine hung with max_num_seqs = 1 under TP=2
    cfg = _ref.EngineConfig(
        model=model_dir, context_len=context, max_num_seqs=min(args.max_num_seqs, 256),
        max_num_batched_tokens=args.max_batched_tokens, kvcache_block_size=256, prefix_backend="none",
        enforce_eager=args.eager, torch_compile=False, dtype="bfloat16", tp_size=args.gpus,
        gpu_memory_utilization=0.9, nccl_port=29650)
    # transformers >= 5 keeps the rotary base under rope_parameters; the reference (pinned to
    # transformers < 5) reads config.rope_theta. Supplying the attribute adapts the environment,
    # not the reference.
    if not hasattr(cfg.hf_config, "rope_theta"):
        rope = getattr(cfg.hf_config, "rope_parameters", None) or {}
        cfg.hf_config.rope_theta = float(rope.get("rope_theta", 1000000.0))
    engine = _ref.Engine(cfg)
    try:
        sched = engine.scheduler
        wl = Workload(args, cfg.hf_config.vocab_size)
        SP = _ref.SamplingParams

        def top_up(staggered):
            while len(sched.waiting) < 4:
                ids, out = wl.next(staggered)
                engine.add_request(ids, SP(temperature=0.0, max_tokens=out, ignore_eos=True))

        mode = getattr(args, "mode", "steady")
        if mode != "steady":
            def make_sp(n_out):
                return SP(temperature=0.0, max_tokens=n_out, ignore_eos=True)

            clocks = ClockSampler(0)
            clocks.start()
            if mode == "full":
                r = run_to_completion(engine, make_sp, wl, args.requests, torch.cuda.synchronize)
                extra = {"requests": args.requests, "step": "all requests submitted at once and run to completion"}
            else:
                r = run_decode_only(engine, make_sp, cfg.hf_config.vocab_size, args.decode_batch, args.decode_context,
                                    args.steps, args.warmup, torch.cuda.synchronize, args.seed)
                extra = {"decode_batch": args.decode_batch, "decode_context": args.decode_context,
                         "step": "one decode step of the whole batch"}
            return {"value": r["value"], "ms_per_step": None, "ttft_ms": r.get("ttft_ms"),
                    "decode_tpot_ms": r.get("decode_tpot_ms"), "output_tokens": r["output_tokens"], "wall_s": r["wall_s"],
                    "timing": "wall clock around Engine.step() calls, device synchronised at both ends",
                    "config": {"model": args.model, "global_batch": cfg.max_num_seqs, "seq_len": context,
                               "parallelism": f"tp{args.gpus}", "kv_block_size": 256,
                               "decode_cuda_graph": not args.eager, **extra},
                    "clocks": clocks.stop(), "gpu_launches": None}
        runner = engine._client.engine_core.executor.worker.model_runner
        events = []
        inner = runner.run_forward

        def timed_forward(sched_out):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = inner(sched_out)
            e1.record()
            events.append((e0, e1))
            return r

        runner.run_forward = timed_forward

        def completed():
            return sum(s.num_completion_tokens for s in engine._seqs.values())

        top_up(True)
        while len(sched.running) < cfg.max_num_seqs:
            engine.step()
            top_up(True)
        for _ in range(args.warmup):
            top_up(False)
            engine.step()

        device = torch.device("cuda", 0)
        clocks = ClockSampler(0)
        torch.cuda.synchronize()
        events.clear()
        clocks.start()
        out_tokens, step_s = 0, 0.0
        t0 = time.perf_counter()
        for _ in range(args.steps):
            top_up(False)
            flush_l2(device)
            before = completed()
            ts = time.perf_counter()
            engine.step()
            step_s += time.perf_counter() - ts
            out_tokens += completed() - before
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        clk = clocks.stop()
        dev_ms = sum(a.elapsed_time(b) for a, b in events)
        return {
            "value": out_tokens / (dev_ms / 1e3), "ms_per_step": dev_ms / args.steps,
            "config": {"model": args.model, "global_batch": cfg.max_num_seqs, "seq_len": context,
                       "parallelism": f"tp{args.gpus}", "prompt_len": f"U[{args.prompt_min},{args.prompt_max}]",
                       "output_len": args.out_tokens, "max_num_batched_tokens": args.max_batched_tokens,
                       "kv_block_size": 256, "decode_cuda_graph": not args.eager,
                       "l2": "flushed between timed steps (256 MiB write)",
                       "device_time": "rank-0 forward only; other tensor-parallel ranks are separate processes"},
            "clocks": clk,
            "e2e": {"value": out_tokens / step_s, "unit": "tokens/s", "ms_per_step": 1e3 * step_s / args.steps,
                    "h2d_bytes_per_step": None, "d2h_bytes_per_step": None, "wall_s_incl_flush": wall},
            "gpu_launches": None, "output_tokens": out_tokens,
        }
    finally:
        engine.destroy()
