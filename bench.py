"""Serving benchmark: output tokens per second of continuous batching on Qwen3-8B.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--model Qwen3-8B]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Workload (synthetic: random-init bf16 weights of the named architecture, uniform random
token prompts): requests with prompt length U[256, 2048] and 512 output tokens each,
greedy, EOS ignored, continuous batching with at most 256 running sequences and 16384
batched tokens per step, tensor parallel over N GPUs.

A bench *step* is one engine step (schedule -> forward -> sample -> update). The engine is
first brought to the workload's steady state without timing: the running batch is filled and
the initial requests get staggered remaining lengths, so finished requests are replaced at
the steady rate (a replacement's whole prompt is prefilled in the same step as the other
sequences' decodes). Then W untimed warm-up steps run, then exactly K timed steps.

Two numbers come out of the timed region:
* ``value``   - output tokens / device time, where device time is the sum over the K steps of
                the CUDA-event time of each step's forward+sampling on the GPU (max over ranks);
* ``e2e``     - output tokens / wall time of the K ``Engine.step()`` calls, bracketed by a
                barrier and a device synchronise on both sides. Every step copies its inputs
                host->device from pinned memory and reads its sampled ids back device->host.

``--impl reference`` runs the unmodified reference engine installed under ``baseline/_ref``
through its own ``Engine`` API on the same workload and prints the same line with
``"impl": "reference"`` (its paged attention needs 256-token pages; ours uses 16).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "output_tokens_per_s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--mode", default="steady", choices=("steady", "full", "decode"),
                    help="steady: K timed engine steps of steady-state continuous batching (the headline); "
                         "full: --requests requests run to completion (output tok/s, TTFT, TPOT); "
                         "decode: --decode-batch sequences decoding together (time per output token)")
    ap.add_argument("--requests", type=int, default=512, help="requests of --mode full")
    ap.add_argument("--decode-batch", type=int, default=256, help="sequences of --mode decode")
    ap.add_argument("--decode-context", type=int, default=256, help="prompt length of --mode decode")
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--model", default="Qwen3-8B")
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-batched-tokens", type=int, default=16384)
    ap.add_argument("--prompt-min", type=int, default=256)
    ap.add_argument("--prompt-max", type=int, default=2048)
    ap.add_argument("--out-tokens", type=int, default=512)
    ap.add_argument("--eager", action="store_true", help="disable decode CUDA graphs")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--tp-comm", default="auto", choices=("auto", "fused", "nccl"),
                    help="tensor-parallel reduction path (fused peer-memory kernels or NCCL)")
    ap.add_argument("--emulate-tp", type=int, default=1,
                    help="single GPU, model dimensions cut to one rank's shard of this tensor-parallel degree "
                         "(compute share of a rank without any communication; diagnostic, not a benchmark)")
    ap.add_argument("--pp", type=int, default=1,
                    help="pipeline stages (must divide --gpus; the rest is tensor parallel). The headline is tp = gpus")
    ap.add_argument("--pp-microbatches", type=int, default=1, help="pieces of a step the stages work on in turn")
    ap.add_argument("--profile", action="store_true",
                    help="bracket the timed region with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    return ap.parse_args()


class Workload:
    """Endless stream of requests drawn from the benchmark's distribution."""

    def __init__(self, args, vocab: int) -> None:
        import numpy as np

        self.rng = np.random.default_rng(args.seed)
        self.args, self.vocab = args, vocab

    def next(self, staggered: bool):
        a = self.args
        n = int(self.rng.integers(a.prompt_min, a.prompt_max + 1))
        ids = self.rng.integers(0, self.vocab, size=n).tolist()
        out = int(self.rng.integers(1, a.out_tokens + 1)) if staggered else a.out_tokens
        return ids, out


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0) -> None:
        self.gpu_index = gpu_index
        self.lines: list[str] = []
        self.proc = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()           # the exact child we started
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def flush_l2(device) -> None:
    """Writes a buffer larger than the 126 MB L2 so the next step starts cold."""
    import torch

    if not hasattr(flush_l2, "buf"):
        flush_l2.buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    flush_l2.buf.zero_()


def emit(record: dict) -> None:
    print(json.dumps(record), flush=True)


def baseline_number(model: str = "Qwen3-8B", n_gpus: int = 1, mode: str = "steady"):
    """The reference publishes no numbers; the comparison figures are its own engine measured on B200s through
    ``--impl reference`` (``baseline/measured_reference.json``, keyed by model, GPU count and mode). None when that
    case was not measured."""
    path = os.path.join(ROOT, "baseline", "measured_reference.json")
    try:
        with open(path) as f:
            table = json.load(f)
        return table[model][mode][str(n_gpus)]["output_tokens_per_s"]
    except (OSError, KeyError, ValueError, TypeError):
        return None


def _known(sq) -> int:
    """Completion tokens whose value the host has (the reference's sequences have no tokens in flight)."""
    v = getattr(sq, "num_known_completion_tokens", None)
    return sq.num_completion_tokens if v is None else v


def run_to_completion(engine, make_sp, wl, n_requests: int, sync) -> dict:
    """``n_requests`` requests of the workload submitted at once and stepped until all are done, through the
    engine's public API (works for both arms). Output tokens per second of wall time, time to first token and
    time per output token after the first (host clock, per request)."""
    seqs = []
    for _ in range(n_requests):
        ids, out = wl.next(False)
        seqs.append(engine.add_request(ids, make_sp(out)))
    sync()
    t0 = time.perf_counter()
    first = [None] * len(seqs)
    done = [None] * len(seqs)
    steps = 0
    pending = set(range(len(seqs)))
    while engine.has_unfinished():
        engine.step()
        steps += 1
        now = time.perf_counter()
        for i in list(pending):
            sq = seqs[i]
            if first[i] is None and _known(sq) > 0:
                first[i] = now
            if sq.is_finished:
                done[i] = now
                pending.discard(i)
    sync()
    wall = time.perf_counter() - t0
    out_tokens = sum(_known(sq) for sq in seqs)
    ttft = sorted((f - t0) * 1e3 for f in first if f is not None)
    tpot = sorted((d - f) * 1e3 / max(1, _known(sq) - 1)
                  for f, d, sq in zip(first, done, seqs) if f is not None and d is not None)

    def pct(v, q):
        return v[min(len(v) - 1, int(q * len(v)))] if v else None

    return {"output_tokens": out_tokens, "wall_s": wall, "steps": steps, "value": out_tokens / wall,
            "ttft_ms": {"p50": pct(ttft, 0.5), "p99": pct(ttft, 0.99)},
            "decode_tpot_ms": {"p50": pct(tpot, 0.5), "p99": pct(tpot, 0.99)}}


def run_decode_only(engine, make_sp, vocab: int, batch: int, context: int, steps: int, warmup: int, sync, seed: int = 0) -> dict:
    """``batch`` sequences with ``context``-token prompts decoding together: wall time per engine step once every
    prompt has been prefilled = time per output token of each sequence."""
    import numpy as np

    rng = np.random.default_rng(seed)
    seqs = [engine.add_request(rng.integers(0, vocab, size=context).tolist(), make_sp(steps + warmup + 8))
            for _ in range(batch)]
    while any(_known(sq) == 0 for sq in seqs):
        engine.step()
    for _ in range(warmup):
        engine.step()
    sync()
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    sync()
    wall = time.perf_counter() - t0
    return {"decode_tpot_ms": 1e3 * wall / steps, "value": batch * steps / wall, "output_tokens": batch * steps,
            "wall_s": wall}


# ----------------------------------------------------------------------------------------------
# ours
# ----------------------------------------------------------------------------------------------
def run_ours(args) -> None:
    import torch

    os.environ["XV_TIME_STEPS"] = "1"
    from xixi_vllm_b200 import EngineConfig, SamplingParams
    from xixi_vllm_b200.control.torchrun import env_rank_info, launch_from_env, shutdown_from_env
    from xixi_vllm_b200.models.synth import make_model_dir
    from xixi_vllm_b200.ops import cuda

    rank, local_rank, world = env_rank_info()
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with --nproc-per-node {args.gpus}")
        raise SystemExit(f"WORLD_SIZE={world} does not match --gpus {args.gpus}")
    model_dir = os.path.join(tempfile.gettempdir(), f"xv_bench_{args.model}_{args.emulate_tp}_{os.getuid()}")
    if rank == 0:
        over = {}
        if args.emulate_tp > 1:
            from xixi_vllm_b200.config import qwen3_arch_config

            full = qwen3_arch_config(args.model)
            t = args.emulate_tp
            over = dict(num_attention_heads=full["num_attention_heads"] // t,
                        num_key_value_heads=max(1, full["num_key_value_heads"] // t),
                        intermediate_size=full["intermediate_size"] // t, vocab_size=full["vocab_size"] // t)
        make_model_dir(model_dir, args.model, weights=False, **over)
    context = args.prompt_max + args.out_tokens
    if args.mode == "decode":
        context = args.decode_context + args.steps + args.warmup + 16
        args.max_num_seqs = max(1, args.decode_batch)
    if args.tp_comm == "auto" and args.gpus // args.pp > 1:
        args.tp_comm = "fused"      # a broken peer-memory setup must fail loudly, not fall back to NCCL
    cfg_kwargs = dict(model=model_dir, load_format="dummy", dtype="bfloat16", context_len=context,
                      max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_batched_tokens,
                      kvcache_block_size=16, prefix_backend="none", enforce_eager=args.eager,
                      tp_size=args.gpus // args.pp, pp_size=args.pp, pp_microbatches=args.pp_microbatches,
                      seed=args.seed, gpu_memory_utilization=0.9, tp_comm=args.tp_comm)
    # rank 0 writes config.json before the others read it
    if world > 1:
        import torch.distributed as dist  # noqa: F401
        deadline = time.time() + 60
        while not os.path.isfile(os.path.join(model_dir, "config.json")) and time.time() < deadline:
            time.sleep(0.05)
    cfg = EngineConfig(**cfg_kwargs)
    engine = launch_from_env(cfg)
    if engine is None:      # ranks >= 1 served the driver until shutdown
        return

    device = torch.device("cuda", local_rank)
    wl = Workload(args, cfg.hf_config.vocab_size)
    core = engine._client.engine_core
    sched = core.scheduler
    comm = getattr(core.executor.worker.model, "comm", None)
    comm_ran = {"tp_comm_ran": "fused" if hasattr(comm, "symm") else ("nccl" if args.gpus // args.pp > 1 else "none"),
                "nvls_multicast": bool(getattr(comm, "mc_ptr", 0)),
                "one_kernel_row_parallel": bool(getattr(comm, "fuse_gemm", False))}
    parallelism = (f"tp{args.gpus}" if args.pp == 1 else f"tp{args.gpus // args.pp}pp{args.pp}mb{args.pp_microbatches}")

    def make_sp(n_out):
        return SamplingParams(temperature=0.0, max_tokens=n_out, ignore_eos=True)

    def sync():
        torch.cuda.synchronize(device)

    if args.mode != "steady":
        clocks = ClockSampler(local_rank)
        clocks.start()
        launches0 = cuda.launch_count
        if args.mode == "full":
            r = run_to_completion(engine, make_sp, wl, args.requests, sync)
            cfg_extra = {"requests": args.requests, "step": "all requests submitted at once and run to completion"}
        else:
            r = run_decode_only(engine, make_sp, cfg.hf_config.vocab_size, args.decode_batch, args.decode_context,
                                args.steps, args.warmup, sync, args.seed)
            cfg_extra = {"decode_batch": args.decode_batch, "decode_context": args.decode_context,
                         "step": "one decode step of the whole batch"}
        clk = clocks.stop()
        runner = core.executor.worker.model_runner
        rec = {"metric": METRIC, "value": r["value"], "unit": "tokens/s", "n_gpus": args.gpus, "steps": r.get("steps", args.steps),
               "warmup": args.warmup, "mode": args.mode, "higher_is_better": True, "scaling": "strong",
               "vs_baseline": (r["value"] / b) if (b := baseline_number(args.model, args.gpus, args.mode)) else None,
               "dtype": "bf16", "data": "synthetic (random-init weights, uniform random token prompts)", "impl": "ours",
               "timing": "wall clock around Engine.step() calls, device synchronised at both ends",
               "ttft_ms": r.get("ttft_ms"), "decode_tpot_ms": r.get("decode_tpot_ms"),
               "config": {"model": args.model, "global_batch": args.max_num_seqs, "seq_len": context,
                          "parallelism": parallelism, "kv_block_size": 16, "decode_cuda_graph": not args.eager,
                          "tp_comm": args.tp_comm, **comm_ran, **cfg_extra},
               "clocks": clk, "output_tokens": r["output_tokens"], "wall_s": r["wall_s"],
               "gpu_launches": cuda.launch_count - launches0 + (runner.graphs.replayed_kernels if runner.graphs else 0)}
        emit(rec)
        if world > 1:
            shutdown_from_env(engine)
        else:
            engine.destroy()
        return

    def top_up(staggered: bool) -> None:
        while len(sched.waiting) < 4:
            ids, out = wl.next(staggered)
            engine.add_request(ids, SamplingParams(temperature=0.0, max_tokens=out, ignore_eos=True))

    # fill phase (untimed): admit until the running batch is full
    top_up(True)
    while len(sched.running) < args.max_num_seqs:
        engine.step()
        top_up(True)
    for _ in range(args.warmup):
        top_up(False)
        engine.step()

    runner = core.executor.worker.model_runner
    clocks = ClockSampler(local_rank)
    torch.cuda.synchronize(device)
    first_step = sched._step + 1
    launches0 = cuda.launch_count + (runner.graphs.replayed_kernels if runner.graphs else 0)
    clocks.start()
    if args.profile:
        torch.cuda.profiler.start()
    out_tokens = 0
    h2d = d2h = 0
    step_ms = []
    torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        top_up(False)
        flush_l2(device)
        ts = time.perf_counter()
        before = core.metrics.sampled_tokens
        engine.step()
        out_tokens += core.metrics.sampled_tokens - before
        h2d += runner.h2d_bytes
        d2h += runner.d2h_bytes
        step_ms.append((time.perf_counter() - ts) * 1e3)
    torch.cuda.synchronize(device)
    wall = time.perf_counter() - t0
    if args.profile:
        torch.cuda.profiler.stop()
    clk = clocks.stop()
    launches = cuda.launch_count + (runner.graphs.replayed_kernels if runner.graphs else 0) - launches0
    # one-step-late scheduling: the timed calls read the steps launched one call earlier
    lag = 1 if getattr(core, "_inflight", None) is not None else 0
    dev_ms = core.executor.device_time_ms(first_step - lag, sched._step + 1 - lag)
    if lag:
        # One-step-late scheduling: a call launches step n + 1 and returns step n, and the GPU keeps working between
        # two calls, so only the whole loop is a fair clock: from the synchronised start to the synchronisation
        # after the last call it holds exactly `steps` forwards and `steps` steps' tokens (plus the L2 flushes
        # and the host's refill of the queue, which run while the GPU is busy).
        e2e_wall = wall
    else:
        e2e_wall = sum(step_ms) / 1e3        # Engine.step() wall time only (excludes the L2 flush)
    cuda.check_status(device)

    rec = {
        "metric": METRIC, "value": out_tokens / (dev_ms / 1e3), "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "mode": "steady",
        "vs_baseline": ((out_tokens / (dev_ms / 1e3)) / b) if (b := baseline_number(args.model, args.gpus)) else None,
        "dtype": "bf16",
        "data": "synthetic (random-init weights, uniform random token prompts)", "impl": "ours",
        "ttft_ms": {"p50": core.metrics.summary().get("ttft_ms_p50"), "note": "includes the untimed fill phase; see --mode full"},
        "decode_tpot_ms": {"pure_decode_step_ms_median": (sorted(step_ms)[len(step_ms) // 4] if step_ms else None),
                           "note": "lower quartile of the timed steps' wall time = a step without a prefill chunk"},
        "config": {"model": args.model, "global_batch": args.max_num_seqs, "seq_len": context,
                   "parallelism": parallelism, "prompt_len": f"U[{args.prompt_min},{args.prompt_max}]",
                   "output_len": args.out_tokens, "max_num_batched_tokens": args.max_batched_tokens,
                   "kv_block_size": 16, "decode_cuda_graph": not args.eager, "tp_comm": args.tp_comm, **comm_ran,
                   **({"emulate_tp_shard": args.emulate_tp} if args.emulate_tp > 1 else {}),
                   "l2": "flushed between timed steps (256 MiB write)",
                   "async_scheduling": bool(getattr(core, "one_step_late", False)),
                   "step": "one engine step in steady-state continuous batching"},
        "clocks": clk,
        "e2e": {"value": out_tokens / e2e_wall, "unit": "tokens/s", "h2d_bytes_per_step": h2d / args.steps,
                "d2h_bytes_per_step": d2h / args.steps, "ms_per_step": 1e3 * e2e_wall / args.steps,
                "wall_s_incl_flush": wall,
                "timed": ("whole timed loop incl. L2 flushes, synchronised at both ends (step n + 1 is launched "
                          "before step n is read)") if lag else "sum of Engine.step() wall times"},
        "gpu_launches": launches,
        "output_tokens": out_tokens,
        "engine": core.metrics.summary(),
    }
    emit(rec)
    if world > 1:
        shutdown_from_env(engine)
    else:
        engine.destroy()


# ----------------------------------------------------------------------------------------------
# reference
# ----------------------------------------------------------------------------------------------
def run_reference(args) -> None:
    ref_root = os.path.join(ROOT, "baseline")
    if not os.path.isfile(os.path.join(ref_root, "_ref", "control", "engine.py")):
        emit({"impl": "reference", "unavailable": "baseline/_ref is not installed (pip --target install of the reference package)"})
        return
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        # the reference's single-node path spawns its own tensor-parallel workers from rank 0
        return
    try:
        from baseline.ref_harness import run as run_ref

        rec = run_ref(args, Workload, ClockSampler, flush_l2, run_to_completion, run_decode_only)
    except Exception as e:  # the line must still be printed and the exit code stay 0
        emit({"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:300]}"})
        return
    rec.update({"metric": METRIC, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
                "warmup": args.warmup, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": 1.0 if baseline_number(args.model, args.gpus, args.mode) else None, "dtype": "bf16",
                "impl": "reference", "mode": args.mode,
                "data": "synthetic (random-init weights, uniform random token prompts)"})
    emit(rec)


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
