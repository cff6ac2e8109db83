"""Latency / throughput cases in the style of the reference's bench scripts
(reference: bench/measure.py:19-105, bench/common.py:15-27, bench/bench_v4.py:65-86):

* ``single``  - one request: TTFT (submit -> first token) and decode tokens/s = (n-1)/(e2e-ttft)
* ``batch``   - N requests submitted together: total completion tokens / wall time
* ``decode``  - pure decode at a fixed batch size: per-step latency (TPOT) from CUDA events
* ``prefix``  - requests that share system prefixes (prefix-cache hit rate and throughput)

Each case appends one JSON record to ``--out`` (JSONL, same spirit as the reference's
``bench/out/bench.jsonl``); ``python -m bench.report`` renders the file as Markdown.

    python -m bench.serving --model Qwen3-8B --case decode --batch 1,32,256 [--tp 1] [--cg]
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PROMPT_LEN, OUTPUT_LEN, BATCH = 256, 128, 8       # the reference's bench constants


def make_engine(args, **over):
    from xixi_vllm_b200 import Engine, EngineConfig
    from xixi_vllm_b200.models.synth import make_model_dir

    d = os.path.join(tempfile.gettempdir(), f"xv_serving_{args.model}_{os.getuid()}")
    make_model_dir(d, args.model, weights=False)
    kw = dict(model=d, load_format="dummy", dtype="bfloat16", context_len=args.context_len,
              max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_batched_tokens,
              prefix_backend=args.prefix_backend, enforce_eager=not args.cg, tp_size=args.tp, pp_size=args.pp,
              dp_size=args.dp, gpu_memory_utilization=0.85)
    kw.update(over)
    return Engine(EngineConfig(**kw))


def _ids(n, salt, vocab):
    from xixi_vllm_b200.utils.run_utils import dummy_token_ids

    return [t % vocab for t in dummy_token_ids(n, salt)]


def _sync():
    import torch

    if torch.cuda.is_available():
        torch.cuda.synchronize()


def warmup(engine, vocab, rounds=3):
    from xixi_vllm_b200 import SamplingParams

    for r in range(rounds):
        engine.add_request(_ids(PROMPT_LEN, 900 + r, vocab), SamplingParams(max_tokens=4, ignore_eos=True))
        while engine.has_unfinished():
            engine.step()
    _sync()


def case_single(engine, args, vocab):
    from xixi_vllm_b200 import SamplingParams

    _sync()
    t0 = time.perf_counter()
    seq = engine.add_request(_ids(args.prompt_len, 1, vocab), SamplingParams(max_tokens=args.output_len, ignore_eos=True))
    t_first = None
    while not seq.is_finished:
        engine.step()
        if t_first is None and seq.num_known_completion_tokens > 0:
            _sync()
            t_first = time.perf_counter()
    _sync()
    e2e = time.perf_counter() - t0
    ttft = t_first - t0
    n = seq.num_known_completion_tokens
    return dict(case="single", ttft_ms=1e3 * ttft, decode_tps=(n - 1) / max(e2e - ttft, 1e-9),
                tpot_ms=1e3 * (e2e - ttft) / max(n - 1, 1), e2e_s=e2e, output_tokens=n)


def case_batch(engine, args, vocab):
    from xixi_vllm_b200 import SamplingParams

    _sync()
    t0 = time.perf_counter()
    seqs = [engine.add_request(_ids(args.prompt_len, 10 + i, vocab),
                               SamplingParams(max_tokens=args.output_len, ignore_eos=True)) for i in range(args.requests)]
    while engine.has_unfinished():
        engine.step()
    _sync()
    wall = time.perf_counter() - t0
    n = sum(s.num_known_completion_tokens for s in seqs)
    return dict(case="batch", requests=args.requests, batch_tps=n / wall, wall_s=wall, output_tokens=n)


def case_decode(engine, args, vocab, bs):
    """Steady decode at batch ``bs``: prefill everything, then time ``--decode-steps`` decode steps."""
    import torch

    from xixi_vllm_b200 import SamplingParams

    steps = args.decode_steps
    for i in range(bs):
        engine.add_request(_ids(args.prompt_len, 100 + i, vocab),
                           SamplingParams(max_tokens=steps + 16, ignore_eos=True))
    sched = engine.scheduler
    while sched.waiting:
        engine.step()
    for _ in range(4):
        engine.step()
    _sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        engine.step()
    e1.record()
    _sync()
    wall = time.perf_counter() - t0
    while engine.has_unfinished():
        engine.step()
    return dict(case="decode", batch=bs, context=args.prompt_len, tpot_ms=1e3 * wall / steps,
                tpot_ms_device_span=e0.elapsed_time(e1) / steps, decode_tps=bs * steps / wall)


def case_prefix(engine, args, vocab):
    """Requests share a few long system prefixes; reports hit rate and throughput."""
    import numpy as np

    from xixi_vllm_b200 import SamplingParams

    rng = np.random.default_rng(0)
    prefixes = [rng.integers(0, vocab, size=args.prefix_len).tolist() for _ in range(args.num_prefixes)]
    _sync()
    t0 = time.perf_counter()
    seqs = []
    for i in range(args.requests):
        p = prefixes[int(rng.integers(len(prefixes)))] + rng.integers(0, vocab, size=args.suffix_len).tolist()
        seqs.append(engine.add_request(p, SamplingParams(max_tokens=args.output_len, ignore_eos=True)))
    while engine.has_unfinished():
        engine.step()
    _sync()
    wall = time.perf_counter() - t0
    n = sum(s.num_known_completion_tokens for s in seqs)
    m = engine.metrics.summary() if args.dp == 1 else {}
    return dict(case="prefix", requests=args.requests, num_prefixes=args.num_prefixes, prefix_len=args.prefix_len,
                throughput_tps=n / wall, wall_s=wall, prefix_hit_rate=m.get("prefix_hit_rate"),
                ttft_ms_p50=m.get("ttft_ms_p50"))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="Qwen3-0.6B")
    ap.add_argument("--case", default="single,batch,decode")
    ap.add_argument("--batch", default="1,32,256", help="decode batch sizes")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN)
    ap.add_argument("--output-len", type=int, default=OUTPUT_LEN)
    ap.add_argument("--requests", type=int, default=BATCH)
    ap.add_argument("--decode-steps", type=int, default=64)
    ap.add_argument("--num-prefixes", type=int, default=8)
    ap.add_argument("--prefix-len", type=int, default=1536)
    ap.add_argument("--suffix-len", type=int, default=256)
    ap.add_argument("--context-len", type=int, default=4096)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-batched-tokens", type=int, default=8192)
    ap.add_argument("--prefix-backend", default="none")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--cg", action="store_true")
    ap.add_argument("--out", default=os.path.join(ROOT, "bench", "out", "bench.jsonl"))
    args = ap.parse_args()

    engine = make_engine(args)
    vocab = engine.config.hf_config.vocab_size
    records = []
    try:
        warmup(engine, vocab)
        for case in args.case.split(","):
            if case == "single":
                records.append(case_single(engine, args, vocab))
            elif case == "batch":
                records.append(case_batch(engine, args, vocab))
            elif case == "decode":
                for bs in [int(b) for b in args.batch.split(",")]:
                    records.append(case_decode(engine, args, vocab, min(bs, args.max_num_seqs)))
            elif case == "prefix":
                records.append(case_prefix(engine, args, vocab))
            else:
                raise SystemExit(f"unknown case {case}")
    finally:
        engine.destroy()
    os.makedirs(os.path.dirname(args.out), exist_ok=True)
    with open(args.out, "a", encoding="utf-8") as f:
        for r in records:
            r.update(ts=time.time(), model=args.model, tp=args.tp, pp=args.pp, dp=args.dp, cuda_graph=args.cg,
                     prefix_backend=args.prefix_backend, prompt_len=args.prompt_len)
            f.write(json.dumps(r) + "\n")
            print(json.dumps(r), flush=True)


if __name__ == "__main__":
    main()
