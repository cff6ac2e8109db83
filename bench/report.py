"""Renders ``bench/out/bench.jsonl`` (records written by ``bench.serving``) as Markdown tables
(reference: bench/report.py:44-98).

    python -m bench.report [--in bench/out/bench.jsonl]
"""

from __future__ import annotations

import argparse
import json
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
COLUMNS = {
    "single": ["model", "tp", "cuda_graph", "prompt_len", "ttft_ms", "tpot_ms", "decode_tps"],
    "batch": ["model", "tp", "cuda_graph", "requests", "batch_tps", "wall_s"],
    "decode": ["model", "tp", "cuda_graph", "batch", "context", "tpot_ms", "decode_tps"],
    "prefix": ["model", "tp", "dp", "prefix_backend", "requests", "prefix_hit_rate", "throughput_tps", "ttft_ms_p50"],
}


def fmt(v):
    if isinstance(v, float):
        return f"{v:.3f}" if abs(v) < 100 else f"{v:.1f}"
    return str(v)


def render(records: list[dict]) -> str:
    out = []
    for case, cols in COLUMNS.items():
        rows = [r for r in records if r.get("case") == case]
        if not rows:
            continue
        out.append(f"### {case}\n")
        out.append("| " + " | ".join(cols) + " |")
        out.append("|" + "---|" * len(cols))
        for r in rows:
            out.append("| " + " | ".join(fmt(r.get(c, "")) for c in cols) + " |")
        out.append("")
    return "\n".join(out)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--in", dest="inp", default=os.path.join(ROOT, "bench", "out", "bench.jsonl"))
    a = ap.parse_args()
    with open(a.inp, encoding="utf-8") as f:
        records = [json.loads(line) for line in f if line.strip()]
    print(render(records))


if __name__ == "__main__":
    main()
