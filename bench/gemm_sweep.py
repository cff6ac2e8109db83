"""Sweep of the tcgen05 GEMM's kernel / tile / split-K choices on the serving shapes, next to cuBLAS.

    python -m bench.gemm_sweep [--json out/gemm_sweep.jsonl] [--set decode,tp8,mixed,prefill]

For every shape it times the planner's own choice and a grid of forced plans (``xv_gemm_plan_override``:
single-CTA swapped kernel with 1-8 K splits, CTA-pair kernel with tile widths 64-256 and several deals of K
blocks to the SM pairs), each with CUDA events after warm-up and an L2 flush between timed launches. The planner's
cost constants in ``gemm_sm100.cu`` are fitted to this table.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from bench.kernels import timeit  # noqa: E402
from xixi_vllm_b200.ops import cuda  # noqa: E402

SETS = {
    # Qwen3-8B, one GPU, 256 decode rows
    "decode": [(256, 6144, 4096), (256, 4096, 4096), (256, 24576, 4096), (256, 4096, 12288), (128, 6144, 4096),
               (192, 24576, 4096)],
    # one rank's shard at TP=8 (8B) and TP=8 (32B)
    "tp8": [(256, 768, 4096), (256, 4096, 512), (256, 3072, 4096), (256, 4096, 1536), (256, 1280, 5120),
            (256, 5120, 1024), (256, 6400, 5120), (256, 5120, 3200)],
    # a decode batch plus one prefill chunk
    "mixed": [(1400, 6144, 4096), (1400, 4096, 4096), (1400, 24576, 4096), (1400, 4096, 12288), (700, 4096, 4096),
              (2304, 6144, 4096), (1400, 768, 4096), (1400, 4096, 512), (1400, 3072, 4096), (1400, 4096, 1536),
              (384, 6144, 4096), (832, 4096, 4096), (1100, 4096, 4096), (512, 4096, 12288)],
    "prefill": [(4096, 6144, 4096), (4096, 4096, 4096), (4096, 24576, 4096), (4096, 4096, 12288), (8192, 8192, 8192)],
}


def configs(m: int, n: int, k: int):
    """(label, kind, bn, splits-or-units). For the pair kernel the last value is the number of K blocks dealt
    to each SM pair: 0 = an even deal (stream-K), -1 = whole tiles only."""
    yield ("auto", -1, 0, 0)
    if m <= 256:
        for sp in (1, 2, 3, 4, 8):
            yield ("swapped", 0, 0, sp)
    kb = k // 64
    for bn in (0, 64, 128, 192, 256):
        if bn > max(64, n):
            continue
        for units in (0, -1, kb // 2, kb // 4, kb // 8):
            if units > 0 and units < 2:
                continue
            yield ("pair", 2, bn, units)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default="")
    ap.add_argument("--set", default="decode,tp8,mixed,prefill")
    ap.add_argument("--iters", type=int, default=8)
    a = ap.parse_args()
    out = open(a.json, "w") if a.json else None
    for name in a.set.split(","):
        for m, n, k in SETS[name]:
            x = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
            w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
            ref = (x.float() @ w.float().t())
            t_cublas = timeit(lambda: torch.matmul(x, w.t()), iters=a.iters)
            rows = []
            for label, kind, bn, sp in configs(m, n, k):
                cuda.gemm_plan_override(kind, bn, sp, 0)
                try:
                    pl = cuda.gemm_plan(m, n, k, 148)
                    y = cuda.linear(x, w)
                    torch.cuda.synchronize()
                    cuda.check_status()
                    err = float((y.float() - ref).abs().max() / ref.abs().max())
                    ms = timeit(lambda: cuda.linear(x, w), iters=a.iters)
                except RuntimeError as e:
                    rows.append((label, bn, sp, None, str(e)[:60]))
                    continue
                finally:
                    cuda.gemm_plan_override(-1)
                spu = pl.units_per_pair if pl.pair else pl.splits
                rows.append((label, pl.bn, spu, ms, f"err {err:.1e} stages {pl.stages} tiles {pl.tiles_a}x{pl.tiles_b}"))
                if out:
                    out.write(json.dumps(dict(set=name, m=m, n=n, k=k, label=label, bn=pl.bn, splits=spu,
                                              pair=pl.pair, swapped=pl.swapped, ms=ms, cublas_ms=t_cublas,
                                              rel_err=err)) + "\n")
                    out.flush()
            good = [r for r in rows if r[3] is not None]
            best = min(good, key=lambda r: r[3]) if good else ("none", 0, 0, float("nan"), "")
            auto = rows[0]
            print(f"{name} {m}x{n}x{k}: cublas {t_cublas * 1e3:7.1f} us | auto {auto[3] * 1e3:7.1f} us "
                  f"({auto[0]} bn {auto[1]} sp {auto[2]}) | best {best[3] * 1e3:7.1f} us ({best[0]} bn {best[1]} sp {best[2]}) "
                  f"| cublas/auto {t_cublas / auto[3]:.2f} cublas/best {t_cublas / best[3]:.2f}", flush=True)
            for r in sorted(good, key=lambda r: r[3])[:6]:
                print(f"      {r[0]:8s} bn {r[1]:3d} sp {r[2]} {r[3] * 1e3:8.1f} us  {r[4]}")
            for r in rows:
                if r[3] is None:
                    print(f"      {r[0]:8s} bn {r[1]:3d} sp {r[2]}  failed: {r[4]}")
            del x, w, ref
    if out:
        out.close()


if __name__ == "__main__":
    main()
