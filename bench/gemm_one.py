"""Runs one GEMM shape a few times (small, self-contained target for an ncu capture).

    python -m bench.gemm_one --m 256 --n 24576 --k 4096 [--iters 3]
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from xixi_vllm_b200.ops import cuda  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=256)
    ap.add_argument("--n", type=int, default=24576)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--no-pair", action="store_true", help="force the single-CTA kernel")
    a = ap.parse_args()
    if a.no_pair:
        cuda.lib().xv_gemm_disable_pair(1)
    x = torch.randn(a.m, a.k, device="cuda").bfloat16()
    w = torch.randn(a.n, a.k, device="cuda").bfloat16()
    for _ in range(a.iters):
        y = cuda.linear(x, w)
    torch.cuda.synchronize()
    cuda.check_status()
    ref = x.float() @ w.float().t()
    print("max err", float((y.float() - ref).abs().max()), "scale", float(ref.abs().max()))


if __name__ == "__main__":
    main()
