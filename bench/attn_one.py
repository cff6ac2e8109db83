"""Runs one paged-attention shape a few times (small, self-contained target for an ncu capture).

    python -m bench.attn_one --mode decode --batch 64 --len 1408 [--hq 32 --hkv 8 --iters 3]
    python -m bench.attn_one --mode prefill --batch 4 --len 2048
    python -m bench.attn_one --mode prefill --batch 4 --len 2048 --phases    # where the tcgen05 kernel's warps wait
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from bench.kernels import _attn_setup  # noqa: E402
from xixi_vllm_b200.ops import cpu_ref, cuda  # noqa: E402
from xixi_vllm_b200.runtime.staging import AttnBatch  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="decode", choices=("decode", "prefill"))
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--len", type=int, default=1408)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--block", type=int, default=16, help="tokens per KV page")
    ap.add_argument("--time", action="store_true", help="print the CUDA-event time of one more call")
    ap.add_argument("--phases", action="store_true",
                    help="prefill: run the instrumented kernel once and print cycles per phase and tile")
    ap.add_argument("--single-head", action="store_true",
                    help="prefill: one head per CTA instead of two heads of a KV group")
    a = ap.parse_args()
    if a.single_head:
        cuda.prefill_pair_heads(False)
    B, L = a.batch, a.len
    q_lens = [1] * B if a.mode == "decode" else [L] * B
    q, k, v, cu, kvl, bt = _attn_setup(q_lens, [L] * B, a.hq, a.hkv, bs=a.block)
    attn = AttnBatch(cu_q=cu.cuda(), kv_lens=kvl.cuda(), block_tables=bt.cuda(), num_seqs=B,
                     num_decode=B if a.mode == "decode" else 0, max_q_len=max(q_lens), max_kv_len=L,
                     num_tokens=sum(q_lens))
    for _ in range(a.iters):
        out = cuda.paged_attention(q, k, v, attn, 128 ** -0.5, a.hq, a.hkv, 128)
    torch.cuda.synchronize()
    if a.time:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        cuda.paged_attention(q, k, v, attn, 128 ** -0.5, a.hq, a.hkv, 128)
        e1.record()
        torch.cuda.synchronize()
        print(f"time {e0.elapsed_time(e1) * 1e3:.1f} us")
    # spot-check the first sequence against the oracle
    n = q_lens[0]
    ref = cpu_ref.paged_attention(q[:n].float().cpu(), k.float().cpu(), v.float().cpu(), cu[:2], kvl[:1], bt[:1],
                                  128 ** -0.5, a.hq, a.hkv, 128)
    if a.phases and a.mode == "prefill":
        prof = cuda.prefill_phase_profile(q, k, v, attn, 128 ** -0.5, a.hq, a.hkv, 128)
        tiles = max(1, prof["tiles"])
        for name, cyc in prof.items():
            print(f"{name:32s} {cyc:14d}   {cyc / tiles:9.1f} cycles/tile")
    print("max err (seq 0)", float((out[:n].float().cpu() - ref).abs().max()))


if __name__ == "__main__":
    main()
