"""Per-kernel microbenchmarks against the measured roofline.

    python -m bench.kernels [--what gemm,decode,prefill,elementwise] [--json out.json]

Large cases are timed with CUDA events on the launching stream after 3 warm-up launches, with a
256 MiB write between timed launches to flush the 126 MB L2. Kernels of a few microseconds would be
timed mostly for their host launch path that way (about 25 us per launch from Python), so the GEMM and
decode-attention cases are captured into a CUDA graph instead: as many copies of the inputs as it takes
to exceed the L2 (every launch reads cold operands), one launch per copy, back to back, and the graph's
time divided by the number of launches: the figure a decode graph of the engine sees. Results are
reported as achieved bytes/s or FLOP/s and as a fraction of the measured peaks in
``MEASURED_PEAKS.json`` (a STREAM-style copy and a cuBLAS bf16 GEMM on this machine). cuBLAS
(``torch.matmul``) is timed next to the GEMM the same way.
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

from xixi_vllm_b200.ops import cuda  # noqa: E402
from xixi_vllm_b200.runtime.staging import AttnBatch  # noqa: E402

DEV = "cuda"


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "src": "fallback"}


_flush = None


def timeit(fn, iters: int = 10, warmup: int = 3) -> float:
    """Median milliseconds per call."""
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        _flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def timeit_graph(make_fn, bytes_per_copy: float, min_copies: int = 4, reps: int = 5) -> float:
    """Median milliseconds per launch of ``make_fn(i)()`` inside a CUDA graph of back-to-back launches, copy i of
    the inputs each; enough copies that their operands exceed the L2 twice over."""
    n = max(min_copies, int(2 * 126e6 / max(bytes_per_copy, 1.0)) + 1)
    n = min(n, 256)
    fns = [make_fn(i) for i in range(n)]
    for f in fns[:3]:
        f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns:
            f()
    g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / n)
    times.sort()
    return times[len(times) // 2]


def bench_gemm(out: list) -> None:
    pk = peaks()
    shapes = [
        # decode (weight streaming): Qwen3-8B TP1 and TP8, 32B TP8
        (1, 6144, 4096), (32, 6144, 4096), (256, 6144, 4096), (256, 4096, 4096), (256, 24576, 4096),
        (256, 4096, 12288), (64, 151936, 4096), (32, 768, 4096), (32, 4096, 512), (32, 3072, 4096),
        (32, 4096, 1536), (256, 768, 4096), (256, 4096, 512), (256, 3072, 4096), (256, 4096, 1536),
        (256, 6400, 5120), (256, 5120, 3200),
        # a decode batch plus one prefill chunk
        (1400, 6144, 4096), (1400, 4096, 4096), (1400, 24576, 4096), (1400, 4096, 12288),
        # prefill (compute bound)
        (4096, 6144, 4096), (4096, 4096, 4096), (4096, 24576, 4096), (4096, 4096, 12288),
        (16384, 24576, 4096), (8192, 8192, 8192),
    ]
    for m, n, k in shapes:
        x = torch.randn(m, k, device=DEV).bfloat16()
        w = torch.randn(n, k, device=DEV).bfloat16()
        if 2.0 * n * k <= 64e6:
            # small: cold copies inside one graph, no host launch path in the figure
            copies = max(4, int(2 * 126e6 / (2.0 * n * k)) + 1)
            copies = min(copies, 256)
            ws = [w] + [torch.randn(n, k, device=DEV).bfloat16() for _ in range(copies - 1)]
            ys = [torch.empty(m, n, device=DEV, dtype=torch.bfloat16) for _ in range(2)]
            ms = timeit_graph(lambda i: (lambda: cuda.linear(x, ws[i % len(ws)], out=ys[i & 1])), 2.0 * n * k)
            ms_cublas = timeit_graph(lambda i: (lambda: torch.matmul(x, ws[i % len(ws)].t(), out=ys[i & 1])), 2.0 * n * k)
            del ws
        else:
            ms = timeit(lambda: cuda.linear(x, w))
            ms_cublas = timeit(lambda: torch.matmul(x, w.t()))
        flops = 2.0 * m * n * k
        byts = 2.0 * (m * k + n * k + m * n)
        tf, gbs = flops / ms / 1e9, byts / ms / 1e6
        frac = max(tf / pk["tflops"], gbs / pk["hbm_gbs"])
        pl = cuda.gemm_plan(m, n, k, 148)
        out.append(dict(kernel="gemm_tcgen05", m=m, n=n, k=k, ms=ms, tflops=tf, gbs=gbs, frac_of_peak=frac,
                        cublas_ms=ms_cublas, vs_cublas=ms_cublas / ms, swapped=pl.swapped, splits=pl.splits,
                        bn=pl.bn, stages=pl.stages))
        print(f"gemm {m:6d}x{n:6d}x{k:6d}: {ms:8.3f} ms {tf:8.1f} TF {gbs:8.1f} GB/s frac {frac:5.2f} of {pk['src']}"
              f" | cublas {ms_cublas:8.3f} ms (x{ms_cublas / ms:4.2f})", flush=True)
        del x, w


def _attn_setup(q_lens, kv_lens, hq, hkv, bs=16):
    B = len(kv_lens)
    maxb = max(-(-l // bs) for l in kv_lens)
    nblocks = sum(-(-l // bs) for l in kv_lens) + 1
    bt = torch.zeros(B, maxb, dtype=torch.int32)
    nxt = 0
    perm = torch.randperm(nblocks)
    for b, l in enumerate(kv_lens):
        nb = -(-l // bs)
        bt[b, :nb] = perm[nxt:nxt + nb].to(torch.int32)
        nxt += nb
    k = torch.randn(nblocks, hkv, bs, 128, device=DEV).bfloat16()
    v = torch.randn(nblocks, hkv, bs, 128, device=DEV).bfloat16()
    T = sum(q_lens)
    q = torch.randn(T, hq * 128, device=DEV).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    return q, k, v, cu, torch.tensor(kv_lens, dtype=torch.int32), bt


def _flash_attn():
    """flash-attn 2 from the image, for a same-box comparison only (the reference's attention backend:
    src/compute/layers/attention.py:80-99); None when it cannot be imported."""
    try:
        import flash_attn
        return flash_attn
    except Exception:   # noqa: BLE001
        return None


def bench_decode(out: list) -> None:
    pk = peaks()
    fa = _flash_attn()
    for B, L, hq, hkv in [(256, 1408, 32, 8), (32, 1408, 32, 8), (1, 2048, 32, 8), (256, 1408, 4, 1),
                          (256, 2048, 8, 1), (8, 4096, 32, 8)]:
        q, k, v, cu, kvl, bt = _attn_setup([1] * B, [L] * B, hq, hkv)
        attn = AttnBatch(cu_q=cu.to(DEV), kv_lens=kvl.to(DEV), block_tables=bt.to(DEV), num_seqs=B, num_decode=B,
                         max_q_len=1, max_kv_len=L, num_tokens=B)
        byts = 2.0 * B * L * hkv * 128 * 2
        # graph-timed in every case: the figure is device time, not the Python launch path; the KV copies
        # alternate so that no launch finds its operands in L2
        copies = min(64, max(2, int(2 * 126e6 / byts) + 1))
        kvs = [(k, v)] + [(torch.randn_like(k), torch.randn_like(v)) for _ in range(copies - 1)]
        ms = timeit_graph(lambda i: (lambda: cuda.paged_attention(q, kvs[i % len(kvs)][0], kvs[i % len(kvs)][1], attn,
                                                                  128 ** -0.5, hq, hkv, 128)), byts, min_copies=4)
        del kvs
        gbs = byts / ms / 1e6
        ms_fa = float("nan")
        if fa is not None:
            try:
                # flash-attn 2 wants pages of 256 tokens laid out [page, token, head, dim]
                pages = -(-L // 256)
                n_fa = min(16, max(2, int(2 * 126e6 / byts) + 1))
                kcs = [(torch.randn(B * pages + 1, 256, hkv, 128, device=DEV).bfloat16(),
                        torch.randn(B * pages + 1, 256, hkv, 128, device=DEV).bfloat16()) for _ in range(n_fa)]
                tbl = torch.randperm(B * pages, device=DEV).to(torch.int32).view(B, pages)
                lens = torch.full((B,), L, dtype=torch.int32, device=DEV)
                q4 = q.view(B, 1, hq, 128)
                ms_fa = timeit_graph(lambda i: (lambda: fa.flash_attn_with_kvcache(
                    q4, kcs[i % n_fa][0], kcs[i % n_fa][1], cache_seqlens=lens, block_table=tbl,
                    softmax_scale=128 ** -0.5, causal=True)), byts, min_copies=4)
                del kcs
            except Exception as e:   # noqa: BLE001
                print(f"  flash-attn decode failed: {type(e).__name__}: {e}")
        out.append(dict(kernel="attn_decode", batch=B, kv_len=L, hq=hq, hkv=hkv, ms=ms, gbs=gbs,
                        frac_of_peak=gbs / pk["hbm_gbs"], ms_flash_attn2=ms_fa))
        print(f"decode B={B:4d} L={L:5d} hq={hq} hkv={hkv}: {ms:8.3f} ms {gbs:8.1f} GB/s frac "
              f"{gbs / pk['hbm_gbs']:5.2f} of {pk['src']} | flash-attn2 {ms_fa:8.3f} ms (x{ms_fa / ms:4.2f})", flush=True)
        del q, k, v


def bench_prefill(out: list) -> None:
    pk = peaks()
    fa = _flash_attn()
    for B, L, hq, hkv in [(8, 2048, 32, 8), (16, 1024, 32, 8), (4, 4096, 32, 8), (8, 2048, 4, 1)]:
        q, k, v, cu, kvl, bt = _attn_setup([L] * B, [L] * B, hq, hkv)
        attn = AttnBatch(cu_q=cu.to(DEV), kv_lens=kvl.to(DEV), block_tables=bt.to(DEV), num_seqs=B, num_decode=0,
                         max_q_len=L, max_kv_len=L, num_tokens=B * L)
        ms = timeit(lambda: cuda.paged_attention(q, k, v, attn, 128 ** -0.5, hq, hkv, 128))
        flops = 4.0 * B * hq * 128 * L * L / 2       # causal: half the square
        tf = flops / ms / 1e9
        ms_fa = float("nan")
        if fa is not None:
            try:
                # contiguous K/V (no page table): flash-attn 2's best case
                kf = torch.randn(B * L, hkv, 128, device=DEV).bfloat16()
                vf = torch.randn_like(kf)
                cu_dev = cu.to(DEV)
                ms_fa = timeit(lambda: fa.flash_attn_varlen_func(q.view(B * L, hq, 128), kf, vf, cu_dev, cu_dev, L, L,
                                                                 softmax_scale=128 ** -0.5, causal=True))
                del kf, vf
            except Exception as e:   # noqa: BLE001
                print(f"  flash-attn prefill failed: {type(e).__name__}: {e}")
        out.append(dict(kernel="attn_prefill", batch=B, seq=L, hq=hq, hkv=hkv, ms=ms, tflops=tf,
                        frac_of_peak=tf / pk["tflops"], ms_flash_attn2=ms_fa))
        print(f"prefill B={B:3d} L={L:5d} hq={hq} hkv={hkv}: {ms:8.3f} ms {tf:8.1f} TF frac "
              f"{tf / pk['tflops']:5.2f} of {pk['src']} | flash-attn2 {ms_fa:8.3f} ms (x{ms_fa / ms:4.2f})", flush=True)
        del q, k, v


def bench_elementwise(out: list) -> None:
    pk = peaks()
    T, H, I = 16384, 4096, 12288
    x = torch.randn(T, H, device=DEV).bfloat16()
    r = torch.randn(T, H, device=DEV).bfloat16()
    w = torch.ones(H, device=DEV).bfloat16()
    cases = [("rmsnorm", lambda: cuda.rmsnorm(x, w, 1e-6), 2.0 * T * H * 2),
             ("add_rmsnorm", lambda: cuda.add_rmsnorm(x, r, w, 1e-6), 4.0 * T * H * 2)]
    gu = torch.randn(T, 2 * I, device=DEV).bfloat16()
    cases.append(("silu_mul", lambda: cuda.silu_mul(gu), 3.0 * T * I * 2))
    for name, fn, byts in cases:
        ms = timeit(fn)
        gbs = byts / ms / 1e6
        out.append(dict(kernel=name, tokens=T, ms=ms, gbs=gbs, frac_of_peak=gbs / pk["hbm_gbs"]))
        print(f"{name:12s} T={T}: {ms:8.3f} ms {gbs:8.1f} GB/s frac {gbs / pk['hbm_gbs']:5.2f} of {pk['src']}", flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="gemm,decode,prefill,elementwise")
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    out: list = []
    table = {"gemm": bench_gemm, "decode": bench_decode, "prefill": bench_prefill, "elementwise": bench_elementwise}
    for name in a.what.split(","):
        table[name](out)
    cuda.check_status()
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"peaks": peaks(), "results": out}, f, indent=1)


if __name__ == "__main__":
    main()
