"""Timeline of one launch of the single-CTA tcgen05 GEMM kernel (where a small GEMM's microseconds go).

    python -m bench.gemm_phases [--shapes 256x4096x512 256x4096x1536 32x6144x4096] [--flush]

Every CTA stamps the global nanosecond timer at its phase boundaries (``xv_gemm_profile_buffer``); printed are,
relative to the first CTA's entry, the times at which the first and the last CTA passed each boundary, next to the
CUDA-event time of the launch.
"""

from __future__ import annotations

import argparse
import ctypes
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from xixi_vllm_b200.ops import cuda  # noqa: E402

NAMES = ("entry", "barriers + TMEM ready", "first tile load issued", "first stage landed", "first tile: MMAs issued",
         "first tile: accumulator complete", "last epilogue done", "exit")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", nargs="*", default=["256x4096x512", "256x4096x1536", "32x6144x4096", "256x768x4096"])
    ap.add_argument("--flush", action="store_true", help="write 256 MiB before the profiled launch (cold L2)")
    a = ap.parse_args()
    L = cuda.lib()
    L.xv_gemm_profile_buffer.argtypes = [ctypes.c_void_p]
    L.xv_gemm_profile_buffer.restype = None
    L.xv_gemm_disable_pair(1)
    prof = torch.zeros(1024 * 8, dtype=torch.int64, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for shape in a.shapes:
        m, n, k = (int(v) for v in shape.split("x"))
        x = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
        w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
        for _ in range(5):
            cuda.linear(x, w, defer=True)
        torch.cuda.synchronize()
        if a.flush:
            flush.zero_()
            torch.cuda.synchronize()
        prof.zero_()
        L.xv_gemm_profile_buffer(prof.data_ptr())
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        cuda.linear(x, w, defer=True)
        e1.record()
        torch.cuda.synchronize()
        L.xv_gemm_profile_buffer(None)
        cuda.check_status()
        pl = cuda.gemm_plan(m, n, k, 148)
        p = prof.view(-1, 8).cpu()
        p = p[p[:, 0] > 0]
        t0 = int(p[:, 0].min())
        print(f"{shape}: {len(p)} CTAs, bn {pl.bn} splits {pl.splits} stages {pl.stages} ctas/SM {pl.ctas_per_sm}, "
              f"{pl.k_blocks_per_split} K blocks per CTA; event time {e0.elapsed_time(e1) * 1e3:.1f} us")
        for i, name in enumerate(NAMES):
            col = p[:, i]
            col = col[col > 0]
            if len(col):
                print(f"   {name:34s} {(int(col.min()) - t0) / 1e3:7.2f} .. {(int(col.max()) - t0) / 1e3:7.2f}  median "
                      f"{(int(col.median()) - t0) / 1e3:7.2f}")
    L.xv_gemm_disable_pair(0)


if __name__ == "__main__":
    main()
