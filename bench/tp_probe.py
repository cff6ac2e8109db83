"""Latency of one tensor-parallel reduction point, library collective against the fused kernels.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench/tp_probe.py [--hidden 4096 --iters 50 --layers 36]

For T = 1 .. 4096 rows of ``hidden`` bf16 it times, with CUDA events on every rank (max over ranks):
  nccl          all-reduce of the [T, hidden] partial, then the add + RMSNorm kernel (what the reference does)
  fused         the one-shot kernel: barrier, cross-rank sum (multimem.ld_reduce or peer loads), residual add, RMSNorm
  fused-sharded the row-sharded kernel: reduce own rows, keep the residual shard, broadcast normalised rows
and prints the per-step cost of a model with ``layers`` decoder layers (2 * layers + 1 reduction points).
A second table times the whole row-parallel projection [T, K / world] x [hidden, K / world]^T with its
reduction point (``--k`` is the unsharded K, 4096 for Qwen3-8B's o_proj, 12288 for down_proj):
  gemm+nccl     tcgen05 GEMM, NCCL all-reduce, add + RMSNorm kernel
  gemm+sharded  tcgen05 GEMM into the symmetric buffer, then the row-sharded reduction kernel
  one-kernel    GEMM whose epilogue pushes its tiles to the reducing ranks, which sum, add the residual,
                normalise and broadcast in the same kernel (two-shot), or every rank reduces all rows (one-shot)
with the roofline of the fused path: the slower of 2*T*hidden*K/world FLOP at the measured GEMM peak and the
bytes that must cross NVLink at the measured 770 GB/s per direction.
Every timed call is preceded by the write of the partial into the symmetric buffer, as in the model, so the
buffer-reuse rule of the kernels (never the same buffer in two consecutive calls) holds.
The reference's probe prints the NCCL all-reduce latency curve only (reference: bench/probe_server.py:82-137).
"""

from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--max-rows", type=int, default=4096)
    ap.add_argument("--k", type=int, nargs="*", default=[4096, 12288], help="unsharded K of the projections to time")
    ap.add_argument("--peak-tflops", type=float, default=0.0, help="GEMM peak for the roofline (default: MEASURED_PEAKS.json)")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    from xixi_vllm_b200.ops import cuda
    from xixi_vllm_b200.parallel import groups
    from xixi_vllm_b200.parallel.symm import SPIN_LIMIT, FusedTPComm

    groups.init_distributed_environment(world_size=world, rank=rank, local_rank=local, backend="nccl")
    groups.initialize_model_parallel(world, 1)
    tp = groups.get_tp_group()
    comm = FusedTPComm(tp, dev, a.hidden, a.max_rows, torch.bfloat16)
    H = a.hidden
    w = torch.ones(H, dtype=torch.bfloat16, device=dev)
    L = cuda.lib()
    comm.begin_forward()

    def timed(fn, iters):
        """Microseconds per call, max over ranks. The calls are captured into one CUDA graph so that the
        figure is device time, not the Python launch path; falls back to eager launches if capture fails."""
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        graph = None
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(iters):
                    fn()
            graph = g
        except Exception as e:   # noqa: BLE001
            if rank == 0:
                print(f"  (graph capture failed: {type(e).__name__}; timing eager launches)")
        torch.cuda.synchronize()
        dist.barrier()
        reps = 3 if graph is not None else 1
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if graph is not None:
            graph.replay()
            torch.cuda.synchronize()
            dist.barrier()
        e0.record()
        for _ in range(reps):
            if graph is not None:
                graph.replay()
            else:
                for _ in range(iters):
                    fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / (iters * reps) * 1e3], device=dev)      # us per call
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    rows = [t for t in (1, 8, 32, 128, 256, 1024, 4096) if t <= a.max_rows]
    if rank == 0:
        print(f"world {world}, hidden {H}, multicast {'yes' if comm.mc_ptr else 'no'}; microseconds per reduction point "
              "(includes the 2-byte-per-element write of the partial)")
        print(f"{'rows':>6} {'KiB':>8} {'nccl+norm':>10} {'fused':>8} {'sharded':>8}   per step ({2 * a.layers + 1} points), ms")
    for T in rows:
        part = torch.randn(T, H, device=dev).bfloat16()
        resid = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
        scratch = torch.empty_like(part)

        def nccl():
            scratch.copy_(part)
            dist.all_reduce(scratch, group=tp.device_group)
            cuda.add_rmsnorm(scratch, resid, w, 1e-6)

        def fused():
            buf = comm.alloc_partial(T)          # alternates between two buffers of the symmetric heap
            buf.copy_(part)
            comm.reduce_add_rmsnorm(buf, resid, w, 1e-6)

        def sharded():
            buf = comm.alloc_partial(T)
            buf.copy_(part)
            rc = L.xv_tp_reduce_norm_sharded(comm._bufs, comm._flags, comm.mc_ptr or None, comm.epoch.data_ptr(),
                                             comm.rank, comm.world, buf.data_ptr() - comm._base, comm.h_off, 1,
                                             resid.data_ptr(), w.data_ptr(), T, H, 1e-6, SPIN_LIMIT,
                                             comm.status.data_ptr(), torch.cuda.current_stream().cuda_stream)
            if rc:
                raise RuntimeError(f"xv_tp_reduce_norm_sharded returned {rc}")

        iters = a.iters if T <= 1024 else max(6, a.iters // 5)
        iters += iters % 2               # an even count keeps the two-buffer rotation aligned across graph replays
        t_n, t_f, t_s = timed(nccl, iters), timed(fused, iters), timed(sharded, iters)
        cuda.check_status(dev)
        if rank == 0:
            pts = 2 * a.layers + 1
            print(f"{T:6d} {T * H * 2 / 1024:8.0f} {t_n:10.1f} {t_f:8.1f} {t_s:8.1f}   "
                  f"{t_n * pts / 1e3:6.2f} {t_f * pts / 1e3:6.2f} {t_s * pts / 1e3:6.2f}", flush=True)
    # ---- the whole row-parallel projection with its reduction point ----
    peak = a.peak_tflops
    if peak <= 0:
        import json
        path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        peak = json.load(open(path))["bf16_tflops"] if os.path.isfile(path) else 1590.0
    link_gbs = 770.0
    for k_full in a.k:
        K = k_full // world
        if K % 64:
            continue
        wt = (torch.randn(H, K, device=dev) * 0.02).bfloat16()
        if rank == 0:
            print(f"\nrow-parallel projection K = {k_full} / {world} = {K} per rank, N = {H}; microseconds (max over ranks)")
            print(f"{'rows':>6} {'gemm+nccl':>10} {'gemm+sharded':>13} {'one-kernel 2-shot':>18} {'one-kernel 1-shot':>18} "
                  f"{'roofline':>9} {'best/roofline':>14}")
        for T in [t for t in (1, 8, 32, 64, 128, 256, 512, 1024, 2048, 4096) if t <= a.max_rows]:
            x = (torch.randn(T, K, device=dev) * 0.5).bfloat16()
            resid = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
            scratch = torch.empty(T, H, dtype=torch.bfloat16, device=dev)

            def gemm_nccl():
                cuda.linear(x, wt, out=scratch)
                dist.all_reduce(scratch, group=tp.device_group)
                cuda.add_rmsnorm(scratch, resid, w, 1e-6)

            def gemm_sharded():
                buf = comm.alloc_partial(T)
                cuda.linear(x, wt, out=buf)
                rc = L.xv_tp_reduce_norm_sharded(comm._bufs, comm._flags, comm.mc_ptr or None, comm.epoch.data_ptr(),
                                                 comm.rank, comm.world, buf.data_ptr() - comm._base, comm.h_off, 1,
                                                 resid.data_ptr(), w.data_ptr(), T, H, 1e-6, SPIN_LIMIT,
                                                 comm.status.data_ptr(), torch.cuda.current_stream().cuda_stream)
                if rc:
                    raise RuntimeError(f"xv_tp_reduce_norm_sharded returned {rc}")

            def one_kernel_two_shot():
                comm.gemm_reduce_norm(x, wt, resid, w, 1e-6, two_shot=True)

            def one_kernel_one_shot():
                comm.gemm_reduce_norm(x, wt, resid, w, 1e-6, two_shot=False)

            iters = a.iters if T <= 1024 else max(6, a.iters // 5)
            iters += iters % 2
            t1, t2, t3 = timed(gemm_nccl, iters), timed(gemm_sharded, iters), timed(one_kernel_two_shot, iters)
            t4 = timed(one_kernel_one_shot, iters) if world * T * H * 2 <= comm.buf_bytes and T <= 512 else float("nan")
            cuda.check_status(dev)
            flop_us = 2.0 * T * H * K / (peak * 1e12) * 1e6
            # two-shot: (world-1)/world of the partial leaves this GPU, the same share of the result comes back
            link_us = 2.0 * T * H * 2 * (world - 1) / world / (link_gbs * 1e9) * 1e6
            roof = max(flop_us, link_us)
            best = min(v for v in (t3, t4) if v == v)
            if rank == 0:
                print(f"{T:6d} {t1:10.1f} {t2:13.1f} {t3:18.1f} {t4:18.1f} {roof:9.1f} {roof / best:14.2f}", flush=True)
    dist.barrier()
    comm.destroy()
    groups.destroy_model_parallel()
    groups.destroy_distributed_environment()


if __name__ == "__main__":
    main()
