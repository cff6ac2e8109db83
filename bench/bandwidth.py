"""Interconnect probe: topology report, peer copy bandwidth and latency, and the NCCL all-reduce curve
(reference: bench/bench_bandwidth.py:124-160, bench/probe_server.py:82-137).

    python -m bench.bandwidth                              # topology + peer copies from GPU 0
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench/bandwidth.py --collective                    # NCCL all-reduce latency / bus bandwidth over N GPUs

All timings are CUDA events after warm-up. Bus bandwidth of an all-reduce is algbw * 2 (n - 1) / n.
"""

from __future__ import annotations

import argparse
import os
import subprocess

import torch


def topology() -> None:
    n = torch.cuda.device_count()
    print(f"{n} GPUs")
    for i in range(n):
        p = torch.cuda.get_device_properties(i)
        print(f"  cuda:{i} {p.name}, {p.total_memory / 2**30:.0f} GiB, {p.multi_processor_count} SMs")
    print("peer access (row can read column):")
    for i in range(n):
        print("  " + " ".join("x" if i == j else ("1" if torch.cuda.can_device_access_peer(i, j) else "0") for j in range(n)))
    try:
        out = subprocess.run(["nvidia-smi", "topo", "-m"], capture_output=True, text=True, timeout=20).stdout
        print(out.strip())
    except (OSError, subprocess.TimeoutExpired):
        pass


def _time(fn, warmup=5, iters=20) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def peer_copies(src: int, max_bytes: int) -> None:
    n = torch.cuda.device_count()
    print(f"peer copies from cuda:{src} (GB/s per direction; 4-byte copy time as latency)")
    for dst in range(n):
        if dst == src:
            continue
        torch.cuda.set_device(src)
        tiny_s = torch.zeros(1, dtype=torch.float32, device=f"cuda:{src}")
        tiny_d = torch.zeros(1, dtype=torch.float32, device=f"cuda:{dst}")
        lat = _time(lambda: tiny_d.copy_(tiny_s, non_blocking=True))
        row = [f"  -> cuda:{dst}: latency {lat * 1e3:6.1f} us |"]
        size = 1 << 20
        while size <= max_bytes:
            x = torch.empty(size, dtype=torch.uint8, device=f"cuda:{src}")
            y = torch.empty(size, dtype=torch.uint8, device=f"cuda:{dst}")
            ms = _time(lambda: y.copy_(x, non_blocking=True), iters=10)
            row.append(f"{size >> 20} MiB {size / ms / 1e6:6.0f}")
            del x, y
            size *= 8
        print(" ".join(row), flush=True)


def collective(max_bytes: int) -> None:
    import torch.distributed as dist

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if rank == 0:
        print(f"NCCL all-reduce over {world} GPUs (bf16): size, time (max over ranks), algbw, busbw")
    size = 2048
    while size <= max_bytes:
        x = torch.zeros(size // 2, dtype=torch.bfloat16, device="cuda")
        ms = _time(lambda: dist.all_reduce(x), warmup=10, iters=30)
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
        if rank == 0:
            alg = size / ms / 1e6
            print(f"  {size / 1024:10.0f} KiB {ms * 1e3:9.1f} us {alg:8.1f} GB/s {alg * 2 * (world - 1) / world:8.1f} GB/s", flush=True)
        del x
        size *= 4
    dist.barrier()
    dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--collective", action="store_true", help="run under torchrun: NCCL all-reduce curve")
    ap.add_argument("--src", type=int, default=0)
    ap.add_argument("--max-mib", type=int, default=512)
    a = ap.parse_args()
    if a.collective:
        collective(a.max_mib << 20)
    else:
        topology()
        if torch.cuda.device_count() > 1:
            peer_copies(a.src, a.max_mib << 20)


if __name__ == "__main__":
    main()
