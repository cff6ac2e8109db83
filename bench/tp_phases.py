"""Where the time of the one-kernel row-parallel projection goes: per-phase timeline of one launch.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench/tp_phases.py [--rows 256 --k 4096 --hidden 4096 --one-shot]

Every CTA of the kernel stamps the global nanosecond timer at its phase boundaries (``xv_tp_profile_buffer``);
rank 0 prints, relative to the first CTA's entry, when the first and the last CTA passed each boundary.
"""

from __future__ import annotations

import argparse
import ctypes
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

NAMES = ("entry", "GEMM roles done, tiles pushed", "all sources' tiles arrived", "own rows reduced + stored",
         "broadcast raised", "all owners' rows arrived (CTA 0)", "exit")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, nargs="*", default=[32, 256, 1024])
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--one-shot", action="store_true")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    from xixi_vllm_b200.ops import cuda
    from xixi_vllm_b200.parallel import groups
    from xixi_vllm_b200.parallel.symm import FusedTPComm

    groups.init_distributed_environment(world_size=world, rank=rank, local_rank=local, backend="nccl")
    groups.initialize_model_parallel(world, 1)
    comm = FusedTPComm(groups.get_tp_group(), dev, a.hidden, max(a.rows) * (world if a.one_shot else 1),
                       torch.bfloat16)
    L = cuda.lib()
    L.xv_tp_profile_buffer.argtypes = [ctypes.c_void_p]
    L.xv_tp_profile_buffer.restype = None
    H, K = a.hidden, a.k // world
    w = torch.ones(H, dtype=torch.bfloat16, device=dev)
    wt = (torch.randn(H, K, device=dev) * 0.02).bfloat16()
    prof = torch.zeros(512 * 8, dtype=torch.int64, device=dev)
    comm.begin_forward()
    for T in a.rows:
        x = (torch.randn(T, K, device=dev) * 0.5).bfloat16()
        resid = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
        for _ in range(6):
            comm.gemm_reduce_norm(x, wt, resid, w, 1e-6, two_shot=not a.one_shot)
        torch.cuda.synchronize()
        dist.barrier()
        prof.zero_()
        L.xv_tp_profile_buffer(prof.data_ptr())
        comm.gemm_reduce_norm(x, wt, resid, w, 1e-6, two_shot=not a.one_shot)
        torch.cuda.synchronize()
        L.xv_tp_profile_buffer(None)
        cuda.check_status(dev)
        p = prof.view(-1, 8).cpu()
        used = p[:, 0] > 0
        p = p[used]
        t0 = int(p[:, 0].min())
        if rank == 0:
            print(f"rows {T}, K/rank {K}, world {world}, {'one' if a.one_shot else 'two'}-shot, {int(used.sum())} CTAs; "
                  "microseconds after the first CTA's entry (first CTA .. last CTA to pass)")
            for i, name in enumerate(NAMES):
                col = p[:, i]
                col = col[col > 0]
                if len(col):
                    print(f"   {name:36s} {(int(col.min()) - t0) / 1e3:7.1f} .. {(int(col.max()) - t0) / 1e3:7.1f}   ({len(col)} CTAs)")
        dist.barrier()
    comm.destroy()
    groups.destroy_model_parallel()
    groups.destroy_distributed_environment()


if __name__ == "__main__":
    main()
