"""Runs the fused tensor-parallel reduction kernels on ONE GPU with a world of one rank (small,
self-contained target for an ncu capture of their memory behaviour; with one rank the "peers"
are this GPU's own buffer, so link traffic is absent but every load, the residual update, the
norm and the broadcast store run as in a real group).

    python -m bench.tp_reduce_one [--rows 4096 --hidden 4096 --iters 3] [--sharded]
    python -m bench.tp_reduce_one --what argmax|gather|sample|project [--rows 256 --vocab 151936 --k 4096]

``--what`` selects the other tensor-parallel kernels: vocabulary-parallel argmax, the logits column gather, the
sharded sampler (top-k 50, top-p 0.9) and the one-kernel row-parallel projection (GEMM whose epilogue pushes its
tiles into the reducing rank's slots, then residual add and RMSNorm).
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
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--sharded", action="store_true", help="row-sharded (two-shot) kernel instead of one-shot")
    ap.add_argument("--what", default="reduce", choices=["reduce", "argmax", "gather", "sample", "project"])
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--k", type=int, default=4096, help="K of the projection (--what project)")
    a = ap.parse_args()
    os.environ.setdefault("XV_TP_NVLS", "0")
    torch.cuda.set_device(0)
    dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29377", world_size=1, rank=0,
                            device_id=torch.device("cuda:0"))
    from xixi_vllm_b200.ops import cpu_ref, cuda
    from xixi_vllm_b200.parallel import groups
    from xixi_vllm_b200.parallel.symm import SPIN_LIMIT, FusedTPComm

    groups.init_distributed_environment(world_size=1, rank=0, backend="nccl")
    groups.initialize_model_parallel(1, 1)
    if a.what != "reduce":
        other_kernels(a, groups, cuda, FusedTPComm)
        dist.destroy_process_group()
        return
    comm = FusedTPComm(groups.get_tp_group(), torch.device("cuda:0"), a.hidden, a.rows, torch.bfloat16)
    g = torch.Generator().manual_seed(0)
    part = torch.randn(a.rows, a.hidden, generator=g).bfloat16().cuda()
    resid = torch.randn(a.rows, a.hidden, generator=g).bfloat16().cuda()
    w = torch.ones(a.hidden).bfloat16().cuda()
    ref_res = (part.float() + resid.float()).bfloat16()
    ref_y = cpu_ref.rmsnorm(ref_res.cpu(), w.cpu(), 1e-6)
    for _ in range(a.iters):
        comm.begin_forward()
        buf = comm.alloc_partial(a.rows)
        buf.copy_(part)
        r = resid.clone()
        if a.sharded:
            L = cuda.lib()
            rc = L.xv_tp_reduce_norm_sharded(comm._bufs, comm._flags, None, comm.epoch.data_ptr(), 0, 1,
                                             buf.data_ptr() - comm._base, comm.h_off, 1, r.data_ptr(), w.data_ptr(),
                                             a.rows, a.hidden, 1e-6, SPIN_LIMIT, comm.status.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream)
            assert rc == 0
            y = comm.h_view[: a.rows * a.hidden].view(a.rows, a.hidden)
        else:
            y, r = comm.reduce_add_rmsnorm(buf, r, w, 1e-6)
    torch.cuda.synchronize()
    cuda.check_status()
    print("max err y", float((y.float().cpu() - ref_y.float()).abs().max()),
          "residual", float((r.float() - ref_res.float()).abs().max()))
    dist.destroy_process_group()


def other_kernels(a, groups, cuda, FusedTPComm) -> None:
    dev = torch.device("cuda:0")
    os.environ["XV_TP_PUSH"] = "1"
    rows = min(a.rows, 512)
    comm = FusedTPComm(groups.get_tp_group(), dev, a.hidden, max(rows, 512), torch.bfloat16, logits_rows=rows,
                       logits_local_cols=a.vocab)
    g = torch.Generator().manual_seed(0)
    if a.what == "project":
        x = (torch.randn(rows, a.k, generator=g) * 0.5).bfloat16().to(dev)
        wt = (torch.randn(a.hidden, a.k, generator=g) * 0.05).bfloat16().to(dev)
        resid = torch.randn(rows, a.hidden, generator=g).bfloat16().to(dev)
        nw = torch.ones(a.hidden).bfloat16().to(dev)
        for _ in range(a.iters):
            comm.begin_forward()
            y, r = comm.gemm_reduce_norm(x, wt, resid.clone(), nw, 1e-6, two_shot=False)
        torch.cuda.synchronize()
        ref = ((x.float() @ wt.float().t()).bfloat16().float() + resid.float()).bfloat16()
        print("max err residual", float((r.float() - ref.float()).abs().max()))
    else:
        logits = (torch.randn(rows, a.vocab, generator=g) * 2.0).bfloat16().to(dev)
        temp = torch.full((rows,), 0.8, device=dev)
        top_k = torch.full((rows,), 50, dtype=torch.int32, device=dev)
        top_p = torch.full((rows,), 0.9, device=dev)
        min_p = torch.zeros(rows, device=dev)
        rng = torch.tensor([1, 2], dtype=torch.int32, device=dev)
        for _ in range(a.iters):
            if a.what == "argmax":
                out = comm.argmax(logits, a.vocab, 0)
            elif a.what == "gather":
                out = comm.gather_logits(logits)
            else:
                out = comm.sample(logits, a.vocab, 0, a.vocab, temp, top_k, top_p, min_p, rng)
        torch.cuda.synchronize()
        if a.what == "argmax":
            print("argmax equal", bool(torch.equal(out.cpu(), logits.float().argmax(-1).cpu())))
        elif a.what == "gather":
            print("gather equal", bool(torch.equal(out, logits)))
        else:
            want = cuda.sample(logits, temp, top_k, top_p, min_p, rng)
            print("sample equal", int((out == want).sum()), "of", rows)
    cuda.check_status()
    comm.destroy()


if __name__ == "__main__":
    main()
