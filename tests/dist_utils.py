"""Spawn helpers for multi-rank CPU tests over gloo."""
import multiprocessing as mp
import os
import socket
import sys
import traceback


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _entry(fn, rank, world, port, tp, pp, q, args):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    sys.path.insert(0, os.path.join(root, "tests"))
    try:
        import torch

        from xixi_vllm_b200.parallel import groups
        torch.set_num_threads(1)
        groups.init_distributed_environment(world_size=world, rank=rank, backend="gloo",
                                            init_method=f"tcp://127.0.0.1:{port}", timeout_s=60)
        groups.initialize_model_parallel(tp, pp, backend="gloo")
        q.put((rank, "ok", fn(rank, world, *args)))
    except BaseException:
        q.put((rank, "err", traceback.format_exc()))
    finally:
        try:
            from xixi_vllm_b200.parallel import groups
            groups.destroy_model_parallel()
            groups.destroy_distributed_environment()
        except Exception:
            pass


def run_ranks(fn, world: int, tp: int, pp: int = 1, args=(), timeout: float = 120.0):
    """Runs ``fn(rank, world, *args)`` in ``world`` gloo ranks; returns results ordered by rank."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(fn, r, world, port, tp, pp, q, args)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, status, payload = q.get(timeout=timeout)
            if status != "ok":
                raise AssertionError(f"rank {rank} failed:\n{payload}")
            results[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.terminate()
    return [results[r] for r in range(world)]


def _entry_gpu(fn, rank, world, port, tp, pp, q, args):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    sys.path.insert(0, os.path.join(root, "tests"))
    try:
        import torch

        from xixi_vllm_b200.parallel import groups
        torch.cuda.set_device(rank)
        groups.set_nccl_env("", disable_ib=True)
        groups.init_distributed_environment(world_size=world, rank=rank, local_rank=rank, backend="nccl",
                                            init_method=f"tcp://127.0.0.1:{port}", timeout_s=120)
        groups.initialize_model_parallel(tp, pp, backend="nccl")
        out = fn(rank, world, *args)
        torch.cuda.synchronize()
        q.put((rank, "ok", out))
    except BaseException:
        q.put((rank, "err", traceback.format_exc()))
    finally:
        try:
            from xixi_vllm_b200.parallel import groups
            groups.destroy_model_parallel()
            groups.destroy_distributed_environment()
        except Exception:
            pass


def run_ranks_gpu(fn, world: int, tp: int, pp: int = 1, args=(), timeout: float = 300.0):
    """Like ``run_ranks`` but one CUDA device per rank over NCCL."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry_gpu, args=(fn, r, world, port, tp, pp, q, args)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, status, payload = q.get(timeout=timeout)
            if status != "ok":
                raise AssertionError(f"rank {rank} failed:\n{payload}")
            results[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.terminate()
    return [results[r] for r in range(world)]
