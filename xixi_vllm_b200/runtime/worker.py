"""Per-rank lifecycle (reference: src/compute/worker.py:28-215): process groups, model load,
KV sizing, model runner, reset, teardown."""

from __future__ import annotations

import gc
import os
import tempfile

import torch

from ..models.loader import load_model
from ..models.qwen3 import Qwen3ForCausalLM
from ..parallel import groups
from ..parallel.pp import set_pp_layer_ranges
from ..parallel.tp_comm import make_tp_comm
from .kv_pool import KVPool
from .model_runner import ModelRunner
from .sampler import Sampler

__all__ = ["Worker"]


class Worker:
    def __init__(self, config, rank: int, tp_rank: int, pp_rank: int, local_rank: int | None = None) -> None:
        self.config = config
        self.rank, self.tp_rank, self.pp_rank = rank, tp_rank, pp_rank
        self.tp_size, self.pp_size, self.world_size = config.tp_size, config.pp_size, config.world_size
        self.local_rank = rank if local_rank is None else local_rank
        self.on_cuda = config.device == "cuda"
        self.device = torch.device(f"cuda:{self._device_id()}") if self.on_cuda else torch.device("cpu")
        from ..control.engine import resolve_dtype

        self.dtype = resolve_dtype(config)
        self.model = None
        self.kv: KVPool | None = None
        self.sampler: Sampler | None = None
        self.model_runner: ModelRunner | None = None
        self.is_last_pp = pp_rank == config.pp_size - 1

    def _device_id(self) -> int:
        if self.config.device_ids is not None:
            return self.config.device_ids[self.rank]
        return self.local_rank

    # --- environment ---------------------------------------------------------------------
    def init_environment(self, init_method: str | None = None) -> None:
        cfg = self.config
        if self.on_cuda:
            torch.cuda.set_device(self.device)
        if self.world_size == 1:
            groups.single_process_groups()
        else:
            backend = "nccl" if self.on_cuda else "gloo"
            if backend == "nccl":
                groups.set_nccl_env(cfg.nccl_ifname, disable_ib=not bool(cfg.nccl_ifname))
            if init_method is None:
                if cfg.master_addr in ("", "127.0.0.1", "localhost"):
                    # a file store needs no rank to listen first; the path is unique per launch
                    # and removed at teardown
                    init_method = "file://" + rendezvous_path(cfg)
                else:
                    init_method = f"tcp://{cfg.master_addr}:{cfg.nccl_port}"
            groups.init_distributed_environment(world_size=self.world_size, rank=self.rank,
                                                local_rank=self._device_id(), backend=backend,
                                                init_method=init_method)
            groups.initialize_model_parallel(self.tp_size, self.pp_size, self.tp_rank, self.pp_rank,
                                             backend=backend)
        set_pp_layer_ranges(cfg.pp_layer_counts)
        self.is_last_pp = groups.get_pp_group().is_last_rank

    # --- model + KV ------------------------------------------------------------------------
    def initialize(self) -> None:
        cfg = self.config
        torch.manual_seed(cfg.seed)
        with torch.no_grad():
            self.model = Qwen3ForCausalLM(cfg.hf_config, dtype=self.dtype, device=self.device)
            if cfg.load_format == "dummy":
                self.model.init_random(cfg.seed)
            else:
                report = load_model(self.model, cfg.model)
                if report["skipped"] and self.rank == 0 and self.pp_size == 1:
                    print(f"[loader] {len(report['skipped'])} tensors not used, e.g. {report['skipped'][:3]}")
        max_tokens = max(cfg.max_num_batched_tokens, cfg.max_num_seqs)
        # last pipeline stage: room for gathering the full logits of sampled rows over peer memory
        head = getattr(self.model, "lm_head", None)
        fused_logits = hasattr(head, "weight") and os.environ.get("XV_TP_LOGITS_GATHER", "fused") != "nccl"
        self.model.comm = make_tp_comm(groups.get_tp_group(), cfg.tp_comm, self.device,
                                       cfg.hf_config.hidden_size, max_tokens, self.dtype,
                                       logits_rows=cfg.max_num_seqs if fused_logits else 0,
                                       logits_local_cols=head.weight.shape[0] if fused_logits else 0)
        if self.on_cuda:
            torch.cuda.synchronize(self.device)
            torch.cuda.empty_cache()
        self.sampler = Sampler(cfg.seed)
        self.kv = self._make_kv()
        self.model_runner = ModelRunner(self.model, self.kv, self.sampler, config=cfg, device=self.device)

    def _make_kv(self) -> KVPool:
        cfg = self.config
        n = cfg.num_kvcache_blocks
        if n <= 0:
            # leave room for activations of the largest step and for CUDA-graph pools
            H, I = cfg.hf_config.hidden_size, cfg.hf_config.intermediate_size
            per_tok = (6 * H + 3 * (2 * I // self.tp_size)) * 2
            reserve = max(cfg.max_num_batched_tokens, cfg.max_num_seqs) * per_tok + (1 << 30)
            if not cfg.enforce_eager:
                reserve += 2 << 30
            n = KVPool.auto_num_blocks(cfg.hf_config, block_size=cfg.block_size, dtype=self.dtype,
                                       device=self.device, gpu_memory_utilization=cfg.gpu_memory_utilization,
                                       reserve_bytes=reserve if self.on_cuda else 0,
                                       max_useful_tokens=cfg.max_num_seqs * cfg.context_len)
            cfg.num_kvcache_blocks = n
        pool = KVPool(cfg.hf_config, num_blocks=n, block_size=cfg.block_size, device=self.device, dtype=self.dtype)
        if self.rank == 0:
            gib = n * pool.bytes_per_block / 2**30
            print(f"[kv] {n} pages x {cfg.block_size} tokens = {n * cfg.block_size} tokens, {gib:.2f} GiB per rank")
        return pool

    def get_kv_cache_size(self) -> int:
        assert self.kv is not None, "initialize() must run first"
        return self.kv.num_blocks_total

    def reset_kv(self, prefix_backend: str | None = None) -> None:
        """Forget all cached KV. The pool tensor is reused (its contents are unreachable once
        the ledger is rebuilt); only the per-sequence staging rows are dropped."""
        if prefix_backend is not None:
            self.config.prefix_backend = prefix_backend
        assert self.model_runner is not None
        self.model_runner.stager.reset()

    # --- steps ---------------------------------------------------------------------------------
    def execute_model(self, sched):
        """Launch one step; returns (n_prefill, n_decode) on the last pipeline stage, else None."""
        counts = self.model_runner.run_forward(sched)
        return counts if self.is_last_pp else None

    def read_samples(self, n_p: int, n_d: int):
        return self.model_runner.read_samples(n_p, n_d)

    def device_time_ms(self, lo: int, hi: int) -> float:
        """Forward device time of steps [lo, hi) on this rank, maximised over the replica's ranks."""
        t = self.model_runner.device_time_ms(lo, hi) if self.on_cuda else 0.0
        world = groups.get_world_group()
        if world.size > 1:
            import torch.distributed as dist

            buf = torch.tensor([t], dtype=torch.float64)
            dist.all_reduce(buf, op=dist.ReduceOp.MAX, group=world.cpu_group)
            t = float(buf.item())
        return t

    def destroy_environment(self) -> None:
        if self.on_cuda and torch.cuda.is_available():
            try:
                torch.cuda.synchronize(self.device)
            except RuntimeError:
                pass
        if self.model_runner is not None:
            self.model_runner.destroy()
        comm = getattr(self.model, "comm", None)
        if hasattr(comm, "destroy"):
            comm.destroy()
        self.model_runner = self.kv = self.model = None
        set_pp_layer_ranges(None)
        groups.destroy_model_parallel()
        groups.destroy_distributed_environment()
        if self.rank == 0 and self.world_size > 1:
            try:
                os.unlink(rendezvous_path(self.config))
            except OSError:
                pass
        gc.collect()
        if self.on_cuda and torch.cuda.is_available():
            torch.cuda.empty_cache()


def rendezvous_path(cfg) -> str:
    """File-store path shared by the ranks of one replica launch (keyed by port and driver pid)."""
    tag = os.environ.get("XV_RDV_TAG", str(os.getpid()))
    return os.path.join(tempfile.gettempdir(), f"xv_b200_rdv_{cfg.nccl_port}_{cfg.tp_size}_{cfg.pp_size}_{tag}")
