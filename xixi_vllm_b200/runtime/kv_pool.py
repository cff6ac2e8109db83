"""GPU-side KV storage (reference: src/compute/kv_pool.py:9-83).

One tensor ``[layers_local, 2, num_blocks, kv_heads_local, block_size, head_dim]``. Inside a
page the layout is head-major, so one head's 16 tokens are a contiguous 4 KiB run that a
single bulk copy can fetch. Only the local pipeline stage's layers and the local
tensor-parallel KV heads are stored.
"""

from __future__ import annotations

import torch

from ..parallel.groups import get_pp_group, get_tp_group, get_world_group
from ..parallel.pp import get_pp_indices

__all__ = ["KVPool", "get_kv_dims"]


def get_kv_dims(hf_config) -> tuple[int, int, int]:
    """(local layers, local kv heads, head_dim) for this rank."""
    tp, pp = get_tp_group(), get_pp_group()
    lo, hi = get_pp_indices(hf_config.num_hidden_layers, pp.group_rank, pp.size)
    kv_heads = hf_config.num_key_value_heads
    local_heads = 1 if tp.size >= kv_heads else kv_heads // tp.size
    return hi - lo, local_heads, hf_config.head_dim


class KVPool:
    def __init__(self, hf_config, *, num_blocks: int, block_size: int, device, dtype) -> None:
        if num_blocks <= 0:
            raise ValueError(f"num_blocks must be > 0, got {num_blocks}")
        self.num_layers, self.num_kv_heads, self.head_dim = get_kv_dims(hf_config)
        self.num_blocks_total = num_blocks
        self.block_size = block_size
        self.dtype = dtype
        self.device = torch.device(device)
        self.kv_cache = torch.zeros(
            (self.num_layers, 2, num_blocks, self.num_kv_heads, block_size, self.head_dim),
            dtype=dtype, device=self.device)

    def k_cache(self, layer: int) -> torch.Tensor:
        return self.kv_cache[layer, 0]

    def v_cache(self, layer: int) -> torch.Tensor:
        return self.kv_cache[layer, 1]

    @property
    def bytes_per_block(self) -> int:
        return self.block_bytes(self.num_layers, self.num_kv_heads, self.head_dim, self.block_size, self.dtype)

    @staticmethod
    def block_bytes(layers: int, kv_heads: int, head_dim: int, block_size: int, dtype) -> int:
        return 2 * layers * kv_heads * block_size * head_dim * torch.empty((), dtype=dtype).element_size()

    @staticmethod
    def auto_num_blocks(hf_config, *, block_size: int, dtype, device, gpu_memory_utilization: float,
                        reserve_bytes: int = 0, max_useful_tokens: int | None = None) -> int:
        """Pages that fit in ``utilization * total - already used - reserve``, the minimum over
        all ranks of the replica so every rank agrees on the page-id space."""
        layers, heads, hd = get_kv_dims(hf_config)
        per = KVPool.block_bytes(layers, heads, hd, block_size, dtype)
        device = torch.device(device)
        if device.type == "cuda":
            free, total = torch.cuda.mem_get_info(device)
            budget = int(total * gpu_memory_utilization) - (total - free) - reserve_bytes
        else:
            budget = 256 << 20
        n = max(budget // per, 0)
        if max_useful_tokens is not None:
            n = min(n, -(-max_useful_tokens // block_size))
        world = get_world_group()
        if world.size > 1:
            import torch.distributed as dist

            t = torch.tensor([n], dtype=torch.int64)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=world.cpu_group)
            n = int(t.item())
        if n <= 0:
            raise RuntimeError("no memory left for the KV cache; lower the model size or raise gpu_memory_utilization")
        return int(n)
