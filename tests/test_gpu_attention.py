"""Paged attention kernels (decode and prefill) against the PyTorch oracle."""
import pytest
import torch

from xixi_vllm_b200.ops import cpu_ref
from xixi_vllm_b200.runtime.staging import AttnBatch

pytestmark = pytest.mark.gpu
DEV = "cuda"
D = 128


def _make_cache(num_blocks, hkv, bs, seed):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(num_blocks, hkv, bs, D, generator=g).bfloat16()
    v = torch.randn(num_blocks, hkv, bs, D, generator=g).bfloat16()
    return k, v


def _run(q_lens, kv_lens, hq, hkv, bs=16, n_decode=0, seed=0, q_scale=1.0, poison=None):
    B = len(kv_lens)
    maxb = max(-(-l // bs) for l in kv_lens) + 1
    num_blocks = B * maxb + 3
    g = torch.Generator().manual_seed(seed + 100)
    perm = torch.randperm(num_blocks, generator=g)
    bt = torch.zeros(B, maxb, dtype=torch.int32)
    for b in range(B):
        bt[b] = perm[b * maxb:(b + 1) * maxb].to(torch.int32)
    k, v = _make_cache(num_blocks, hkv, bs, seed)
    if poison is not None:
        # Everything outside the sequences' tokens is NaN in K; in V it is NaN too, except that ``poison ==
        # "v_tail_zero"`` leaves zeros after the last token inside its page (what the append kernel guarantees).
        used_k = torch.zeros(num_blocks, bs, dtype=torch.bool)
        used_v = torch.zeros(num_blocks, bs, dtype=torch.bool)
        for b in range(B):
            for t in range(kv_lens[b]):
                used_k[bt[b, t // bs], t % bs] = True
                used_v[bt[b, t // bs], t % bs] = True
            if poison == "v_tail_zero" and kv_lens[b] % bs:
                blk = bt[b, kv_lens[b] // bs]
                v[blk, :, kv_lens[b] % bs:] = 0
                used_v[blk, kv_lens[b] % bs:] = True
        k[~used_k.unsqueeze(1).expand(-1, hkv, -1)] = float("nan")
        v[~used_v.unsqueeze(1).expand(-1, hkv, -1)] = float("nan")
    T = sum(q_lens)
    q = (torch.randn(T, hq * D, generator=g) * q_scale).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    kvl = torch.tensor(kv_lens, dtype=torch.int32)
    scale = D ** -0.5
    ref = cpu_ref.paged_attention(q.float(), torch.nan_to_num(k.float()), torch.nan_to_num(v.float()), cu, kvl, bt,
                                  scale, hq, hkv, D)
    from xixi_vllm_b200.ops import cuda
    attn = AttnBatch(cu_q=cu.to(DEV), kv_lens=kvl.to(DEV), block_tables=bt.to(DEV), num_seqs=B,
                     num_decode=n_decode, max_q_len=max(q_lens), max_kv_len=max(kv_lens), num_tokens=T)
    out = cuda.paged_attention(q.to(DEV), k.to(DEV), v.to(DEV), attn, scale, hq, hkv, D)
    torch.cuda.synchronize()
    cuda.check_status()
    torch.testing.assert_close(out.float().cpu(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("hq,hkv", [(16, 8), (32, 8), (8, 1), (4, 1), (16, 1)])
def test_decode_gqa_groups(hq, hkv):
    _run([1] * 5, [1, 15, 16, 17, 300], hq, hkv, n_decode=5)


def test_decode_page_boundaries_every_batch_size():
    for bsz in (1, 2, 3, 9, 17):
        lens = [((i * 37) % 95) + 1 for i in range(bsz)]
        _run([1] * bsz, lens, 16, 8, n_decode=bsz, seed=bsz)


def test_decode_long_context_uses_splits():
    _run([1, 1], [4000, 2049], 32, 8, n_decode=2)


def test_decode_empty_rows_give_zeros():
    _run([1, 1, 1], [0, 33, 0], 16, 8, n_decode=3)


def test_decode_block_size_32():
    _run([1] * 3, [31, 32, 70], 16, 8, bs=32, n_decode=3)


@pytest.mark.parametrize("hq,hkv", [(16, 8), (8, 1)])
def test_prefill_no_prefix(hq, hkv):
    lens = [1, 15, 16, 17, 63, 64, 65, 200]
    _run(lens, lens, hq, hkv)


def test_prefill_with_cached_prefix():
    _run([5, 64, 100, 17], [16 + 5, 32 + 64, 48 + 100, 512 + 17], 16, 8)


def test_mixed_decode_then_prefill():
    _run([1, 1, 1, 40, 130], [77, 16, 1, 40, 16 + 130], 32, 8, n_decode=3)


# ---- tcgen05 prefill kernel (chunks longer than 64 rows take it by default) ----

@pytest.mark.parametrize("bs", [16, 32, 64, 128, 256])
def test_prefill_tensor_core_kernel_page_sizes(bs):
    from xixi_vllm_b200.ops import cuda
    assert cuda.prefill_uses_tensor_cores(D, bs, 300)
    _run([300, 129, 70, 1], [300, 256 + 129, 70, 513], 16, 8, bs=bs, seed=bs)


def test_prefill_tensor_core_kernel_long_sequence_with_growing_maxima():
    # Large scores make row maxima jump by more than the lazy-rescale threshold between tiles.
    _run([1500, 640], [1500, 2048 + 640], 8, 2, q_scale=6.0, seed=3)


def test_prefill_tensor_core_and_warp_mma_kernels_agree_with_oracle(monkeypatch):
    lens = [128, 127, 129, 255, 257]
    _run(lens, lens, 16, 8, seed=5)
    monkeypatch.setenv("XV_ATTN_PREFILL", "mma")
    from xixi_vllm_b200.ops import cuda
    assert not cuda.prefill_uses_tensor_cores(D, 16, 300)
    _run(lens, lens, 16, 8, seed=5)


def test_prefill_tensor_core_kernel_unsupported_page_size_falls_back():
    from xixi_vllm_b200.ops import cuda
    assert not cuda.prefill_uses_tensor_cores(D, 48, 300)
    _run([200], [200], 16, 8, bs=48)


def test_prefill_tensor_core_kernel_one_head_per_cta_form():
    """Odd KV-group sizes (and the forced single-head form) use one head per CTA."""
    from xixi_vllm_b200.ops import cuda
    _run([300, 129], [300, 256 + 129], 8, 8, seed=11)            # group of 1: cannot pair heads
    _run([200], [200], 3, 1, seed=12)                            # group of 3
    cuda.prefill_pair_heads(False)
    try:
        _run([300, 129, 70, 1], [300, 256 + 129, 70, 513], 16, 8, seed=13)
    finally:
        cuda.prefill_pair_heads(True)


def test_poisoned_cache_does_not_leak_into_results():
    """NaN everywhere outside the live tokens: pages of other sequences, unused pages, and the rest of each
    last page. The warp-MMA kernels zero-fill what they do not need; the tcgen05 prefill kernel relies on the
    append kernel's zeroed V tail."""
    _run([1] * 4, [1, 15, 33, 300], 16, 8, n_decode=4, poison="all")                      # decode
    _run([5, 40, 64], [16 + 5, 40, 128 + 64 - 7], 16, 8, poison="all")                    # short chunks (warp-MMA)
    _run([300, 129, 70], [300, 256 + 129 - 3, 70], 16, 8, poison="v_tail_zero", seed=4)   # tcgen05
