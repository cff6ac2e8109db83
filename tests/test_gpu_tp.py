"""Tensor-parallel GPU paths on 2 GPUs: fused peer-memory kernels vs NCCL + separate ops."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _fused_rank(rank, world, nvls):
    os.environ["XV_TP_NVLS"] = "1" if nvls else "0"
    import torch.distributed as dist

    from xixi_vllm_b200.ops import cpu_ref, cuda
    from xixi_vllm_b200.parallel.groups import get_tp_group
    from xixi_vllm_b200.parallel.symm import FusedTPComm
    dev = torch.device("cuda", rank)
    H = 1024
    comm = FusedTPComm(get_tp_group(), dev, H, 512, torch.bfloat16)
    errs = []
    for it, T in enumerate([1, 7, 64, 300, 512, 3, 3, 129]):
        g = torch.Generator().manual_seed(100 + it)
        parts = [torch.randn(T, H, generator=g).bfloat16() for _ in range(world)]
        resid = torch.randn(T, H, generator=g).bfloat16()
        w = (1 + 0.1 * torch.randn(H, generator=g)).bfloat16()
        comm.begin_forward()
        buf = comm.alloc_partial(T, final=(it % 3 == 2))
        buf.copy_(parts[rank].to(dev))
        use_res = it % 2 == 0
        r_dev = resid.to(dev).clone() if use_res else None
        y, r_out = comm.reduce_add_rmsnorm(buf, r_dev, w.to(dev), 1e-6)
        total = sum(p.float() for p in parts)
        r_ref = (total + (resid.float() if use_res else 0)).bfloat16()
        y_ref = cpu_ref.rmsnorm(r_ref, w, 1e-6)
        errs.append(float((r_out.float().cpu() - r_ref.float()).abs().max()))
        errs.append(float((y.float().cpu() - y_ref.float()).abs().max()))
        # plain all-reduce through the same machinery
        buf2 = comm.alloc_partial(T)
        buf2.copy_(parts[rank].to(dev))
        s = comm.all_reduce(buf2)
        errs.append(float((s.float().cpu() - total).abs().max()))
    # vocab-parallel argmax: every rank must pick the global best
    g = torch.Generator().manual_seed(7)
    full = torch.randn(5, 4096, generator=g).bfloat16()
    full[2, 100] = 9.0
    full[2, 3000] = 9.0                      # tie across ranks resolves to the lower id
    per = 4096 // world
    local = full[:, rank * per:(rank + 1) * per].contiguous().to(dev)
    ids = comm.argmax(local, per, rank * per).cpu()
    want = full.float().argmax(-1)
    torch.cuda.synchronize()
    cuda.check_status(dev)
    dist.barrier()
    return max(errs), ids.tolist(), want.tolist(), bool(comm.mc_ptr)


@pytest.mark.parametrize("nvls", [False, True])
def test_fused_reduce_norm_and_argmax(nvls):
    _need(2)
    from dist_utils import run_ranks_gpu
    for err, ids, want, has_mc in run_ranks_gpu(_fused_rank, world=2, tp=2, args=(nvls,)):
        assert err < 0.08, err
        assert ids[2] == 100
        assert ids == want or all(a == b for i, (a, b) in enumerate(zip(ids, want)) if i != 2)


def _gen(model_dir, prompts, **kw):
    from xixi_vllm_b200 import Engine, EngineConfig, SamplingParams
    cfg = EngineConfig(model=model_dir, dtype="bfloat16", num_kvcache_blocks=256, max_num_seqs=16,
                       max_num_batched_tokens=256, context_len=512, **kw)
    eng = Engine(cfg)
    try:
        seqs = [eng.add_request(p, SamplingParams(max_tokens=10, ignore_eos=True)) for p in prompts]
        while eng.has_unfinished():
            eng.step()
        return [s.token_ids[s.num_prompt_tokens:] for s in seqs]
    finally:
        eng.destroy()


@pytest.mark.parametrize("comm,eager", [("nccl", True), ("fused", True), ("fused", False)])
def test_engine_tp2_matches_tp1(tmp_path, comm, eager):
    _need(2)
    from xixi_vllm_b200.models.synth import make_model_dir
    d = make_model_dir(str(tmp_path / "m"), "tiny", std=0.08, num_hidden_layers=2, hidden_size=512,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=1024,
                       vocab_size=2048, torch_dtype="bfloat16", tie_word_embeddings=False)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (5, 16, 40, 100)]
    ref = _gen(d, prompts)
    out = _gen(d, prompts, tp_size=2, tp_comm=comm, enforce_eager=eager, nccl_port=29811)
    same = sum(a == b for x, y in zip(ref, out) for a, b in zip(x[:3], y[:3]))
    assert same >= 10, (ref, out)       # first tokens agree; later ones may flip on bf16 near-ties
