"""Whole engine on CPU: oracle model vs a dense re-implementation, TP/PP/DP equal single rank."""
import math

import pytest
import torch

from xixi_vllm_b200 import Engine, EngineConfig, SamplingParams
from xixi_vllm_b200.models.loader import SafetensorsSource


def _prompts(n=4, length=16, vocab=1024, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]


def _generate(model_dir, prompts, max_tokens=8, **kw):
    base = dict(device="cpu", dtype="float32", num_kvcache_blocks=128, max_num_seqs=8, max_num_batched_tokens=64,
                context_len=256)
    base.update(kw)
    eng = Engine(EngineConfig(model=model_dir, **base))
    try:
        seqs = [eng.add_request(p, SamplingParams(max_tokens=max_tokens, ignore_eos=True)) for p in prompts]
        while eng.has_unfinished():
            eng.step()
        return [s.token_ids[s.num_prompt_tokens:] for s in seqs]
    finally:
        eng.destroy()


def _dense_greedy(model_dir, prompt, n_new):
    """Straightforward full-sequence Qwen3 forward (no paging, no batching) as an independent check."""
    from xixi_vllm_b200.config import load_model_config
    c = load_model_config(model_dir)
    src = SafetensorsSource(model_dir)
    W = {n: src.read(n).double() for n in src.names()}
    H, D, nq, nkv = c.hidden_size, c.head_dim, c.num_attention_heads, c.num_key_value_heads

    def norm(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + c.rms_norm_eps) * w

    ids = list(prompt)
    for _ in range(n_new):
        T = len(ids)
        x = W["model.embed_tokens.weight"][ids]
        pos = torch.arange(T, dtype=torch.float64)
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
        ang = pos[:, None] * inv[None]
        cos, sin = ang.cos()[:, None], ang.sin()[:, None]

        def rope(t):
            a, b = t[..., : D // 2], t[..., D // 2:]
            return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)

        for i in range(c.num_hidden_layers):
            p = f"model.layers.{i}."
            h = norm(x, W[p + "input_layernorm.weight"])
            q = (h @ W[p + "self_attn.q_proj.weight"].t()).view(T, nq, D)
            k = (h @ W[p + "self_attn.k_proj.weight"].t()).view(T, nkv, D)
            v = (h @ W[p + "self_attn.v_proj.weight"].t()).view(T, nkv, D)
            q = rope(norm(q, W[p + "self_attn.q_norm.weight"]))
            k = rope(norm(k, W[p + "self_attn.k_norm.weight"]))
            k, v = k.repeat_interleave(nq // nkv, 1), v.repeat_interleave(nq // nkv, 1)
            s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(D)
            s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
            o = torch.einsum("hqk,khd->qhd", s.softmax(-1), v).reshape(T, nq * D)
            x = x + o @ W[p + "self_attn.o_proj.weight"].t()
            h = norm(x, W[p + "post_attention_layernorm.weight"])
            g, u = h @ W[p + "mlp.gate_proj.weight"].t(), h @ W[p + "mlp.up_proj.weight"].t()
            x = x + (torch.nn.functional.silu(g) * u) @ W[p + "mlp.down_proj.weight"].t()
        head = W.get("lm_head.weight", W["model.embed_tokens.weight"])
        ids.append(int((norm(x[-1], W["model.norm.weight"]) @ head.t()).argmax()))
    return ids[len(prompt):]


def test_engine_matches_dense_forward(tiny_model_dir):
    prompts = _prompts()
    got = _generate(tiny_model_dir, prompts)
    for p, g in zip(prompts, got):
        assert g == _dense_greedy(tiny_model_dir, p, 8)


def test_chunked_prefill_and_prefix_cache_do_not_change_tokens(tiny_model_dir):
    shared = _prompts(1, 40, seed=5)[0]
    prompts = [shared + p for p in _prompts(3, 30, seed=6)]
    base = _generate(tiny_model_dir, prompts, prefix_backend="none")
    for backend in ("hash", "radix"):
        for budget in (64, 24):                      # 24 forces chunked prefill
            assert _generate(tiny_model_dir, prompts, prefix_backend=backend,
                             max_num_batched_tokens=budget) == base


def test_preemption_under_kv_pressure_keeps_outputs(tiny_model_dir):
    prompts = _prompts(4, 24, seed=7)
    base = _generate(tiny_model_dir, prompts, max_tokens=24)
    tight = _generate(tiny_model_dir, prompts, max_tokens=24, num_kvcache_blocks=9, prefix_backend="none")
    assert tight == base


def test_one_step_late_scheduling_keeps_tokens(tiny_model_dir):
    """Launching step n + 1 before step n's samples are read (input tokens fetched from the previous step's
    sample buffer, EOS found one step late, preemption with a token in flight) changes no output."""
    prompts = _prompts(5, 24, seed=11)
    base = _generate(tiny_model_dir, prompts, max_tokens=20, async_scheduling="off")
    assert _generate(tiny_model_dir, prompts, max_tokens=20, async_scheduling="on") == base
    assert _generate(tiny_model_dir, prompts, max_tokens=20, async_scheduling="on", num_kvcache_blocks=9,
                     prefix_backend="none") == base                                   # preemption
    assert _generate(tiny_model_dir, prompts, max_tokens=20, async_scheduling="on", prefix_backend="radix",
                     max_num_batched_tokens=24) == base                               # chunked prefill + prefix cache
    assert _generate(tiny_model_dir, prompts, max_tokens=20, async_scheduling="on", tp_size=2,
                     nccl_port=29721) == base
    # EOS stops a request although its next step has already been launched
    eng = Engine(EngineConfig(model=tiny_model_dir, device="cpu", dtype="float32", num_kvcache_blocks=128,
                              max_num_seqs=8, max_num_batched_tokens=64, context_len=256, async_scheduling="on"))
    try:
        eos_like = base[0][3]
        core = eng._client.engine_core
        assert core.one_step_late
        core.scheduler.eos = eos_like
        seqs = [eng.add_request(p, SamplingParams(max_tokens=20)) for p in prompts]
        while eng.has_unfinished():
            eng.step()
        for s, b in zip(seqs, base):
            want = b[: b.index(eos_like) + 1] if eos_like in b else b
            assert s.token_ids[s.num_prompt_tokens:] == want and s.num_pending == 0
    finally:
        eng.destroy()


def test_tp2_equals_tp1(tiny_model_dir):
    """Benchmark config 1: tiny fp32 Qwen3, gloo world of 2, 4 prompts x 16 ids, greedy 8 tokens."""
    prompts = _prompts()
    assert _generate(tiny_model_dir, prompts, tp_size=2, nccl_port=29711) == _generate(tiny_model_dir, prompts)


def test_pp2_and_tp2pp2_equal_single_rank(tiny_model_dir):
    prompts = _prompts(3, 20, seed=1)
    base = _generate(tiny_model_dir, prompts)
    assert _generate(tiny_model_dir, prompts, pp_size=2, nccl_port=29721) == base
    assert _generate(tiny_model_dir, prompts, tp_size=2, pp_size=2, nccl_port=29731) == base


@pytest.mark.parametrize("kw", [dict(pp_size=2, pp_microbatches=2, nccl_port=29761),
                                dict(pp_size=2, pp_microbatches=3, max_num_batched_tokens=24, nccl_port=29771),
                                dict(tp_size=2, pp_size=2, pp_microbatches=2, nccl_port=29781)])
def test_pp_microbatches_equal_single_rank(tiny_model_dir, kw):
    """Pipeline stages that work on pieces of every step (decodes, whole prompts and mid-prompt chunks end up
    in different pieces) must produce the tokens of the single-rank engine."""
    prompts = _prompts(5, 20, seed=4) + _prompts(1, 50, seed=5)
    base = _generate(tiny_model_dir, prompts, max_tokens=6)
    assert _generate(tiny_model_dir, prompts, max_tokens=6, **kw) == base


def test_uneven_pp_layer_counts(tmp_path):
    from xixi_vllm_b200.models.synth import make_model_dir
    d = make_model_dir(str(tmp_path / "m3"), "tiny", num_hidden_layers=3)
    prompts = _prompts(2, 12, seed=2)
    assert _generate(d, prompts, pp_size=2, pp_layer_counts=[1, 2], nccl_port=29741) == _generate(d, prompts)


def test_dp2_replicas_equal_single_engine(tiny_model_dir):
    prompts = _prompts(4, 16, seed=3)
    base = _generate(tiny_model_dir, prompts)
    assert _generate(tiny_model_dir, prompts, dp_size=2, nccl_port=29751) == base


def test_generate_stream_and_batch_api(tiny_model_dir):
    eng = Engine(EngineConfig(model=tiny_model_dir, device="cpu", dtype="float32", num_kvcache_blocks=64,
                              max_num_seqs=4, max_num_batched_tokens=64, context_len=64))
    try:
        pieces = list(eng.generate([5, 6, 7], max_new_tokens=4))
        assert len(pieces) == 4
        texts = eng.generate_batch([[1, 2, 3], "ab"], SamplingParams(max_tokens=3, ignore_eos=True))
        assert len(texts) == 2 and all(isinstance(t, str) for t in texts)
        with pytest.warns(UserWarning, match="truncating"):
            s = eng.add_request(list(range(100)), SamplingParams(max_tokens=5))
        assert s.num_prompt_tokens == 64 and s.max_tokens == 0
        while eng.has_unfinished():
            eng.step()
        eng.reset_kv("radix")
        assert eng.scheduler.kv.prefix_backend == "radix"
        with pytest.raises(ValueError):
            eng.add_request([])
    finally:
        eng.destroy()


def test_sampled_generation_is_seeded(tiny_model_dir):
    def run(seed):
        eng = Engine(EngineConfig(model=tiny_model_dir, device="cpu", dtype="float32", num_kvcache_blocks=64,
                                  max_num_seqs=4, max_num_batched_tokens=64, context_len=64, seed=seed))
        try:
            s = eng.add_request([3, 4, 5], SamplingParams(temperature=1.0, top_k=50, top_p=0.9, max_tokens=12,
                                                          ignore_eos=True))
            while eng.has_unfinished():
                eng.step()
            return s.token_ids[3:]
        finally:
            eng.destroy()
    assert run(1) == run(1)
    assert run(1) != run(2)


def _cli(args, timeout=300):
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable] + args, cwd=root, capture_output=True, text=True, timeout=timeout)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    lines = [ln for ln in p.stdout.splitlines() if ln.startswith("hello world")]
    assert lines, p.stdout[-2000:]
    return lines[-1]


def test_command_lines_generate_the_same_text(tiny_model_dir):
    """``run.py`` in one process, ``run_torchrun.py`` under torchrun with TP=2 and with two pipeline stages
    working on pieces of each step: the same greedy continuation of the same prompt."""
    common = ["--model", tiny_model_dir, "--device", "cpu", "--max-new-tokens", "5", "--prompt", "hello world"]
    single = _cli(["run.py"] + common)
    launch = ["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1"]
    assert _cli(launch + ["--master-port", "29921", "run_torchrun.py", "--tp", "2"] + common) == single
    assert _cli(launch + ["--master-port", "29922", "run_torchrun.py", "--tp", "1", "--pp", "2",
                          "--pp-microbatches", "2"] + common) == single
