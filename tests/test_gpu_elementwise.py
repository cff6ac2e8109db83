"""CUDA elementwise kernels against the fp32 PyTorch oracle."""
import pytest
import torch

from xixi_vllm_b200.ops import cpu_ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, atol=2e-2, rtol=2e-2):
    torch.testing.assert_close(a.float().cpu(), b.float().cpu(), atol=atol, rtol=rtol)


@pytest.mark.parametrize("rows,hidden", [(1, 1024), (7, 4096), (33, 5120), (256, 2048), (3, 8192)])
def test_rmsnorm(rows, hidden):
    from xixi_vllm_b200.ops import cuda
    g = torch.Generator().manual_seed(rows * hidden)
    x = torch.randn(rows, hidden, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16()
    y = cuda.rmsnorm(x.to(DEV), w.to(DEV), 1e-6)
    _close(y, cpu_ref.rmsnorm(x.float(), w.float(), 1e-6))


@pytest.mark.parametrize("rows,hidden", [(1, 1024), (17, 4096), (64, 5120)])
def test_add_rmsnorm(rows, hidden):
    from xixi_vllm_b200.ops import cuda
    g = torch.Generator().manual_seed(1)
    x = torch.randn(rows, hidden, generator=g).bfloat16()
    r = torch.randn(rows, hidden, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16()
    rd = r.to(DEV).clone()
    y = cuda.add_rmsnorm(x.to(DEV), rd, w.to(DEV), 1e-6)
    r_ref = r.clone()
    y_ref = cpu_ref.add_rmsnorm(x, r_ref, w, 1e-6)
    _close(rd, r_ref, atol=1e-2, rtol=1e-2)
    _close(y, y_ref)


@pytest.mark.parametrize("rows,inter", [(1, 3072), (19, 12288), (300, 1536)])
def test_silu_mul(rows, inter):
    from xixi_vllm_b200.ops import cuda
    x = torch.randn(rows, 2 * inter, generator=torch.Generator().manual_seed(2)).bfloat16()
    _close(cuda.silu_mul(x.to(DEV)), cpu_ref.silu_mul(x.float()))


def test_embedding_and_gather():
    from xixi_vllm_b200.ops import cuda
    g = torch.Generator().manual_seed(3)
    w = torch.randn(500, 1024, generator=g).bfloat16()
    ids = torch.tensor([0, 5, 499, 500, 1200, 100, 99], dtype=torch.int32)
    y = cuda.embedding(ids.to(DEV), w.to(DEV), 100)     # shard owns ids [100, 600)
    ref = cpu_ref.embedding(ids, w, 100)
    assert torch.equal(y.cpu(), ref)
    rows = torch.tensor([3, 0, 3, 6], dtype=torch.int32)
    assert torch.equal(cuda.gather_rows(y, rows.to(DEV)).cpu(), ref[rows.long()])


@pytest.mark.parametrize("hq,hkv,d", [(16, 8, 128), (4, 1, 128), (32, 8, 128), (4, 2, 64)])
def test_qk_norm_rope_cache(hq, hkv, d):
    from xixi_vllm_b200.ops import cuda
    g = torch.Generator().manual_seed(4)
    T, bs, nblocks = 37, 16, 12
    qkv = torch.randn(T, (hq + 2 * hkv) * d, generator=g).bfloat16()
    qw = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16()
    kw = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16()
    cs = cpu_ref.build_cos_sin_cache(d, 512, 1e6)
    pos = torch.randint(0, 512, (T,), generator=g, dtype=torch.int32)
    slots = torch.randperm(nblocks * bs, generator=g)[:T].to(torch.int32)
    slots[5] = -1
    kc = torch.zeros(nblocks, hkv, bs, d).bfloat16()
    vc = torch.zeros_like(kc)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    q_ref = cpu_ref.qk_norm_rope_cache(qkv, qw, kw, 1e-6, cs, pos, slots, kc_ref, vc_ref, hq, hkv, d)
    kd, vd = kc.to(DEV), vc.to(DEV)
    # scattered slots (several rows of a page in arbitrary order): all rows count as decode rows, so no
    # page tail is cleared; the clearing after prefill chunks has its own test below
    q = cuda.qk_norm_rope_cache(qkv.to(DEV), qw.to(DEV), kw.to(DEV), 1e-6, cs.to(DEV), pos.to(DEV),
                                slots.to(DEV), kd, vd, hq, hkv, d, prefill_begin=T)
    _close(q, q_ref, atol=3e-2, rtol=3e-2)
    _close(kd, kc_ref, atol=3e-2, rtol=3e-2)
    assert torch.equal(vd.cpu(), vc_ref)


def test_kv_append_clears_v_rows_after_a_prefill_chunk():
    """Poisoned pages: after the last row a prefill chunk writes into a page the remaining V rows are
    zero (the tcgen05 prefill kernel multiplies them by P = 0); decode rows and other pages are untouched."""
    from xixi_vllm_b200.ops import cuda
    hq, hkv, d, bs, nblocks = 4, 2, 128, 16, 6
    g = torch.Generator().manual_seed(8)
    # row 0: a decode token at slot 3 of page 5; rows 1..20: a chunk filling page 2 and 4 rows of page 0;
    # rows 21..23: a chunk of 3 rows starting at row 6 of page 3
    slots = torch.tensor([5 * bs + 3] + [2 * bs + i for i in range(16)] + [0 * bs + i for i in range(4)] +
                         [3 * bs + 6 + i for i in range(3)], dtype=torch.int32)
    T = slots.numel()
    qkv = torch.randn(T, (hq + 2 * hkv) * d, generator=g).bfloat16()
    w = torch.ones(d).bfloat16()
    cs = cpu_ref.build_cos_sin_cache(d, 64, 1e6)
    pos = torch.arange(T, dtype=torch.int32)
    kd = torch.full((nblocks, hkv, bs, d), float("nan")).bfloat16().to(DEV)
    vd = torch.full((nblocks, hkv, bs, d), float("nan")).bfloat16().to(DEV)
    cuda.qk_norm_rope_cache(qkv.to(DEV), w.to(DEV), w.to(DEV), 1e-6, cs.to(DEV), pos.to(DEV), slots.to(DEV), kd, vd,
                            hq, hkv, d, prefill_begin=1)
    v = vd.float().cpu()
    assert torch.isfinite(v[2]).all()                                   # page 2 fully written
    assert torch.isfinite(v[0, :, :4]).all() and (v[0, :, 4:] == 0).all()    # chunk ended at row 3 of page 0
    assert torch.isnan(v[3, :, :6]).all() and torch.isfinite(v[3, :, 6:9]).all() and (v[3, :, 9:] == 0).all()
    assert torch.isfinite(v[5, :, 3]).all() and torch.isnan(v[5, :, 4:]).all()   # decode row: nothing cleared
    assert torch.isnan(v[1]).all() and torch.isnan(v[4]).all()          # pages nobody wrote
    k = kd.float().cpu()
    assert torch.isnan(k[0, :, 4:]).all()                               # K rows are never cleared (they get masked)


def test_bounded_wait_reports_instead_of_hanging():
    """A device-side wait on a flag nobody sets gives up after its limit and reports status."""
    from xixi_vllm_b200.ops import cuda
    code = cuda.selftest_bounded_wait(limit=2000)
    assert code >> 16 == 99 and code & 0xFFFF == 6
    # the context is still usable afterwards
    assert float(torch.ones(4, device=DEV).sum().item()) == 4.0


@pytest.fixture
def planes_split_k():
    """K splits as fp32 planes (by default up to four splits are summed inside a thread-block cluster)."""
    from xixi_vllm_b200.ops import cuda
    cuda.gemm_plan_override(0, 0, 4, 0)
    yield
    cuda.gemm_plan_override(-1)


def test_split_k_partials_feed_consumers_directly(planes_split_k):
    """A deferred split-K GEMM hands fp32 partial planes to add+RMSNorm and to QK-norm/RoPE."""
    from xixi_vllm_b200.ops import cuda
    g = torch.Generator().manual_seed(9)
    x = (torch.randn(24, 2048, generator=g) * 0.3).bfloat16().to(DEV)
    w = (torch.randn(1024, 2048, generator=g) * 0.05).bfloat16().to(DEV)
    part = cuda.linear(x, w, defer=True)
    assert isinstance(part, cuda.SplitKPartial) and part.splits > 1
    dense = cuda.linear(x, w)
    _close(part.materialize(), dense, atol=2e-2, rtol=2e-2)
    res = torch.randn(24, 1024, generator=g).bfloat16().to(DEV)
    nw = (1 + 0.1 * torch.randn(1024, generator=g)).bfloat16().to(DEV)
    r1, r2 = res.clone(), res.clone()
    part = cuda.linear(x, w, defer=True)
    y1 = cuda.add_rmsnorm(part, r1, nw, 1e-6)
    y2 = cuda.add_rmsnorm(dense, r2, nw, 1e-6)
    _close(r1, r2, atol=3e-2, rtol=3e-2)
    _close(y1, y2, atol=3e-2, rtol=3e-2)
    # QKV: 4 q heads + 2 x 2 kv heads of 128 = 1024 columns
    hq, hkv, d, T = 4, 2, 128, 24
    cs = cpu_ref.build_cos_sin_cache(d, 256, 1e6).to(DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    slots = torch.arange(T, dtype=torch.int32, device=DEV)
    qw = torch.ones(d, dtype=torch.bfloat16, device=DEV)
    caches = [torch.zeros(4, hkv, 16, d, dtype=torch.bfloat16, device=DEV) for _ in range(4)]
    part = cuda.linear(x, w, defer=True)
    qa = cuda.qk_norm_rope_cache(part, qw, qw, 1e-6, cs, pos, slots, caches[0], caches[1], hq, hkv, d)
    qb = cuda.qk_norm_rope_cache(dense, qw, qw, 1e-6, cs, pos, slots, caches[2], caches[3], hq, hkv, d)
    _close(qa, qb, atol=3e-2, rtol=3e-2)
    _close(caches[0], caches[2], atol=3e-2, rtol=3e-2)
    _close(caches[1], caches[3], atol=3e-2, rtol=3e-2)


def test_resolve_token_refs_kernel():
    from xixi_vllm_b200.ops import cuda
    prev = torch.tensor([900, 901, 902, 903], dtype=torch.int64, device="cuda")
    ids = torch.tensor([5, -1, -4, 7, -2, -9], dtype=torch.int32, device="cuda")
    cuda.resolve_token_refs(ids, prev)
    torch.cuda.synchronize()
    assert ids.tolist() == [5, 900, 903, 7, 901, 0]          # a reference beyond the buffer becomes token 0
