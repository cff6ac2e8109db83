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
    q = cuda.qk_norm_rope_cache(qkv.to(DEV), qw.to(DEV), kw.to(DEV), 1e-6, cs.to(DEV), pos.to(DEV),
                                slots.to(DEV), kd, vd, hq, hkv, d)
    _close(q, q_ref, atol=3e-2, rtol=3e-2)
    _close(kd, kc_ref, atol=3e-2, rtol=3e-2)
    assert torch.equal(vd.cpu(), vc_ref)


def test_bounded_wait_reports_instead_of_hanging():
    """A device-side wait on a flag nobody sets gives up after its limit and reports status."""
    from xixi_vllm_b200.ops import cuda
    code = cuda.selftest_bounded_wait(limit=2000)
    assert code >> 16 == 99 and code & 0xFFFF == 6
    # the context is still usable afterwards
    assert float(torch.ones(4, device=DEV).sum().item()) == 4.0
