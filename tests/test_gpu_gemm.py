"""tcgen05 GEMM against an fp32 matmul of the same bf16 inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"

def assert_close_per_element(y, ref):
    """bf16 rounding of an fp32 accumulator is at most 2^-8 relative; every element is held to
    1e-2 * |ref| + 2^-8 * (largest |ref| of its row), so a dropped K block or a wrongly weighted split-K plane on
    a small tile cannot hide behind the matrix maximum."""
    err = (y.float() - ref).abs()
    tol = 1e-2 * ref.abs() + 2.0 ** -8 * ref.abs().amax(dim=-1, keepdim=True)
    bad = err > tol
    assert not bool(bad.any()), (f"{int(bad.sum())} elements off, worst {float((err - tol).max()):.4g} over the bound "
                                 f"at {tuple(torch.nonzero(bad)[0].tolist())}")


SHAPES = [
    # (M, N, K): swapped orientation, with and without split-K
    (1, 1024, 1024), (5, 4096, 4096), (16, 6144, 4096), (32, 4096, 12288), (100, 3072, 1024),
    (256, 24576, 4096), (256, 4096, 1536), (8, 768, 4096), (3, 1000, 512), (17, 136, 192),
    # normal orientation
    (257, 4096, 4096), (1024, 6144, 1024), (4096, 4096, 4096), (300, 1000, 2048), (777, 18992, 512),
]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_matches_fp32(m, n, k):
    from xixi_vllm_b200.ops import cuda
    g = torch.Generator().manual_seed(m * 7 + n * 3 + k)
    x = (torch.randn(m, k, generator=g) * 0.5).bfloat16().to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.5).bfloat16().to(DEV)
    y = cuda.linear(x, w)
    torch.cuda.synchronize()
    cuda.check_status()
    ref = x.float() @ w.float().t()
    assert_close_per_element(y, ref)


def test_gemm_repeated_calls_are_stable():
    from xixi_vllm_b200.ops import cuda
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 2048, generator=g).bfloat16().to(DEV)
    w = torch.randn(4096, 2048, generator=g).bfloat16().to(DEV)
    y0 = cuda.linear(x, w)
    for _ in range(20):
        y = cuda.linear(x, w)
    torch.cuda.synchronize()
    cuda.check_status()
    assert torch.equal(y, y0)


def test_gemm_strided_input_rows():
    """Activations that are a column slice of a wider buffer (row stride > K)."""
    from xixi_vllm_b200.ops import cuda
    g = torch.Generator().manual_seed(1)
    big = torch.randn(48, 4096, generator=g).bfloat16().to(DEV)
    x = big[:, 1024:3072]
    w = torch.randn(512, 2048, generator=g).bfloat16().to(DEV)
    y = cuda.linear(x, w)
    ref = x.float() @ w.float().t()
    assert_close_per_element(y, ref)


def _interleave(gate, up, g=8):
    n, k = gate.shape
    return torch.stack([gate.view(n // g, g, k), up.view(n // g, g, k)], 1).reshape(2 * n, k)


@pytest.mark.parametrize("m,inter,k", [(5, 1536, 1024), (64, 3072, 4096), (256, 12288, 1024), (200, 512, 2048),
                                       (1000, 1536, 1024), (4096, 3072, 512)])
def test_gemm_with_fused_silu_mul(m, inter, k):
    """Swapped, normal and split-K plans of the gate/up projection with the activation fused."""
    from xixi_vllm_b200.ops import cuda
    g = torch.Generator().manual_seed(m + inter)
    x = (torch.randn(m, k, generator=g) * 0.5).bfloat16().to(DEV)
    gate = (torch.randn(inter, k, generator=g) * 0.05).bfloat16().to(DEV)
    up = (torch.randn(inter, k, generator=g) * 0.05).bfloat16().to(DEV)
    y = cuda.linear_silu_mul(x, _interleave(gate, up).contiguous())
    torch.cuda.synchronize()
    cuda.check_status()
    gf, uf = x.float() @ gate.float().t(), x.float() @ up.float().t()
    ref = torch.nn.functional.silu(gf) * uf
    assert y.shape == (m, inter)
    assert (y.float() - ref).abs().max().item() <= 3e-2 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("m,n,k", [(2048, 4096, 1024), (4096, 6144, 4096), (1500, 9000, 512), (19 * 256, 1024, 2048)])
def test_cta_pair_kernel_matches_single_cta_kernel(m, n, k):
    """Large-M problems run on CTA pairs (cta_group::2); forcing the single-CTA kernel must agree."""
    from xixi_vllm_b200.ops import cuda
    L = cuda.lib()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert cuda.gemm_plan(m, n, k, sms).pair == 1
    g = torch.Generator().manual_seed(m + n + k)
    x = (torch.randn(m, k, generator=g) * 0.5).bfloat16().to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.5).bfloat16().to(DEV)
    y_pair = cuda.linear(x, w)
    L.xv_gemm_disable_pair(1)
    try:
        assert cuda.gemm_plan(m, n, k, sms).pair == 0
        y_single = cuda.linear(x, w)
    finally:
        L.xv_gemm_disable_pair(0)
    torch.cuda.synchronize()
    cuda.check_status()
    ref = x.float() @ w.float().t()
    assert_close_per_element(y_pair, ref)
    assert_close_per_element(y_single, ref)
    # tiles that the pairs deal in K blocks are summed from two or three fp32 partial sums
    assert (y_pair.float() - y_single.float()).abs().max().item() <= 1e-2 * ref.abs().max().item()


@pytest.mark.parametrize("m,n,k,parts", [(1400, 4096, 4096, 3), (512, 4096, 12288, 2), (1400, 4096, 1024, 3)])
def test_cta_pair_kernel_splits_last_wave_in_k(m, n, k, parts):
    """When the last wave of 256-row tiles leaves most SM pairs idle its tiles are cut into K parts whose fp32
    accumulators meet in a slot of the workspace. The result matches fp32, repeats bit for bit (a slot takes
    at most two contributions, which commute) and leaves slots and counters zero for the next launch."""
    from xixi_vllm_b200.ops import cuda
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    if sms != 148:
        pytest.skip("plan under test is the one for 148 SMs")
    pl = cuda.gemm_plan(m, n, k, sms)
    assert pl.pair == 1 and pl.sk_tiles > 0 and pl.sk_parts == parts
    g = torch.Generator().manual_seed(m + n + k)
    x = (torch.randn(m, k, generator=g) * 0.5).bfloat16().to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.5).bfloat16().to(DEV)
    ref = x.float() @ w.float().t()
    first = cuda.linear(x, w)
    for _ in range(3):
        again = cuda.linear(x, w)
        assert torch.equal(first, again)
    torch.cuda.synchronize()
    cuda.check_status()
    assert_close_per_element(first, ref)


@pytest.fixture
def swapped_pairs():
    from xixi_vllm_b200.ops import cuda
    cuda.gemm_plan_override(3, 0, 0, 0)
    yield
    cuda.gemm_plan_override(-1, 0, 0, 0)


@pytest.mark.parametrize("m,n,k", [(256, 6144, 4096), (200, 4096, 4096), (161, 4096, 12288), (256, 24576, 1024),
                                   (256, 1024, 512), (250, 3080, 4096)])
def test_decode_batch_runs_on_swapped_cta_pairs(m, n, k, swapped_pairs):
    """161..256 rows: weights on the pairs' 256-row M axis, all tokens in one N tile, transposed epilogue
    (and K parts when the weight tiles do not fill the SM pairs)."""
    from xixi_vllm_b200.ops import cuda
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    pl = cuda.gemm_plan(m, n, k, sms)
    assert pl.pair == 1 and pl.swapped == 1 and pl.tiles_b == 1
    g = torch.Generator().manual_seed(m + n + k)
    x = (torch.randn(m, k, generator=g) * 0.5).bfloat16().to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.5).bfloat16().to(DEV)
    ref = x.float() @ w.float().t()
    y = cuda.linear(x, w)
    again = cuda.linear(x, w)
    torch.cuda.synchronize()
    cuda.check_status()
    assert torch.equal(y, again)
    assert_close_per_element(y, ref)


def test_decode_batch_swapped_cta_pairs_fused_silu_mul(swapped_pairs):
    from xixi_vllm_b200.ops import cuda
    m, inter, k = 256, 3072, 4096
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    pl = cuda.gemm_plan(m, 2 * inter, k, sms)
    assert pl.pair == 1 and pl.swapped == 1
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(m, k, generator=g) * 0.5).bfloat16().to(DEV)
    gate = (torch.randn(inter, k, generator=g) * 0.05).bfloat16().to(DEV)
    up = (torch.randn(inter, k, generator=g) * 0.05).bfloat16().to(DEV)
    y = cuda.linear_silu_mul(x, _interleave(gate, up).contiguous())
    torch.cuda.synchronize()
    cuda.check_status()
    ref = torch.nn.functional.silu(x.float() @ gate.float().t()) * (x.float() @ up.float().t())
    assert y.shape == (m, inter)
    assert (y.float() - ref).abs().max().item() <= 3e-2 * ref.abs().max().item() + 1e-2
