"""The allocation-free GEMM entry point, called through its exported C symbol.

Some callers of this library cannot create GPU allocations at call time (a plug-in running
inside another runtime's execute callback, or a serving loop whose memory pool is frozen).
``xv_gemm_bf16_noalloc`` serves them from a fixed scratch buffer compiled into the library.
This file is named so that pytest collects it last.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _sym():
    from xixi_vllm_b200.ops import cuda
    L = cuda.lib()
    f = L.xv_gemm_bf16_noalloc
    f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                  ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p]
    f.restype = ctypes.c_int
    L.xv_gemm_noalloc_max_scratch_bytes.restype = ctypes.c_longlong
    L.xv_gemm_plan_planes.argtypes = [ctypes.c_int] * 4 + [ctypes.POINTER(cuda.GemmPlan)]
    return L, f


def _plan(L, m, n, k):
    """The plan the allocation-free entry point runs (its K splits always go through the scratch buffer)."""
    from xixi_vllm_b200.ops import cuda
    pl = cuda.GemmPlan()
    assert L.xv_gemm_plan_planes(m, n, k, torch.cuda.get_device_properties(0).multi_processor_count, ctypes.byref(pl)) == 0
    return pl


def test_noalloc_gemm_matches_workspace_gemm_twice_in_a_row():
    from xixi_vllm_b200.ops import cuda
    L, f = _sym()
    assert L.xv_gemm_noalloc_max_scratch_bytes() == 16 << 20
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for m, n, k in [(32, 4096, 4096), (7, 1024, 2048)]:        # both plans split K and use the scratch
        assert _plan(L, m, n, k).workspace_bytes > 0
        g = torch.Generator().manual_seed(m + n)
        x = torch.randn(m, k, generator=g).bfloat16().cuda()
        w = torch.randn(n, k, generator=g).bfloat16().cuda()
        want = cuda.linear(x, w)                                 # existing entry point, caller-owned workspace
        for _ in range(2):
            y = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
            rc = f(x.data_ptr(), w.data_ptr(), y.data_ptr(), m, n, k, k, k, n, status.data_ptr(), stream)
            assert rc == 0
            torch.cuda.synchronize()
            torch.testing.assert_close(y.float(), want.float(), atol=2e-2, rtol=2e-2)
        ref = x.float() @ w.float().t()
        assert (y.float() - ref).abs().max() <= 2e-2 * ref.abs().max() + 1e-2
    assert int(status.item()) == 0


def test_noalloc_gemm_rejects_oversized_problem(capfd):
    from xixi_vllm_b200.ops import cuda
    L, f = _sym()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    m, n, k = 128, 16640, 8192          # two split-K planes of 8.1 MiB each
    need = _plan(L, m, n, k).workspace_bytes
    assert need > L.xv_gemm_noalloc_max_scratch_bytes()
    x = torch.zeros(m, k, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(n, k, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
    rc = f(x.data_ptr(), w.data_ptr(), y.data_ptr(), m, n, k, k, k, n, None, torch.cuda.current_stream().cuda_stream)
    assert rc == -3
    assert "needs" in capfd.readouterr().err
