"""ctypes bindings of the sm_100a kernel library (``_xv_cuda.so``, built by ``ops.build``).

Tensors are passed as raw device pointers together with the current CUDA stream; outputs
are allocated with torch so they live in its caching allocator (and in CUDA-graph pools
during capture). Only bf16 activations and weights are supported on the GPU. A missing
library raises: there is no silent fallback to library kernels.

``XV_GEMM=cublas`` in the environment swaps the GEMM for ``torch.matmul`` (cuBLAS); it
exists to A/B the hand-written kernel and to bisect numerical differences.
"""

from __future__ import annotations

import ctypes
import os

import torch

from . import build as _build

__all__ = [
    "lib", "rmsnorm", "add_rmsnorm", "linear", "silu_mul", "embedding", "gather_rows",
    "qk_norm_rope_cache", "paged_attention", "prefill_pair_heads", "prefill_phase_profile", "argmax", "sample", "check_status", "gemm_plan",
    "decode_splits", "launch_count",
]

_lib = None
_vp, _i32, _i64, _f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float

ERRORS = {-1: "bad shape", -2: "misaligned pointer or stride", -3: "workspace too small",
          -4: "driver entry point missing", -5: "tensor map encode failed", -6: "launch failed",
          -7: "unsupported configuration"}

# number of kernel launches issued through this module (bench.py reports it)
launch_count = 0


class GemmPlan(ctypes.Structure):
    _fields_ = [("swapped", _i32), ("bn", _i32), ("tiles_a", _i32), ("tiles_b", _i32), ("splits", _i32),
                ("k_blocks_per_split", _i32), ("stages", _i32), ("smem_bytes", _i32),
                ("ctas_per_sm", _i32), ("cluster", _i32), ("pair", _i32), ("sk_tiles", _i32), ("sk_parts", _i32), ("units_per_pair", _i32),
                ("workspace_bytes", _i64)]


def lib():
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB
    if not os.path.isfile(path) or _build.needs_build():
        path = _build.build()
    L = ctypes.CDLL(path)
    L.xv_gemm_plan.argtypes = [_i32, _i32, _i32, _i32, ctypes.POINTER(GemmPlan)]
    L.xv_gemm_bf16.argtypes = [_vp, _vp, _vp, _i32, _i32, _i32, _i64, _i64, _i64, _vp, _i64, _i32, _vp, _vp]
    L.xv_gemm_bf16_defer.argtypes = [_vp, _vp, _vp, _i32, _i32, _i32, _i64, _i64, _i64, _vp, _i64, _i32, _vp, _vp,
                                     ctypes.POINTER(_i32)]
    L.xv_add_rmsnorm_partials.argtypes = [_vp, _i32, _i64, _vp, _vp, _vp, _i32, _i32, _f32, _vp]
    L.xv_qk_norm_rope_cache_partials.argtypes = [_vp, _i32, _i64, _vp, _vp, _f32, _vp, _vp, _vp, _vp, _vp, _vp,
                                                 _i32, _i32, _i32, _i32, _i32, _i32, _vp]
    L.xv_gemm_bf16_silu_mul.argtypes = [_vp, _vp, _vp, _i32, _i32, _i32, _i64, _i64, _i64, _vp, _i64, _i32, _vp, _vp]
    L.xv_silu_mul_interleaved.argtypes = [_vp, _vp, _i32, _i64, _vp, _i32, _i32, _vp]
    L.xv_rmsnorm.argtypes = [_vp, _vp, _vp, _i32, _i32, _f32, _vp]
    L.xv_add_rmsnorm.argtypes = [_vp, _vp, _vp, _vp, _i32, _i32, _f32, _vp]
    L.xv_silu_mul.argtypes = [_vp, _vp, _i32, _i32, _vp]
    L.xv_embedding.argtypes = [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]
    L.xv_gather_rows.argtypes = [_vp, _vp, _vp, _i32, _i32, _vp]
    L.xv_resolve_token_refs.argtypes = [_vp, _i32, _vp, _i32, _vp]
    L.xv_qk_norm_rope_cache.argtypes = [_vp, _vp, _vp, _f32, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32,
                                        _i32, _i32, _i32, _vp]
    L.xv_attn_decode_workspace_bytes.argtypes = [_i32, _i32, _i32, _i32]
    L.xv_attn_decode_workspace_bytes.restype = _i64
    L.xv_attn_decode.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _i32,
                                 _vp, _vp]
    L.xv_attn_prefill.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32,
                                  _i32, _f32, _vp]
    L.xv_attn_prefill_tc_supported.argtypes = [_i32, _i32]
    L.xv_attn_prefill_tc_single_unit.argtypes = [_i32]
    L.xv_attn_prefill_tc_single_unit.restype = None
    L.xv_attn_prefill_tc.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32,
                                     _i32, _i32, _i32, _f32, _vp, _vp]
    L.xv_attn_prefill_tc_profile.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32,
                                             _i32, _i32, _i32, _f32, _vp, _vp, _vp]
    L.xv_argmax.argtypes = [_vp, _vp, _i32, _i32, _i64, _vp]
    L.xv_sample.argtypes = [_vp, _vp, _i32, _i32, _i64, _vp, _vp, _vp, _vp, _vp, _vp]
    L.xv_tp_reduce_norm.argtypes = [_vp, _vp, _vp, _vp, _i32, _i32, _i64, _vp, _vp, _vp, _vp, _i32, _i32, _f32,
                                    _i32, ctypes.c_uint, _vp, _vp]
    L.xv_tp_reduce_norm_sharded.argtypes = [_vp, _vp, _vp, _vp, _i32, _i32, _i64, _i64, _i32, _vp, _vp, _i32, _i32,
                                            _f32, ctypes.c_uint, _vp, _vp]
    L.xv_tp_allgather_cols.argtypes = [_vp, _vp, _vp, _vp, _i32, _i32, _vp, _i64, _i32, _i64, _i32, ctypes.c_uint,
                                       _vp, _vp]
    L.xv_tp_argmax.argtypes = [_vp, _vp, _vp, _i32, _i32, _i64, _vp, _i64, _i32, _i32, _i32, _vp, _i32,
                               ctypes.c_uint, _vp, _vp]
    L.xv_gemm_bf16_tp.argtypes = [_vp, _vp, _i32, _i32, _i32, _i64, _i64, _vp, _i64, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i64,
                                  _i64, _i32, _i64, _vp, _vp, _vp, _vp, _f32, _i32, _i32, ctypes.c_uint, _vp, _vp]
    L.xv_tp_sample_region_bytes.argtypes = [_i32, _i32]
    L.xv_tp_sample_region_bytes.restype = _i64
    L.xv_tp_sample.argtypes = [_vp, _vp, _vp, _i32, _i32, _i64, _i32, _vp, _i64, _i32, _i32, _i32, _vp, _i32, _vp, _vp,
                               _vp, _vp, _vp, ctypes.c_uint, _vp, _vp]
    L.xv_gemm_plan_override.argtypes = [_i32, _i32, _i32, _i32]
    L.xv_gemm_plan_override.restype = None
    L.xv_selftest_bounded_wait.argtypes = [_vp, _vp, ctypes.c_uint, _vp]
    L.xv_num_sms.restype = _i32
    _lib = L
    return L


def _check(rc: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if rc != 0:
        raise RuntimeError(f"{what}: {ERRORS.get(rc, rc)}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _bf16(*tensors) -> None:
    for t in tensors:
        if t.dtype != torch.bfloat16:
            raise TypeError(f"GPU kernels take bfloat16 tensors, got {t.dtype}")


class _DeviceState:
    """Per-device scratch: split-K / split-KV workspaces, the status word, SM count."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.num_sms = torch.cuda.get_device_properties(device).multi_processor_count
        # zero-filled: the last 20 MiB serve the pair GEMM's stream-K (partial tiles and counters, kept at zero
        # by the kernels), the front part holds split-K planes
        self.gemm_ws = torch.zeros(56 << 20, dtype=torch.uint8, device=device)
        self.attn_ws = torch.empty(16 << 20, dtype=torch.uint8, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)


_states: dict[int, _DeviceState] = {}


def _state(t: torch.Tensor) -> _DeviceState:
    idx = t.device.index if t.device.index is not None else torch.cuda.current_device()
    st = _states.get(idx)
    if st is None:
        st = _states[idx] = _DeviceState(torch.device("cuda", idx))
    return st


def check_status(device=None) -> int:
    """Reads (and clears) the device status word; raises if a kernel reported a problem."""
    idx = torch.device(device).index if device is not None else torch.cuda.current_device()
    st = _states.get(idx)
    if st is None:
        return 0
    code = int(st.status.item())
    if code:
        st.status.zero_()
        raise RuntimeError(f"kernel {code >> 16} reported status {code & 0xFFFF} "
                           "(1/2/3 = pipeline wait ran out, 4 = peer flag wait ran out, 5 = bad index)")
    return 0


def gemm_plan(m: int, n: int, k: int, num_sms: int = 148) -> GemmPlan:
    pl = GemmPlan()
    rc = lib().xv_gemm_plan(m, n, k, num_sms, ctypes.byref(pl))
    if rc:
        raise RuntimeError(f"gemm_plan({m},{n},{k}): {ERRORS.get(rc, rc)}")
    return pl


_USE_CUBLAS = os.environ.get("XV_GEMM", "") == "cublas"


class SplitKPartial:
    """Result of a split-K GEMM whose reduction is left to the consumer kernel: ``splits`` fp32
    planes ``[M, N]`` in the device's GEMM workspace. Valid until the next split-K GEMM on
    that device; ``materialize()`` reduces it to an ordinary bf16 tensor."""

    __slots__ = ("ws", "splits", "shape", "device")

    def __init__(self, ws: torch.Tensor, splits: int, m: int, n: int) -> None:
        self.ws, self.splits, self.shape, self.device = ws, splits, (m, n), ws.device

    @property
    def is_cuda(self) -> bool:
        return True

    @property
    def stride_elems(self) -> int:
        return self.shape[0] * self.shape[1]

    def materialize(self) -> torch.Tensor:
        m, n = self.shape
        planes = self.ws[: self.splits * m * n * 4].view(torch.float32).view(self.splits, m, n)
        return planes.sum(0).to(torch.bfloat16)


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
           out: torch.Tensor | None = None, defer: bool = False):
    """``x[M,K] @ w[N,K]^T`` on the tcgen05 GEMM; ``out`` (dense [M,N]) receives the result if given.
    ``defer=True`` may return a ``SplitKPartial`` instead of a tensor (see there)."""
    _bf16(x, w)
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise ValueError(f"linear: bad shapes {tuple(x.shape)} x {tuple(w.shape)}")
    M, K = x.shape
    N = w.shape[0]
    if M == 0:
        return x.new_empty((0, N)) if out is None else out
    if out is not None and (out.shape != (M, N) or not out.is_contiguous() or out.dtype != torch.bfloat16):
        raise ValueError("linear: out must be a contiguous bf16 [M, N] tensor")
    if _USE_CUBLAS:
        y = torch.matmul(x, w.t(), out=out) if out is not None else torch.matmul(x, w.t())
    else:
        if x.stride(1) != 1 or w.stride(1) != 1:
            x, w = x.contiguous(), w.contiguous()
        st = _state(x)
        if defer and out is None and bias is None:
            pl = gemm_plan(M, N, K, st.num_sms)
            if pl.splits > 1 and not pl.cluster:        # a cluster sums its K splits itself: the output is final
                used = _i32(0)
                rc = lib().xv_gemm_bf16_defer(x.data_ptr(), w.data_ptr(), None, M, N, K, x.stride(0), w.stride(0), N,
                                              st.gemm_ws.data_ptr(), st.gemm_ws.numel(), st.num_sms,
                                              st.status.data_ptr(), _stream(), ctypes.byref(used))
                _check(rc, f"gemm {M}x{N}x{K}")
                return SplitKPartial(st.gemm_ws, used.value, M, N)
        y = out if out is not None else torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        rc = lib().xv_gemm_bf16(x.data_ptr(), w.data_ptr(), y.data_ptr(), M, N, K, x.stride(0), w.stride(0), N,
                                st.gemm_ws.data_ptr(), st.gemm_ws.numel(), st.num_sms, st.status.data_ptr(),
                                _stream())
        _check(rc, f"gemm {M}x{N}x{K}")
    if bias is not None:
        y += bias
    return y


def linear_silu_mul(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``silu(x @ Wg^T) * (x @ Wu^T)`` where ``w`` [2*I, K] stores gate and up rows interleaved in
    groups of 16 = [8 gate | 8 up]. The activation runs in the GEMM epilogue; when the plan
    splits K it runs in the kernel that sums the partial planes instead."""
    _bf16(x, w)
    M, K = x.shape
    N = w.shape[0]
    inter = N // 2
    if M == 0:
        return x.new_empty((0, inter))
    if x.stride(1) != 1:
        x = x.contiguous()
    st = _state(x)
    y = torch.empty((M, inter), dtype=torch.bfloat16, device=x.device)
    if _USE_CUBLAS:
        gu = torch.matmul(x, w.t())
        _check(lib().xv_silu_mul_interleaved(gu.data_ptr(), None, 0, 0, y.data_ptr(), M, inter, _stream()),
               "silu_mul_interleaved")
        return y
    pl = gemm_plan(M, N, K, st.num_sms)
    if pl.splits == 1 or pl.cluster:
        _check(lib().xv_gemm_bf16_silu_mul(x.data_ptr(), w.data_ptr(), y.data_ptr(), M, N, K, x.stride(0),
                                           w.stride(0), inter, st.gemm_ws.data_ptr(), st.gemm_ws.numel(),
                                           st.num_sms, st.status.data_ptr(), _stream()),
               f"gemm+silu {M}x{N}x{K}")
        return y
    part = linear(x, w, defer=True)
    _check(lib().xv_silu_mul_interleaved(None, part.ws.data_ptr(), part.splits, part.stride_elems, y.data_ptr(), M,
                                         inter, _stream()), "silu_mul_interleaved")
    return y


def rmsnorm(x, w, eps):
    _bf16(x, w)
    x = x.contiguous()
    y = torch.empty_like(x)
    rows = x.numel() // x.shape[-1]
    _check(lib().xv_rmsnorm(x.data_ptr(), w.data_ptr(), y.data_ptr(), rows, x.shape[-1], eps, _stream()), "rmsnorm")
    return y


def add_rmsnorm(x, residual, w, eps):
    if isinstance(x, SplitKPartial):
        _bf16(residual, w)
        if not residual.is_contiguous():
            raise ValueError("add_rmsnorm needs a contiguous residual")
        m, n = x.shape
        y = torch.empty((m, n), dtype=torch.bfloat16, device=residual.device)
        _check(lib().xv_add_rmsnorm_partials(x.ws.data_ptr(), x.splits, x.stride_elems, residual.data_ptr(),
                                             w.data_ptr(), y.data_ptr(), m, n, eps, _stream()), "add_rmsnorm_partials")
        return y
    _bf16(x, residual, w)
    if not (x.is_contiguous() and residual.is_contiguous()):
        raise ValueError("add_rmsnorm needs contiguous inputs (the residual is updated in place)")
    y = torch.empty_like(x)
    rows = x.numel() // x.shape[-1]
    _check(lib().xv_add_rmsnorm(x.data_ptr(), residual.data_ptr(), w.data_ptr(), y.data_ptr(), rows,
                                x.shape[-1], eps, _stream()), "add_rmsnorm")
    return y


def silu_mul(x):
    _bf16(x)
    x = x.contiguous()
    inter = x.shape[-1] // 2
    rows = x.numel() // x.shape[-1]
    y = torch.empty(x.shape[:-1] + (inter,), dtype=x.dtype, device=x.device)
    _check(lib().xv_silu_mul(x.data_ptr(), y.data_ptr(), rows, inter, _stream()), "silu_mul")
    return y


def embedding(ids, w, vocab_start=0, out=None):
    _bf16(w)
    if ids.dtype != torch.int32:
        ids = ids.to(torch.int32)
    y = out if out is not None else torch.empty((ids.numel(), w.shape[1]), dtype=w.dtype, device=w.device)
    _check(lib().xv_embedding(ids.data_ptr(), w.data_ptr(), y.data_ptr(), ids.numel(), w.shape[1], vocab_start,
                              w.shape[0], _stream()), "embedding")
    return y


def gather_rows(x, rows):
    _bf16(x)
    if rows.dtype != torch.int32:
        rows = rows.to(torch.int32)
    x = x.contiguous()
    y = torch.empty((rows.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    _check(lib().xv_gather_rows(x.data_ptr(), rows.data_ptr(), y.data_ptr(), rows.numel(), x.shape[1], _stream()),
           "gather_rows")
    return y


def resolve_token_refs(ids, prev) -> None:
    """In place: every ``ids[i] < 0`` becomes ``prev[-ids[i] - 1]`` (int32 ids, int64 previous samples)."""
    if ids.dtype != torch.int32 or prev.dtype != torch.int64 or not ids.is_contiguous() or not prev.is_contiguous():
        raise TypeError("resolve_token_refs needs contiguous int32 ids and int64 samples")
    _check(lib().xv_resolve_token_refs(ids.data_ptr(), ids.numel(), prev.data_ptr(), prev.numel(), _stream()),
           "resolve_token_refs")


def qk_norm_rope_cache(qkv, q_w, k_w, eps, cos_sin, positions, slots, k_cache, v_cache, num_q_heads,
                       num_kv_heads, head_dim, prefill_begin: int = 0):
    if isinstance(qkv, SplitKPartial):
        _bf16(q_w, k_w, k_cache, v_cache)
        T = qkv.shape[0]
        q = torch.empty((T, num_q_heads * head_dim), dtype=torch.bfloat16, device=k_cache.device)
        _check(lib().xv_qk_norm_rope_cache_partials(
            qkv.ws.data_ptr(), qkv.splits, qkv.stride_elems, q_w.data_ptr(), k_w.data_ptr(), eps, cos_sin.data_ptr(),
            positions.data_ptr(), slots.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), T,
            num_q_heads, num_kv_heads, head_dim, k_cache.shape[2], prefill_begin, _stream()),
            "qk_norm_rope_cache_partials")
        return q
    _bf16(qkv, q_w, k_w, k_cache, v_cache)
    if not (qkv.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("qk_norm_rope_cache needs contiguous qkv and cache tensors")
    T = qkv.shape[0]
    q = torch.empty((T, num_q_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    _check(lib().xv_qk_norm_rope_cache(qkv.data_ptr(), q_w.data_ptr(), k_w.data_ptr(), eps, cos_sin.data_ptr(),
                                       positions.data_ptr(), slots.data_ptr(), q.data_ptr(), k_cache.data_ptr(),
                                       v_cache.data_ptr(), T, num_q_heads, num_kv_heads, head_dim,
                                       k_cache.shape[2], prefill_begin, _stream()), "qk_norm_rope_cache")
    return q


def decode_splits(num_seqs: int, num_kv_heads: int, num_sms: int, max_blocks_tokens: int) -> int:
    """KV splits so that a small batch still fills the GPU; depends only on launch-shape
    constants (never on sequence lengths) so it is stable under CUDA-graph replay."""
    forced = os.environ.get("XV_DECODE_SPLITS")
    if forced:
        return int(forced)
    ctas = max(1, num_seqs * num_kv_heads)
    want = -(-2 * num_sms // ctas)
    by_len = max(1, max_blocks_tokens // 256)      # at least ~256 tokens per split
    return int(max(1, min(want, by_len, 16)))


def prefill_uses_tensor_cores(head_dim: int, block_size: int, max_q_len: int) -> bool:
    """Chunks longer than 64 rows run on the tcgen05 kernel (128-row tiles); shorter ones, unsupported
    page sizes, or ``XV_ATTN_PREFILL=mma`` use the 64-row warp-MMA kernel."""
    if os.environ.get("XV_ATTN_PREFILL", "tc") == "mma" or max_q_len <= 64:
        return False
    return bool(lib().xv_attn_prefill_tc_supported(head_dim, block_size))


def prefill_pair_heads(on: bool) -> None:
    """The tcgen05 prefill kernel gives one CTA two query heads of a KV group (shared K/V tiles) when the
    group size is even; ``False`` forces one head per CTA, for comparisons."""
    lib().xv_attn_prefill_tc_single_unit(0 if on else 1)


def paged_attention(q, k_cache, v_cache, attn, scale, num_q_heads, num_kv_heads, head_dim):
    """Decode rows (the first ``attn.num_decode`` sequences) and prefill chunks of one packed batch."""
    _bf16(q, k_cache, v_cache)
    st = _state(q)
    L = lib()
    out = torch.empty_like(q)
    bs = k_cache.shape[2]
    maxb = attn.block_tables.shape[1]
    n_d = attn.num_decode
    if n_d > 0:
        splits = decode_splits(n_d, num_kv_heads, st.num_sms, maxb * bs)
        need = L.xv_attn_decode_workspace_bytes(n_d, num_q_heads, head_dim, splits)
        if need > st.attn_ws.numel():
            st.attn_ws = torch.empty(need, dtype=torch.uint8, device=q.device)
        _check(L.xv_attn_decode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), attn.block_tables.data_ptr(),
                                attn.kv_lens.data_ptr(), out.data_ptr(), n_d, num_q_heads, num_kv_heads, head_dim,
                                bs, maxb, scale, splits, st.attn_ws.data_ptr(), _stream()), "attn_decode")
    n_p = attn.num_seqs - n_d
    if n_p > 0 and prefill_uses_tensor_cores(head_dim, bs, attn.max_q_len):
        _check(L.xv_attn_prefill_tc(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), attn.block_tables.data_ptr(),
                                    attn.cu_q.data_ptr(), attn.kv_lens.data_ptr(), out.data_ptr(), n_d, n_p,
                                    attn.max_q_len, q.shape[0], k_cache.shape[0], num_q_heads, num_kv_heads, head_dim,
                                    bs, maxb, scale, st.status.data_ptr(), _stream()), "attn_prefill_tc")
    elif n_p > 0:
        _check(L.xv_attn_prefill(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), attn.block_tables.data_ptr(),
                                 attn.cu_q.data_ptr(), attn.kv_lens.data_ptr(), out.data_ptr(), n_d, n_p,
                                 attn.max_q_len, num_q_heads, num_kv_heads, head_dim, bs, maxb, scale, _stream()),
               "attn_prefill")
    return out


PREFILL_PHASES = ("softmax: wait S", "softmax: tcgen05.ld S", "softmax: mask+max", "softmax: rescale O",
                  "softmax: exp+pack", "softmax: wait for the MUFU turn", "softmax: store P", "softmax: epilogue",
                  "mma: wait K tile", "mma: wait P", "mma: wait V tile", "mma: issue", "load: wait free slot",
                  "load: block table + TMA issue", "CTA lifetime", "tiles", "CTA setup", "ring slots")


def prefill_phase_profile(q, k_cache, v_cache, attn, scale, num_q_heads, num_kv_heads, head_dim) -> dict[str, int]:
    """Runs the instrumented tcgen05 prefill kernel once and returns cycles per phase summed over CTAs
    (one observer thread per warp role), plus the tile count."""
    L = lib()
    st = _state(q)
    n = L.xv_attn_prefill_tc_profile_slots()
    prof = torch.zeros(n, dtype=torch.int64, device=q.device)
    out = torch.empty_like(q)
    n_d = attn.num_decode
    _check(L.xv_attn_prefill_tc_profile(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                        attn.block_tables.data_ptr(), attn.cu_q.data_ptr(), attn.kv_lens.data_ptr(),
                                        out.data_ptr(), n_d, attn.num_seqs - n_d, attn.max_q_len, q.shape[0],
                                        k_cache.shape[0], num_q_heads, num_kv_heads, head_dim, k_cache.shape[2],
                                        attn.block_tables.shape[1], scale, st.status.data_ptr(), prof.data_ptr(),
                                        _stream()), "attn_prefill_tc_profile")
    vals = prof.cpu().tolist()
    return dict(zip(PREFILL_PHASES, vals))


def argmax(logits):
    _bf16(logits)
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int64, device=logits.device)
    _check(lib().xv_argmax(logits.data_ptr(), out.data_ptr(), rows, vocab, logits.stride(0), _stream()), "argmax")
    return out


def sample(logits, temperature, top_k, top_p, min_p, rng):
    _bf16(logits)
    rows, vocab = logits.shape
    if rng is None:
        rng = torch.zeros(2, dtype=torch.int32, device=logits.device)
    out = torch.empty(rows, dtype=torch.int64, device=logits.device)
    _check(lib().xv_sample(logits.data_ptr(), out.data_ptr(), rows, vocab, logits.stride(0),
                           temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(), min_p.data_ptr(),
                           rng.data_ptr(), _stream()), "sample")
    return out


def tp_reduce_norm(peer_bufs, peer_flags, mc_ptr: int, epoch, rank: int, world: int, buf_offset: int,
                   residual_in, residual_out, w, y, rows: int, hidden: int, eps: float, mode: int,
                   spin_limit: int, status) -> None:
    """Sum the ranks' partial tiles (+ residual, RMSNorm when ``mode == 0``); see tp_fused.cu."""
    _check(lib().xv_tp_reduce_norm(peer_bufs, peer_flags, mc_ptr or None, epoch.data_ptr(), rank, world, buf_offset,
                                   residual_in.data_ptr() if residual_in is not None else None,
                                   residual_out.data_ptr() if residual_out is not None else None,
                                   w.data_ptr() if w is not None else None, y.data_ptr(), rows, hidden, eps, mode,
                                   spin_limit, status.data_ptr(), _stream()), "tp_reduce_norm")


def tp_argmax(peer_bufs, peer_flags, epoch, rank: int, world: int, slots_offset: int, logits, local_vocab: int,
              valid_vocab: int, vocab_start: int, out, spin_limit: int, status) -> None:
    _bf16(logits)
    _check(lib().xv_tp_argmax(peer_bufs, peer_flags, epoch.data_ptr(), rank, world, slots_offset, logits.data_ptr(),
                              logits.stride(0), local_vocab, valid_vocab, vocab_start, out.data_ptr(),
                              logits.shape[0], spin_limit, status.data_ptr(), _stream()), "tp_argmax")


def tp_sample_region_bytes(max_rows: int, world: int) -> int:
    return int(lib().xv_tp_sample_region_bytes(max_rows, world))


def tp_sample(peer_bufs, peer_flags, epoch, rank: int, world: int, region_offset: int, max_rows: int, logits,
              valid_vocab: int, vocab_start: int, total_vocab: int, temperature, top_k, top_p, min_p, rng,
              spin_limit: int, status):
    """Temperature / top-k / top-p / min-p sampling over vocabulary shards without gathering them
    (``xv_tp_sample``): the ranks exchange row maxima, selection histograms and their best candidates."""
    _bf16(logits)
    if logits.stride(1) != 1:
        raise ValueError("tp_sample needs unit column stride")
    rows = logits.shape[0]
    if rng is None:
        rng = torch.zeros(2, dtype=torch.int32, device=logits.device)
    out = torch.empty(rows, dtype=torch.int64, device=logits.device)
    _check(lib().xv_tp_sample(peer_bufs, peer_flags, epoch.data_ptr(), rank, world, region_offset,
                              max_rows, logits.data_ptr(), logits.stride(0), valid_vocab,
                              vocab_start, total_vocab, out.data_ptr(), rows, temperature.data_ptr(),
                              top_k.data_ptr(), top_p.data_ptr(), min_p.data_ptr(), rng.data_ptr(), spin_limit,
                              status.data_ptr(), _stream()), "tp_sample")
    return out


def tp_allgather_cols(peer_bufs, peer_flags, mc_ptr: int, epoch, rank: int, world: int, src, total_cols: int,
                      spin_limit: int, status) -> None:
    """Pushes this rank's ``[rows, local_cols]`` shard into column block ``rank`` of the symmetric
    ``[rows, total_cols]`` matrix on every rank (``xv_tp_allgather_cols``)."""
    _bf16(src)
    if src.stride(1) != 1:
        raise ValueError("tp_allgather_cols needs unit column stride")
    _check(lib().xv_tp_allgather_cols(peer_bufs, peer_flags, mc_ptr or None, epoch.data_ptr(), rank, world,
                                      src.data_ptr(), src.stride(0), src.shape[1], total_cols, src.shape[0],
                                      spin_limit, status.data_ptr(), _stream()), "tp_allgather_cols")


def gemm_tp_fused(x, w, peer_bufs, peer_flags, mc_ptr: int, epoch, rank: int, world: int, slot_offset: int,
                  slot_bytes: int, two_shot: bool, h_offset: int, residual_in, residual_out, norm_w, y, eps: float,
                  mode: int, spin_us: int, defer_row_wait: bool = False) -> None:
    """RowParallel GEMM + cross-rank sum + residual add + RMSNorm in one kernel (``xv_gemm_bf16_tp``): the GEMM
    epilogue pushes its tiles into the slot array of the ranks that reduce them."""
    _bf16(x, w)
    if x.stride(1) != 1:
        x = x.contiguous()
    M, K = x.shape
    N = w.shape[0]
    st = _state(x)
    _check(lib().xv_gemm_bf16_tp(
        x.data_ptr(), w.data_ptr(), M, N, K, x.stride(0), w.stride(0), st.gemm_ws.data_ptr(), st.gemm_ws.numel(),
        st.num_sms, peer_bufs, peer_flags,
        mc_ptr or None, epoch.data_ptr(), rank, world, slot_offset, slot_bytes, 1 if two_shot else 0, h_offset,
        residual_in.data_ptr() if residual_in is not None else None,
        residual_out.data_ptr() if residual_out is not None else None,
        norm_w.data_ptr() if norm_w is not None else None, y.data_ptr() if y is not None else None, eps, mode,
        1 if defer_row_wait else 0, spin_us, st.status.data_ptr(), _stream()), f"gemm+allreduce {M}x{N}x{K}")


def gemm_plan_override(kind: int = -1, bn: int = 0, splits: int = 0, stages: int = 0) -> None:
    """Tuning hook: force kernel kind (0 single CTA, 1 single CTA normal orientation, 2 CTA pairs, 3 CTA pairs in
    the swapped orientation for at most 256 rows), tile width,
    split-K and stages for every following GEMM; ``kind < 0`` restores the planner."""
    lib().xv_gemm_plan_override(kind, bn, splits, stages)


def device_status(t: torch.Tensor) -> torch.Tensor:
    """The per-device status word kernels report problems through."""
    return _state(t).status


def selftest_bounded_wait(limit: int = 1000) -> int:
    """Runs a kernel that waits on a flag nobody sets; returns the status code it reports."""
    dev = torch.device("cuda", torch.cuda.current_device())
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    _check(lib().xv_selftest_bounded_wait(flag.data_ptr(), status.data_ptr(), limit, _stream()), "selftest")
    return int(status.item())
