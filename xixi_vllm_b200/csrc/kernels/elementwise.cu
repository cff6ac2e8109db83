// Memory-bound glue kernels in bf16 with 16-byte vector accesses: RMSNorm, fused
// residual-add + RMSNorm, SiLU-mul, vocab-shard embedding lookup, row gather, and the fused
// per-head QK-RMSNorm + NeoX RoPE + paged KV-cache append.
//
// The reference runs these as separate library kernels (FlashInfer RMSNorm / fused add+norm /
// RoPE / SiLU-mul, a Triton KV-append kernel, ATen embedding) with extra slice copies in
// between (reference: src/compute/layers/ops.py:20-85, src/compute/kv_ops.py:8-62,
// src/compute/models/qwen3.py:117-128). Here the q-norm, k-norm, RoPE and cache append are one
// pass over the QKV activations.

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "xv_cuda.h"

namespace xv {

struct alignas(16) Bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const Bf16x8 r = *reinterpret_cast<const Bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(r.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  Bf16x8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<Bf16x8*>(p) = r;
}

__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < nw ? scratch[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;   // up to 256 * 4 * 8 = 8192 columns held in registers

// One CTA per row. ADD: residual += x first, and the sum is what gets normalised.
template <bool ADD>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ residual,
               const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, int hidden, float eps) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ float scratch[32];
  const size_t row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * hidden;
  __nv_bfloat16* rr = ADD ? residual + row * hidden : nullptr;
  __nv_bfloat16* yr = y + row * hidden;
  const int nvec = hidden >> 3;
  float vals[kNormMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      load8(xr + v * 8, vals[i]);
      if (ADD) {
        float r[8];
        load8(rr + v * 8, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[i][j] += r[j];
        store8(rr + v * 8, vals[i]);
        // normalise what was stored (the rounded sum), as a separate add kernel would
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[i][j] = __bfloat162float(__float2bfloat16(vals[i][j]));
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
    }
  }
  const float inv = rsqrtf(block_sum(ss, scratch) / static_cast<float>(hidden) + eps);
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      float g[8], o[8];
      load8(w + v * 8, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * inv * g[j];
      store8(yr + v * 8, o);
    }
  }
}

// residual += sum_s partial[s]; y = rmsnorm(residual) * w. One CTA per row.
__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_partials_kernel(const float* __restrict__ partials, int splits, long long split_stride,
                            __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ w,
                            __nv_bfloat16* __restrict__ y, int hidden, float eps) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ float scratch[32];
  const size_t row = blockIdx.x;
  __nv_bfloat16* rr = residual + row * hidden;
  __nv_bfloat16* yr = y + row * hidden;
  const int nvec = hidden >> 3;
  float vals[kNormMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      load8(rr + v * 8, vals[i]);
      const float* src = partials + row * hidden + v * 8;
      for (int s = 0; s < splits; ++s) {
        const float4 a = *reinterpret_cast<const float4*>(src + s * split_stride);
        const float4 b = *reinterpret_cast<const float4*>(src + s * split_stride + 4);
        vals[i][0] += a.x; vals[i][1] += a.y; vals[i][2] += a.z; vals[i][3] += a.w;
        vals[i][4] += b.x; vals[i][5] += b.y; vals[i][6] += b.z; vals[i][7] += b.w;
      }
      store8(rr + v * 8, vals[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        vals[i][j] = __bfloat162float(__float2bfloat16(vals[i][j]));
        ss += vals[i][j] * vals[i][j];
      }
    }
  }
  const float inv = rsqrtf(block_sum(ss, scratch) / static_cast<float>(hidden) + eps);
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      float g[8], o[8];
      load8(w + v * 8, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * inv * g[j];
      store8(yr + v * 8, o);
    }
  }
}

__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long rows,
                                int inter) {
  grid_dep_launch();
  grid_dep_wait();
  const int vec_per_row = inter >> 3;
  const long long total = rows * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i - r * vec_per_row) * 8;
    float g[8], u[8], o[8];
    load8(x + r * 2 * inter + c, g);
    load8(x + r * 2 * inter + inter + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    store8(y + r * inter + c, o);
  }
}

// Columns come in groups of 16 = [8 gate | 8 up]; input is bf16 or a sum of fp32 split-K planes.
__global__ void silu_mul_interleaved_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ partials,
                                            int splits, long long split_stride, __nv_bfloat16* __restrict__ y,
                                            long long rows, int inter) {
  grid_dep_launch();
  grid_dep_wait();
  const int groups = inter >> 3;
  const long long total = rows * groups;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / groups;
    const int gidx = static_cast<int>(i - r * groups);
    const long long in_off = r * 2 * inter + static_cast<long long>(gidx) * 16;
    float g[8], u[8], o[8];
    if (partials != nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = u[j] = 0.f;
      for (int s = 0; s < splits; ++s) {
        const float* p = partials + s * split_stride + in_off;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          g[j] += p[j];
          u[j] += p[8 + j];
        }
      }
    } else {
      load8(x + in_off, g);
      load8(x + in_off + 8, u);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    store8(y + r * inter + static_cast<long long>(gidx) * 8, o);
  }
}

// out[t] = w[ids[t] - vocab_start] when the id is inside this rank's shard, zeros otherwise.
__global__ void embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ w,
                                 __nv_bfloat16* __restrict__ y, int hidden, int vocab_start, int vocab_rows) {
  grid_dep_launch();
  grid_dep_wait();
  const size_t t = blockIdx.x;
  const int local = ids[t] - vocab_start;
  const bool mine = local >= 0 && local < vocab_rows;
  const int nvec = hidden >> 3;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 val = zero;
    if (mine) val = *reinterpret_cast<const uint4*>(w + static_cast<size_t>(local) * hidden + v * 8);
    *reinterpret_cast<uint4*>(y + t * hidden + v * 8) = val;
  }
}

__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ rows,
                                   __nv_bfloat16* __restrict__ y, int hidden) {
  grid_dep_launch();
  grid_dep_wait();
  const size_t i = blockIdx.x;
  const size_t src = static_cast<size_t>(rows[i]);
  const int nvec = hidden >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x)
    *reinterpret_cast<uint4*>(y + i * hidden + v * 8) = *reinterpret_cast<const uint4*>(x + src * hidden + v * 8);
}

// One-step-late scheduling: an input id < 0 names row -(id) - 1 of the previous step's sample buffer (the host
// launched this step before it had read those samples). A reference beyond that buffer becomes token 0.
__global__ void resolve_token_refs_kernel(int* __restrict__ ids, int n, const long long* __restrict__ prev,
                                          int n_prev) {
  grid_dep_launch();
  grid_dep_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int id = ids[i];
  if (id < 0) {
    const int j = -id - 1;
    ids[i] = j < n_prev ? static_cast<int>(prev[j]) : 0;
  }
}

// One warp per (token, head). Lane l holds elements [2l, 2l+1] of the first half and the same
// of the second half (D = 128: 2 + 2 values; D = 64: lanes 0..15 active per half... handled by
// the generic loop). The NeoX rotation pairs element i with i + D/2, both held by one lane.
template <int D>
__global__ void __launch_bounds__(256)
qk_norm_rope_cache_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ partials, int splits,
                          long long split_stride, const __nv_bfloat16* __restrict__ q_w,
                          const __nv_bfloat16* __restrict__ k_w, float eps, const float* __restrict__ cos_sin,
                          const int* __restrict__ positions, const int* __restrict__ slots,
                          __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache,
                          __nv_bfloat16* __restrict__ v_cache, int tokens, int hq, int hkv, int block_size,
                          int prefill_begin) {
  grid_dep_launch();
  grid_dep_wait();
  constexpr int HALF = D / 2;
  constexpr int PER = HALF / 32;           // elements per lane per half (2 for D=128, 1 for D=64)
  static_assert(PER == 1 || PER == 2, "head_dim must be 64 or 128");
  const int heads = hq + 2 * hkv;
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= static_cast<long long>(tokens) * heads) return;
  const int t = static_cast<int>(gw / heads);
  const int h = static_cast<int>(gw - static_cast<long long>(t) * heads);
  const __nv_bfloat16* src = qkv + static_cast<size_t>(t) * heads * D + static_cast<size_t>(h) * D;
  const int slot = slots[t];

  float lo[PER], hi[PER];
  if (partials != nullptr) {
    // QKV arrives as split-K partial planes: sum them here instead of in a separate kernel
    const float* ps = partials + static_cast<size_t>(t) * heads * D + static_cast<size_t>(h) * D;
#pragma unroll
    for (int i = 0; i < PER; ++i) lo[i] = hi[i] = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float* q = ps + s * split_stride;
      if (PER == 2) {
        const float2 a = *reinterpret_cast<const float2*>(q + lane * 2);
        const float2 b = *reinterpret_cast<const float2*>(q + HALF + lane * 2);
        lo[0] += a.x; lo[PER - 1] += a.y; hi[0] += b.x; hi[PER - 1] += b.y;
      } else {
        lo[0] += q[lane];
        hi[0] += q[HALF + lane];
      }
    }
    // same rounding point as the bf16 GEMM output would have had
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      lo[i] = __bfloat162float(__float2bfloat16(lo[i]));
      hi[i] = __bfloat162float(__float2bfloat16(hi[i]));
    }
  } else if (PER == 2) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + lane * 2));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + HALF + lane * 2));
    lo[0] = a.x; lo[PER - 1] = a.y; hi[0] = b.x; hi[PER - 1] = b.y;
  } else {
    lo[0] = __bfloat162float(src[lane]);
    hi[0] = __bfloat162float(src[HALF + lane]);
  }

  if (h >= hq + hkv) {
    // V head: straight copy into the cache
    if (slot >= 0) {
      const int hv = h - hq - hkv;
      __nv_bfloat16* dst = v_cache + ((static_cast<size_t>(slot / block_size) * hkv + hv) * block_size +
                                      slot % block_size) * D;
      if (PER == 2) {
        *reinterpret_cast<__nv_bfloat162*>(dst + lane * 2) = __floats2bfloat162_rn(lo[0], lo[PER - 1]);
        *reinterpret_cast<__nv_bfloat162*>(dst + HALF + lane * 2) = __floats2bfloat162_rn(hi[0], hi[PER - 1]);
      } else {
        dst[lane] = __float2bfloat16(lo[0]);
        dst[HALF + lane] = __float2bfloat16(hi[0]);
      }
      // Last row that a prefill chunk writes into a page: clear the V rows after it. The tcgen05 prefill
      // kernel multiplies whole 128-token tiles, masked columns included (P = 0 there), so rows past the
      // end of the sequence must hold finite values whatever an earlier owner of the page left behind.
      const int r = slot % block_size;
      if (t >= prefill_begin && r != block_size - 1 && (t == tokens - 1 || slots[t + 1] != slot + 1)) {
        for (int z = r + 1; z < block_size; ++z) {
          __nv_bfloat16* row = dst + static_cast<size_t>(z - r) * D;
          if (PER == 2) {
            *reinterpret_cast<uint32_t*>(row + lane * 2) = 0u;
            *reinterpret_cast<uint32_t*>(row + HALF + lane * 2) = 0u;
          } else {
            row[lane] = __float2bfloat16(0.f);
            row[HALF + lane] = __float2bfloat16(0.f);
          }
        }
      }
    }
    return;
  }

  const bool is_q = h < hq;
  const __nv_bfloat16* nw = is_q ? q_w : k_w;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) ss += lo[i] * lo[i] + hi[i] * hi[i];
  const float inv = rsqrtf(warp_sum(ss) / static_cast<float>(D) + eps);
  const float* cs = cos_sin + static_cast<size_t>(positions[t]) * D;
  float olo[PER], ohi[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane * PER + i;
    const float x1 = lo[i] * inv * __bfloat162float(nw[e]);
    const float x2 = hi[i] * inv * __bfloat162float(nw[HALF + e]);
    const float c = cs[e], s = cs[HALF + e];
    olo[i] = x1 * c - x2 * s;
    ohi[i] = x2 * c + x1 * s;
  }
  __nv_bfloat16* dst;
  if (is_q) {
    dst = q_out + static_cast<size_t>(t) * hq * D + static_cast<size_t>(h) * D;
  } else {
    if (slot < 0) return;
    dst = k_cache + ((static_cast<size_t>(slot / block_size) * hkv + (h - hq)) * block_size + slot % block_size) * D;
  }
  if (PER == 2) {
    *reinterpret_cast<__nv_bfloat162*>(dst + lane * 2) = __floats2bfloat162_rn(olo[0], olo[PER - 1]);
    *reinterpret_cast<__nv_bfloat162*>(dst + HALF + lane * 2) = __floats2bfloat162_rn(ohi[0], ohi[PER - 1]);
  } else {
    dst[lane] = __float2bfloat16(olo[0]);
    dst[HALF + lane] = __float2bfloat16(ohi[0]);
  }
}

__global__ void bounded_wait_kernel(volatile int* flag, int* status, unsigned limit) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    bool seen = false;
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
      if (*flag != 0) {
        seen = true;
        break;
      }
      if (global_timer_ns() - t0 > static_cast<unsigned long long>(limit) * 1000ull) break;   // limit in us
      __nanosleep(100);
    }
    if (!seen) report_status(status, 99, kHostFlagTimeout);
  }
}

}  // namespace xv

using namespace xv;

static inline int launch_ok() { return cudaGetLastError() == cudaSuccess ? 0 : XV_ERR_LAUNCH; }

extern "C" {

int xv_rmsnorm(const void* x, const void* w, void* y, int rows, int hidden, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden % 8 || hidden > kNormThreads * kNormMaxVec * 8) return XV_ERR_SHAPE;
  launch_pdl(rmsnorm_kernel<false>, dim3(rows), dim3(kNormThreads), 0, stream, static_cast<const __nv_bfloat16*>(x), nullptr,
                                                          static_cast<const __nv_bfloat16*>(w),
                                                          static_cast<__nv_bfloat16*>(y), hidden, eps);
  return launch_ok();
}

int xv_add_rmsnorm(const void* x, void* residual, const void* w, void* y, int rows, int hidden, float eps,
                   cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden % 8 || hidden > kNormThreads * kNormMaxVec * 8) return XV_ERR_SHAPE;
  launch_pdl(rmsnorm_kernel<true>, dim3(rows), dim3(kNormThreads), 0, stream, static_cast<const __nv_bfloat16*>(x),
                                                         static_cast<__nv_bfloat16*>(residual),
                                                         static_cast<const __nv_bfloat16*>(w),
                                                         static_cast<__nv_bfloat16*>(y), hidden, eps);
  return launch_ok();
}

int xv_silu_mul(const void* x, void* y, int rows, int inter, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (inter % 8) return XV_ERR_SHAPE;
  const long long total = static_cast<long long>(rows) * (inter / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  launch_pdl(silu_mul_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x),
                                                                     static_cast<__nv_bfloat16*>(y), rows, inter);
  return launch_ok();
}

int xv_silu_mul_interleaved(const void* x, const float* partials, int splits, long long split_stride, void* y,
                            int rows, int inter, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (inter % 8) return XV_ERR_SHAPE;
  const long long total = static_cast<long long>(rows) * (inter / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  launch_pdl(silu_mul_interleaved_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, 
      static_cast<const __nv_bfloat16*>(x), partials, splits, split_stride, static_cast<__nv_bfloat16*>(y), rows, inter);
  return launch_ok();
}

int xv_embedding(const int* ids, const void* w, void* y, int tokens, int hidden, int vocab_start, int vocab_rows,
                 cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (hidden % 8) return XV_ERR_SHAPE;
  launch_pdl(embedding_kernel, dim3(tokens), dim3(128), 0, stream, ids, static_cast<const __nv_bfloat16*>(w),
                                               static_cast<__nv_bfloat16*>(y), hidden, vocab_start, vocab_rows);
  return launch_ok();
}

int xv_gather_rows(const void* x, const int* rows, void* y, int n, int hidden, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (hidden % 8) return XV_ERR_SHAPE;
  launch_pdl(gather_rows_kernel, dim3(n), dim3(128), 0, stream, static_cast<const __nv_bfloat16*>(x), rows,
                                            static_cast<__nv_bfloat16*>(y), hidden);
  return launch_ok();
}

int xv_resolve_token_refs(int* ids, int n, const long long* prev, int n_prev, cudaStream_t stream) {
  if (n <= 0) return 0;
  launch_pdl(resolve_token_refs_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, ids, n, prev, n_prev);
  return launch_ok();
}

static int qk_norm_rope_launch(const void* qkv, const float* partials, int splits, long long split_stride,
                               const void* q_w, const void* k_w, float eps, const float* cos_sin,
                               const int* positions, const int* slots, void* q_out, void* k_cache, void* v_cache,
                               int tokens, int hq, int hkv, int d, int block_size, int prefill_begin,
                               cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const long long warps = static_cast<long long>(tokens) * (hq + 2 * hkv);
  const unsigned blocks = static_cast<unsigned>((warps + 7) / 8);
#define XV_QKR(D)                                                                                         \
  launch_pdl(qk_norm_rope_cache_kernel<D>, dim3(blocks), dim3(256), 0, stream,                                                 \
      static_cast<const __nv_bfloat16*>(qkv), partials, splits, split_stride,                              \
      static_cast<const __nv_bfloat16*>(q_w),                                                              \
      static_cast<const __nv_bfloat16*>(k_w), eps, cos_sin, positions, slots,                              \
      static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),                            \
      static_cast<__nv_bfloat16*>(v_cache), tokens, hq, hkv, block_size, prefill_begin)
  if (d == 128) {
    XV_QKR(128);
  } else if (d == 64) {
    XV_QKR(64);
  } else {
    return XV_ERR_UNSUPPORTED;
  }
#undef XV_QKR
  return launch_ok();
}

int xv_qk_norm_rope_cache(const void* qkv, const void* q_w, const void* k_w, float eps, const float* cos_sin,
                          const int* positions, const int* slots, void* q_out, void* k_cache, void* v_cache,
                          int tokens, int hq, int hkv, int d, int block_size, int prefill_begin,
                          cudaStream_t stream) {
  return qk_norm_rope_launch(qkv, nullptr, 0, 0, q_w, k_w, eps, cos_sin, positions, slots, q_out, k_cache, v_cache,
                             tokens, hq, hkv, d, block_size, prefill_begin, stream);
}

int xv_qk_norm_rope_cache_partials(const float* partials, int splits, long long split_stride, const void* q_w,
                                   const void* k_w, float eps, const float* cos_sin, const int* positions,
                                   const int* slots, void* q_out, void* k_cache, void* v_cache, int tokens, int hq,
                                   int hkv, int d, int block_size, int prefill_begin, cudaStream_t stream) {
  return qk_norm_rope_launch(nullptr, partials, splits, split_stride, q_w, k_w, eps, cos_sin, positions, slots,
                             q_out, k_cache, v_cache, tokens, hq, hkv, d, block_size, prefill_begin, stream);
}

int xv_add_rmsnorm_partials(const float* partials, int splits, long long split_stride, void* residual, const void* w,
                            void* y, int rows, int hidden, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden % 8 || hidden > kNormThreads * kNormMaxVec * 8) return XV_ERR_SHAPE;
  launch_pdl(add_rmsnorm_partials_kernel, dim3(rows), dim3(kNormThreads), 0, stream, partials, splits, split_stride,
                                                                static_cast<__nv_bfloat16*>(residual),
                                                                static_cast<const __nv_bfloat16*>(w),
                                                                static_cast<__nv_bfloat16*>(y), hidden, eps);
  return launch_ok();
}

int xv_selftest_bounded_wait(int* flag, int* status, unsigned limit, cudaStream_t stream) {
  bounded_wait_kernel<<<1, 32, 0, stream>>>(flag, status, limit);
  return launch_ok();
}

int xv_num_sms(void) {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return n;
}

}  // extern "C"
