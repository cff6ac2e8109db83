// Token selection over bf16 logits, one CTA per row, no host synchronisation.
//
//   argmax_kernel  - greedy; ties resolve to the lowest token id.
//   sample_kernel  - temperature, top-k, top-p, min-p, then one draw. The kept set is always
//                    "logit >= threshold", so it is found with MSB-first radix selection over
//                    order-preserving integer keys: by element count for top-k, by probability
//                    mass for top-p (no sort of the 152k-entry row, unlike a full descending
//                    sort). The draw is Gumbel-max over the kept set with a counter-based
//                    random stream keyed by (seed, step, row, token), so replaying a captured
//                    graph with a new step value draws fresh numbers and every tensor-parallel
//                    rank draws the same token. Elements tied with the k-th value are all kept.
//
// The reference does this with ATen softmax / topk / sort / cumsum / multinomial
// (reference: src/compute/sampler.py:27-118).

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "xv_cuda.h"

namespace xv {

constexpr int kSampThreads = 1024;

__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // larger float -> larger key
}

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x85EBCA6Bu; x ^= x >> 13; x *= 0xC2B2AE35u; x ^= x >> 16;
  return x;
}

// Uniform in (0, 1) from (seed, step, row, index).
__device__ __forceinline__ float uniform01(uint32_t seed, uint32_t step, uint32_t row, uint32_t idx) {
  uint32_t h = mix32(seed ^ 0x9E3779B9u);
  h = mix32(h ^ (step * 0x85EBCA77u + 0x165667B1u));
  h = mix32(h ^ (row * 0xC2B2AE3Du + 0x27D4EB2Fu));
  h = mix32(h ^ (idx * 0x9E3779B1u + 0x7F4A7C15u));
  return (static_cast<float>(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

struct ArgPair {
  float v;
  int i;
};
__device__ __forceinline__ ArgPair better(ArgPair a, ArgPair b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ ArgPair block_argmax(ArgPair p, ArgPair* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair q;
    q.v = __shfl_xor_sync(0xffffffffu, p.v, o);
    q.i = __shfl_xor_sync(0xffffffffu, p.i, o);
    p = better(p, q);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) scratch[warp] = p;
  __syncthreads();
  ArgPair r = lane < nw ? scratch[lane] : ArgPair{-CUDART_INF_F, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair q;
    q.v = __shfl_xor_sync(0xffffffffu, r.v, o);
    q.i = __shfl_xor_sync(0xffffffffu, r.i, o);
    r = better(r, q);
  }
  __syncthreads();
  return r;
}
__device__ float block_sum_f(float v, float* scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < nw ? scratch[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

__global__ void __launch_bounds__(kSampThreads)
argmax_kernel(const __nv_bfloat16* __restrict__ logits, long long* __restrict__ out, int vocab, long long ld) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ ArgPair scratch[32];
  const __nv_bfloat16* row = logits + static_cast<size_t>(blockIdx.x) * ld;
  ArgPair best{-CUDART_INF_F, 0x7fffffff};
  const bool vec_ok = (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  const int nvec = vec_ok ? vocab / 8 : 0;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 raw = *reinterpret_cast<const uint4*>(row + v * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      best = better(best, ArgPair{f.x, v * 8 + 2 * j});
      best = better(best, ArgPair{f.y, v * 8 + 2 * j + 1});
    }
  }
  for (int i = nvec * 8 + threadIdx.x; i < vocab; i += blockDim.x)
    best = better(best, ArgPair{__bfloat162float(row[i]), i});
  best = block_argmax(best, scratch);
  if (threadIdx.x == 0) out[blockIdx.x] = best.i;
}

__global__ void __launch_bounds__(kSampThreads)
sample_kernel(const __nv_bfloat16* __restrict__ logits, long long* __restrict__ out, int vocab, long long ld,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p, const int* __restrict__ rng) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ ArgPair scratch[32];
  __shared__ float fscratch[32];
  __shared__ unsigned hist_cnt[256];
  __shared__ float hist_mass[256];
  __shared__ unsigned sh_prefix;
  __shared__ unsigned sh_remaining;
  __shared__ float sh_mass_above;

  const int rowi = blockIdx.x;
  const __nv_bfloat16* row = logits + static_cast<size_t>(rowi) * ld;
  const float T = temperature[rowi];

  // pass 1: maximum (also the greedy answer)
  ArgPair best{-CUDART_INF_F, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) best = better(best, ArgPair{__bfloat162float(row[i]), i});
  best = block_argmax(best, scratch);
  if (T <= 1e-5f) {
    if (threadIdx.x == 0) out[rowi] = best.i;
    return;
  }
  const float invT = 1.f / T;
  const float mx = best.v;

  // top-k: key of the k-th largest element (0 keeps everything)
  unsigned thr_k = 0;
  const int k = top_k[rowi];
  if (k > 0 && k < vocab) {
    if (threadIdx.x == 0) { sh_prefix = 0; sh_remaining = static_cast<unsigned>(k); }
    __syncthreads();
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      const unsigned mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
      if (threadIdx.x < 256) hist_cnt[threadIdx.x] = 0;
      __syncthreads();
      const unsigned prefix = sh_prefix;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const unsigned key = order_key(__bfloat162float(row[i]));
        if ((key & mask) == prefix) atomicAdd(&hist_cnt[(key >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        unsigned need = sh_remaining, d = 255;
        for (;; --d) {
          if (hist_cnt[d] >= need || d == 0) break;
          need -= hist_cnt[d];
        }
        sh_prefix = prefix | (d << shift);
        sh_remaining = need;
      }
      __syncthreads();
    }
    thr_k = sh_prefix;
  }

  // mass of the top-k survivors
  float z = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float x = __bfloat162float(row[i]);
    if (order_key(x) >= thr_k) z += __expf((x - mx) * invT);
  }
  z = block_sum_f(z, fscratch);

  // top-p: smallest key whose strictly-preceding mass is still <= p * z
  unsigned thr_p = thr_k;
  const float pp = top_p[rowi];
  if (pp < 1.f) {
    const float target = pp * z;
    if (threadIdx.x == 0) { sh_prefix = 0; sh_mass_above = 0.f; }
    __syncthreads();
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      const unsigned mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
      if (threadIdx.x < 256) hist_mass[threadIdx.x] = 0.f;
      __syncthreads();
      const unsigned prefix = sh_prefix;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float x = __bfloat162float(row[i]);
        const unsigned key = order_key(x);
        if (key >= thr_k && (key & mask) == prefix)
          atomicAdd(&hist_mass[(key >> shift) & 255u], __expf((x - mx) * invT));
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        float above = sh_mass_above;
        unsigned d = 255;
        for (;; --d) {
          // descend into the first digit class whose mass crosses the target
          if (above + hist_mass[d] > target || d == 0) break;
          above += hist_mass[d];
        }
        sh_prefix = prefix | (d << shift);
        sh_mass_above = above;
      }
      __syncthreads();
    }
    thr_p = sh_prefix > thr_k ? sh_prefix : thr_k;
  }

  // min-p relative to the most likely token: keep x >= mx + T * ln(min_p)
  const float mp = min_p[rowi];
  const float thr_m = mp > 0.f ? mx + T * __logf(mp) : -CUDART_INF_F;

  // draw: Gumbel-max over the kept set
  const uint32_t seed = static_cast<uint32_t>(rng[0]), step = static_cast<uint32_t>(rng[1]);
  ArgPair pick{-CUDART_INF_F, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float x = __bfloat162float(row[i]);
    if (order_key(x) >= thr_p && x >= thr_m) {
      const float u = uniform01(seed, step, static_cast<uint32_t>(rowi), static_cast<uint32_t>(i));
      const float gum = -__logf(-__logf(u));
      pick = better(pick, ArgPair{(x - mx) * invT + gum, i});
    }
  }
  pick = block_argmax(pick, scratch);
  if (threadIdx.x == 0) out[rowi] = pick.i == 0x7fffffff ? best.i : pick.i;
}

}  // namespace xv

using namespace xv;

extern "C" {

int xv_argmax(const void* logits, long long* out, int rows, int vocab, long long ld, cudaStream_t stream) {
  if (rows <= 0) return 0;
  launch_pdl(argmax_kernel, dim3(rows), dim3(kSampThreads), 0, stream, static_cast<const __nv_bfloat16*>(logits), out, vocab, ld);
  return cudaGetLastError() == cudaSuccess ? 0 : XV_ERR_LAUNCH;
}

int xv_sample(const void* logits, long long* out, int rows, int vocab, long long ld, const float* temperature,
              const int* top_k, const float* top_p, const float* min_p, const int* rng, cudaStream_t stream) {
  if (rows <= 0) return 0;
  launch_pdl(sample_kernel, dim3(rows), dim3(kSampThreads), 0, stream, static_cast<const __nv_bfloat16*>(logits), out, vocab, ld,
                                                   temperature, top_k, top_p, min_p, rng);
  return cudaGetLastError() == cudaSuccess ? 0 : XV_ERR_LAUNCH;
}

}  // extern "C"
