// Token selection over bf16 logits, one CTA per row, no host synchronisation.
//
//   argmax_kernel     - greedy; ties resolve to the lowest token id.
//   sample_kernel     - temperature, top-k, top-p, min-p, then one draw. The kept set is always
//                       "logit >= threshold", so it is found with MSB-first radix selection over
//                       order-preserving integer keys: by element count for top-k, by probability
//                       mass for top-p (no sort of the 152k-entry row, unlike a full descending
//                       sort). bf16 logits have 16 significant key bits, so each selection is two
//                       256-bin passes. Probability mass is accumulated in 2^-40 fixed point, so
//                       the thresholds do not depend on the order in which threads add. The draw
//                       is Gumbel-max over the kept set with a counter-based random stream keyed
//                       by (seed, step, row, token), so replaying a captured graph with a new step
//                       value draws fresh numbers. Elements tied with the k-th value are all kept.
//   tp_sample_kernel  - the same selection over a vocabulary that is sharded across tensor-
//                       parallel ranks, without gathering the logits: every rank scans its own
//                       shard and the ranks exchange only the row maximum, the 256-bin
//                       histograms of each selection pass and their best Gumbel candidate (at
//                       most six exchanges of <= 2 KB per row and peer). All ranks add the same
//                       numbers in rank order and so pick the same thresholds and the same token.
//                       Exchange words carry their own sequence number ({value, seq} in one
//                       8-byte store), so an exchange costs one NVLink write latency and needs no
//                       fence; every wait is bounded and reports through the status word.
//
// The reference gathers the full [rows, vocab] logits on every rank and samples with ATen
// softmax / topk / sort / cumsum / multinomial
// (reference: src/compute/layers/vocab_parallel.py:171-216, src/compute/sampler.py:27-118).

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <string.h>

#include <mutex>

#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "tp_device.cuh"
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

// ---------------------------------------------------------------------------------------------
// Cross-rank exchange for tp_sample_kernel.
//
// Symmetric region layout (byte offsets from `base` in every rank's buffer):
//   [launch parity 0..1][row][source rank] -> one kSampSlotBytes block:
//       [0, 2048)      256 x {value, seq}   histogram passes A (steps 1, 3)
//       [2048, 4096)   256 x {value, seq}   histogram passes B (steps 2, 4)
//       [4096, 4112)   {value, seq, id, seq}  row maximum (step 0)
//       [4112, 4128)   {value, seq, id, seq}  best candidate of the draw (step 5)
// seq = 8 * launch + step + 1 with a launch counter kept in device memory (words 24, 25 of the
// communicator's epoch array), so it never repeats and zeroed memory never matches.
// Reuse: a rank reaches step s + 2 only after it has every peer's step s + 1 data, which a peer sends
// after it has read step s, so steps 1 and 3 (2 and 4) may share a block. A rank finishes launch n + 1
// only after it has heard from every peer's launch n + 1, which starts after that peer's launch n has
// ended, so launch n + 2 may overwrite the blocks of launch n: two parities suffice.
// ---------------------------------------------------------------------------------------------
constexpr int kSampSlotBytes = 4160;
constexpr int kSampLaunchWord = 24;
constexpr int kSampTicketWord = 25;

struct LocalOnly {
  static constexpr bool kDist = false;
  __device__ void begin_row(int) {}
  __device__ ArgPair pair(int, ArgPair p, ArgPair*) { return p; }
  __device__ void sum_u32(int, unsigned*) {}
  __device__ void sum_f32(int, float*) {}
};

struct AcrossRanks {
  static constexpr bool kDist = true;
  TpComm c;
  long long base;          // region offset, this launch's parity included
  uint32_t seq0;           // 8 * launch + 1
  int row;
  int* aborted;            // shared: a wait ran out; the remaining waits are skipped

  __device__ void begin_row(int r) { row = r; }
  __device__ char* slot(int dst, int src) const {
    return const_cast<char*>(static_cast<const char*>(c.peer_buf[dst])) + base +
           (static_cast<long long>(row) * c.world + src) * kSampSlotBytes;
  }
  __device__ static int step_offset(int step) {
    return step == 0 ? 4096 : step == 5 ? 4112 : (step & 1) ? 0 : 2048;
  }
  __device__ bool wait_v2(const char* p, uint32_t seq, uint32_t& val) {
    const unsigned long long t0 = global_timer_ns();
    const unsigned long long limit = static_cast<unsigned long long>(c.spin_limit) * 1000ull;
    for (;;) {
      uint32_t v, s;
      asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v), "=r"(s) : "l"(p) : "memory");
      if (s == seq) {
        val = v;
        return true;
      }
      if (*reinterpret_cast<volatile int*>(aborted)) break;
      if (global_timer_ns() - t0 > limit) {
        report_status(c.status, kTpKernelId, kPeerFlagTimeout);
        *reinterpret_cast<volatile int*>(aborted) = 1;
        break;
      }
    }
    val = 0;
    return false;
  }
  // every rank's candidate, best of all (same on every rank); `arr` is shared scratch of kMaxRanks entries
  __device__ ArgPair pair(int step, ArgPair mine, ArgPair* arr) {
    const uint32_t seq = seq0 + step;
    const int off = step_offset(step);
    const int t = threadIdx.x;
    if (t < c.world) {
      if (t == c.rank) {
        arr[t] = mine;
      } else {
        const uint4 w = make_uint4(__float_as_uint(mine.v), seq, static_cast<uint32_t>(mine.i), seq);
        st_relaxed_sys_v4(slot(t, c.rank) + off, w);
        const char* src = slot(c.rank, t) + off;
        const unsigned long long t0 = global_timer_ns();
        const unsigned long long limit = static_cast<unsigned long long>(c.spin_limit) * 1000ull;
        ArgPair got{-CUDART_INF_F, 0x7fffffff};
        for (;;) {
          const uint4 r = ld_relaxed_sys_v4(src);
          if (r.y == seq && r.w == seq) {
            got.v = __uint_as_float(r.x);
            got.i = static_cast<int>(r.z);
            break;
          }
          if (*reinterpret_cast<volatile int*>(aborted)) break;
          if (global_timer_ns() - t0 > limit) {
            report_status(c.status, kTpKernelId, kPeerFlagTimeout);
            *reinterpret_cast<volatile int*>(aborted) = 1;
            break;
          }
        }
        arr[t] = got;
      }
    }
    __syncthreads();
    ArgPair best = arr[0];
    for (int r = 1; r < c.world; ++r) best = better(best, arr[r]);
    __syncthreads();
    return best;
  }
  // hist[256] (shared) becomes the sum over ranks, added in rank order
  template <typename T>
  __device__ void sum256(int step, T* hist) {
    const uint32_t seq = seq0 + step;
    const int off = step_offset(step);
    const int t = threadIdx.x;
    if (t < 256) {
      const T mine = hist[t];
      uint32_t bits;
      memcpy(&bits, &mine, 4);
      for (int d = 0; d < c.world; ++d)
        if (d != c.rank)
          asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(slot(d, c.rank) + off + t * 8), "r"(bits),
                       "r"(seq)
                       : "memory");
      T acc = 0;
      for (int s = 0; s < c.world; ++s) {
        T v = mine;
        if (s != c.rank) {
          uint32_t got;
          wait_v2(slot(c.rank, s) + off + t * 8, seq, got);
          memcpy(&v, &got, 4);
        }
        acc += v;
      }
      hist[t] = acc;
    }
    __syncthreads();
  }
  __device__ void sum_u32(int step, unsigned* hist) { sum256(step, hist); }
  __device__ void sum_f32(int step, float* hist) { sum256(step, hist); }
};

// Calls fn(value, local index) for every element of row[0, n), eight per 16-byte load where the row allows.
template <typename F>
__device__ __forceinline__ void for_each_logit(const __nv_bfloat16* __restrict__ row, int n, bool vec_ok, F fn) {
  const int nvec = vec_ok ? n / 8 : 0;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 raw = *reinterpret_cast<const uint4*>(row + v * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      fn(f.x, v * 8 + 2 * j);
      fn(f.y, v * 8 + 2 * j + 1);
    }
  }
  for (int i = nvec * 8 + threadIdx.x; i < n; i += blockDim.x) fn(__bfloat162float(row[i]), i);
}

__device__ __forceinline__ unsigned key16(float x) { return order_key(x) >> 16; }

struct SampleShared {
  ArgPair scratch[32];
  ArgPair ranks[kMaxRanks];
  unsigned hist_cnt[256];
  unsigned long long hist_fix[256];
  float hist_mass[256];
  unsigned prefix, remaining;
  float mass_above, target;
};

// One row: logits row[0, n_local) are the tokens id_base .. id_base + n_local of a vocabulary of
// total_vocab tokens. Every thread of the CTA calls this; thread 0 writes the token.
template <class X>
__device__ void sample_row(X& x, SampleShared& sh, const __nv_bfloat16* __restrict__ row, int n_local, int id_base,
                           int total_vocab, bool vec_ok, int rowi, float T, int k, float pp, float mp, uint32_t seed,
                           uint32_t step, long long* __restrict__ out) {
  // maximum (also the greedy answer)
  ArgPair best{-CUDART_INF_F, 0x7fffffff};
  for_each_logit(row, n_local, vec_ok, [&](float v, int i) { best = better(best, ArgPair{v, i + id_base}); });
  best = block_argmax(best, sh.scratch);
  best = x.pair(0, best, sh.ranks);
  if (T <= 1e-5f) {
    if (threadIdx.x == 0) out[rowi] = best.i;
    return;
  }
  const float invT = 1.f / T;
  const float mx = best.v;

  // top-k: 16-bit key of the k-th largest element (0 keeps everything)
  unsigned thr_k = 0;
  if (k > 0 && k < total_vocab) {
    if (threadIdx.x == 0) { sh.prefix = 0; sh.remaining = static_cast<unsigned>(k); }
    __syncthreads();
    for (int pass = 0; pass < 2; ++pass) {
      if (threadIdx.x < 256) sh.hist_cnt[threadIdx.x] = 0;
      __syncthreads();
      const unsigned prefix = sh.prefix;
      for_each_logit(row, n_local, vec_ok, [&](float v, int) {
        const unsigned key = key16(v);
        if (pass == 0) atomicAdd(&sh.hist_cnt[key >> 8], 1u);
        else if ((key >> 8) == prefix) atomicAdd(&sh.hist_cnt[key & 255u], 1u);
      });
      __syncthreads();
      x.sum_u32(1 + pass, sh.hist_cnt);
      if (threadIdx.x == 0) {
        unsigned need = sh.remaining, d = 255;
        for (;; --d) {
          if (sh.hist_cnt[d] >= need || d == 0) break;
          need -= sh.hist_cnt[d];
        }
        sh.prefix = pass == 0 ? d : ((prefix << 8) | d);
        sh.remaining = need;
      }
      __syncthreads();
    }
    thr_k = sh.prefix;
  }

  // top-p over the top-k survivors: smallest key whose strictly-preceding mass is still <= p * total mass
  unsigned thr_p = thr_k;
  if (pp < 1.f) {
    if (threadIdx.x == 0) { sh.prefix = 0; sh.mass_above = 0.f; }
    __syncthreads();
    for (int pass = 0; pass < 2; ++pass) {
      if (threadIdx.x < 256) sh.hist_fix[threadIdx.x] = 0ull;
      __syncthreads();
      const unsigned prefix = sh.prefix;
      for_each_logit(row, n_local, vec_ok, [&](float v, int) {
        const unsigned key = key16(v);
        if (key >= thr_k && (pass == 0 || (key >> 8) == prefix)) {
          const unsigned long long m = __float2ull_rz(__expf((v - mx) * invT) * 1099511627776.f);   // 2^40
          atomicAdd(&sh.hist_fix[pass == 0 ? (key >> 8) : (key & 255u)], m);
        }
      });
      __syncthreads();
      if (threadIdx.x < 256)
        sh.hist_mass[threadIdx.x] = static_cast<float>(sh.hist_fix[threadIdx.x]) * (1.f / 1099511627776.f);
      __syncthreads();
      x.sum_f32(3 + pass, sh.hist_mass);
      if (threadIdx.x == 0) {
        if (pass == 0) {
          float z = 0.f;
          for (int d = 0; d < 256; ++d) z += sh.hist_mass[d];
          sh.target = pp * z;
        }
        const float target = sh.target;
        float above = sh.mass_above;
        unsigned d = 255;
        for (;; --d) {
          // descend into the first digit class whose mass crosses the target
          if (above + sh.hist_mass[d] > target || d == 0) break;
          above += sh.hist_mass[d];
        }
        sh.prefix = pass == 0 ? d : ((prefix << 8) | d);
        sh.mass_above = above;
      }
      __syncthreads();
    }
    thr_p = sh.prefix > thr_k ? sh.prefix : thr_k;
  }

  // min-p relative to the most likely token: keep x >= mx + T * ln(min_p)
  const float thr_m = mp > 0.f ? mx + T * __logf(mp) : -CUDART_INF_F;

  // draw: Gumbel-max over the kept set
  ArgPair pick{-CUDART_INF_F, 0x7fffffff};
  for_each_logit(row, n_local, vec_ok, [&](float v, int i) {
    if (key16(v) >= thr_p && v >= thr_m) {
      const int gid = i + id_base;
      const float u = uniform01(seed, step, static_cast<uint32_t>(rowi), static_cast<uint32_t>(gid));
      const float gum = -__logf(-__logf(u));
      pick = better(pick, ArgPair{(v - mx) * invT + gum, gid});
    }
  });
  pick = block_argmax(pick, sh.scratch);
  pick = x.pair(5, pick, sh.ranks);
  if (threadIdx.x == 0) out[rowi] = pick.i == 0x7fffffff ? best.i : pick.i;
}

__global__ void __launch_bounds__(kSampThreads)
sample_kernel(const __nv_bfloat16* __restrict__ logits, long long* __restrict__ out, int vocab, long long ld,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p, const int* __restrict__ rng) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ SampleShared sh;
  const int rowi = blockIdx.x;
  const bool vec_ok = (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  LocalOnly x;
  sample_row(x, sh, logits + static_cast<size_t>(rowi) * ld, vocab, 0, vocab, vec_ok, rowi, temperature[rowi],
             top_k[rowi], top_p[rowi], min_p[rowi], static_cast<uint32_t>(rng[0]), static_cast<uint32_t>(rng[1]), out);
}

// Vocabulary-parallel form: logits is this rank's [rows, local_vocab] shard holding tokens
// vocab_start .. vocab_start + valid_vocab. The grid is capped at what can be resident and walks the rows.
__global__ void __launch_bounds__(kSampThreads, 2)
tp_sample_kernel(const TpComm c, long long region_offset, long long parity_bytes,
                 const __nv_bfloat16* __restrict__ logits, long long ld, int valid_vocab, int vocab_start,
                 int total_vocab, long long* __restrict__ out, int rows, const float* __restrict__ temperature,
                 const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
                 const int* __restrict__ rng) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ SampleShared sh;
  __shared__ int aborted;
  const uint32_t launch = *reinterpret_cast<volatile uint32_t*>(c.epoch + kSampLaunchWord);
  if (threadIdx.x == 0) aborted = 0;
  __syncthreads();
  AcrossRanks x;
  x.c = c;
  x.base = region_offset + static_cast<long long>(launch & 1u) * parity_bytes;
  x.seq0 = launch * 8u + 1u;
  x.row = 0;
  x.aborted = &aborted;
  const bool vec_ok = (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  const uint32_t seed = static_cast<uint32_t>(rng[0]), step = static_cast<uint32_t>(rng[1]);
  for (int rowi = blockIdx.x; rowi < rows; rowi += gridDim.x) {
    x.begin_row(rowi);
    sample_row(x, sh, logits + static_cast<size_t>(rowi) * ld, valid_vocab, vocab_start, total_vocab, vec_ok, rowi,
               temperature[rowi], top_k[rowi], top_p[rowi], min_p[rowi], seed, step, out);
    __syncthreads();
  }
  // the last CTA to finish advances the launch counter (every CTA has read it by then)
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(c.epoch + kSampTicketWord, 1u) == gridDim.x - 1) {
      c.epoch[kSampTicketWord] = 0;
      __threadfence();
      atomicAdd(c.epoch + kSampLaunchWord, 1u);
    }
  }
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

// Bytes of the symmetric region xv_tp_sample needs for `max_rows` rows on `world` ranks.
long long xv_tp_sample_region_bytes(int max_rows, int world) {
  return 2ll * max_rows * world * kSampSlotBytes;
}

int xv_tp_sample(const void* const* peer_bufs, void* const* peer_flags, void* epoch, int rank, int world,
                 long long region_offset, int max_rows, const void* logits, long long ld, int valid_vocab,
                 int vocab_start, int total_vocab, long long* out, int rows, const float* temperature,
                 const int* top_k, const float* top_p, const float* min_p, const int* rng, unsigned spin_us,
                 int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || rows > max_rows) return XV_ERR_SHAPE;
  if (region_offset % 16) return XV_ERR_ALIGN;
  TpComm c;
  for (int r = 0; r < kMaxRanks; ++r) {
    c.peer_buf[r] = r < world ? peer_bufs[r] : nullptr;
    c.peer_flags[r] = r < world ? static_cast<uint32_t*>(peer_flags[r]) : nullptr;
  }
  c.mc_buf = nullptr;
  c.epoch = static_cast<uint32_t*>(epoch);
  c.rank = rank;
  c.world = world;
  c.spin_limit = spin_us;
  c.status = status;
  // CTAs that can be resident at once on this device (occupancy x SM count), looked up once per device
  static int resident[16] = {0};
  static std::mutex resident_mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return XV_ERR_LAUNCH;
  int cap = 0;
  {
    std::lock_guard<std::mutex> g(resident_mu);
    if (resident[dev] == 0) {
      int per_sm = 0, sms = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, tp_sample_kernel, kSampThreads, 0) != cudaSuccess ||
          cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || per_sm < 1 || sms < 1)
        return XV_ERR_LAUNCH;
      resident[dev] = per_sm * sms;
    }
    cap = resident[dev];
  }
  const int grid = rows < cap ? rows : cap;
  const long long parity_bytes = static_cast<long long>(max_rows) * world * kSampSlotBytes;
  launch_pdl(tp_sample_kernel, dim3(grid), dim3(kSampThreads), 0, stream, c, region_offset, parity_bytes,
             static_cast<const __nv_bfloat16*>(logits), ld, valid_vocab, vocab_start, total_vocab, out, rows,
             temperature, top_k, top_p, min_p, rng);
  return cudaGetLastError() == cudaSuccess ? 0 : XV_ERR_LAUNCH;
}

}  // extern "C"
