// Device-side pieces shared by the tensor-parallel kernels: the communicator descriptor, the
// system-scope flag protocol, peer loads and the in-switch (multimem) reduction load.
// See tp_fused.cu for the protocol description.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/ptx.cuh"

namespace xv {

constexpr int kMaxRanks = 8;
constexpr int kTpKernelId = 3;
constexpr int kTpThreads = 256;

struct TpComm {
  const void* peer_buf[kMaxRanks];   // every rank's symmetric buffer base, as mapped here
  uint32_t* peer_flags[kMaxRanks];   // every rank's flag array (kMaxRanks words per channel)
  const void* mc_buf;                // multicast address of the buffer (nullptr = no NVLS)
  uint32_t* epoch;                   // [0] current epoch, [1] finished-CTA ticket (local memory)
  int rank, world;
  unsigned spin_limit;               // longest wait for a peer, in microseconds
  int* status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// Sum over all ranks of eight bf16 values, reduced inside NVSwitch with fp32 accumulation.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}

// Broadcast of eight bf16 values to the same offset on every rank through NVSwitch.
__device__ __forceinline__ void multimem_st_bf16x8(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_v4(void* p, const uint4& v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Announce this rank's data for `epoch` (one thread of the grid) and wait until every rank has
// announced. Returns false if a peer never arrived within the spin limit.
__device__ inline bool tp_barrier(const TpComm& c, uint32_t epoch, int channel) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < c.world) {
    __threadfence_system();   // the producer kernel's writes are ordered before the flag
    st_release_sys(c.peer_flags[threadIdx.x] + channel * kMaxRanks + c.rank, epoch);
  }
  if (threadIdx.x < c.world) {
    const uint32_t* f = c.peer_flags[c.rank] + channel * kMaxRanks + threadIdx.x;
    bool seen = false;
    const unsigned long long t0 = global_timer_ns();
    const unsigned long long limit = static_cast<unsigned long long>(c.spin_limit) * 1000ull;
    for (;;) {
      // epochs only grow; signed distance tolerates wrap-around
      if (static_cast<int32_t>(ld_acquire_sys(f) - epoch) >= 0) {
        seen = true;
        break;
      }
      if (global_timer_ns() - t0 > limit) break;
      __nanosleep(20);
    }
    if (!seen) {
      report_status(c.status, kTpKernelId, kPeerFlagTimeout);
      ok_flag = 0;
    }
  }
  __syncthreads();
  return ok_flag != 0;
}

// Last CTA to finish advances the epoch for the next call and resets the ticket.
__device__ inline void tp_finish(const TpComm& c) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned t = atomicAdd(c.epoch + 1, 1u);
    if (t == gridDim.x - 1) {
      c.epoch[1] = 0;
      __threadfence();
      atomicAdd(c.epoch, 1u);
    }
  }
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  v.x = pack_bf16(f[0], f[1]);
  v.y = pack_bf16(f[2], f[3]);
  v.z = pack_bf16(f[4], f[5]);
  v.w = pack_bf16(f[6], f[7]);
  return v;
}


// Sum over ranks of the eight bf16 values at byte offset `off` of the symmetric buffer.
__device__ __forceinline__ void tp_load_sum8(const TpComm& c, long long off, float (&acc)[8]) {
  if (c.mc_buf != nullptr) {
    unpack8(multimem_ld_reduce_bf16x8(static_cast<const char*>(c.mc_buf) + off), acc);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    // fixed rank order, fp32 accumulation: every rank computes bit-identical sums
    for (int r = 0; r < c.world; ++r) {
      float t[8];
      unpack8(ld_relaxed_sys_v4(static_cast<const char*>(c.peer_buf[r]) + off), t);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += t[j];
    }
  }
}

// Bounded grid-wide barrier for kernels whose whole grid is resident. `sync[0]` counts
// arrivals, `sync[1]` is the generation; both live in local device memory and survive across
// launches. Returns false if the other CTAs did not arrive within `timeout_ns`.
__device__ inline bool grid_barrier(uint32_t* sync, unsigned long long timeout_ns) {
  __shared__ int grid_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    grid_ok = 1;
    volatile uint32_t* gen = sync + 1;
    const uint32_t g = *gen;
    __threadfence();
    if (atomicAdd(sync, 1u) == gridDim.x - 1) {
      sync[0] = 0;
      __threadfence();
      atomicAdd(sync + 1, 1u);
    } else {
      const unsigned long long t0 = global_timer_ns();
      while (*gen == g) {
        if (global_timer_ns() - t0 > timeout_ns) {
          grid_ok = 0;
          break;
        }
        __nanosleep(40);
      }
    }
    __threadfence();
  }
  __syncthreads();
  return grid_ok != 0;
}

// Rows `blockIdx.x, blockIdx.x + gridDim.x, ...` of the cross-rank sum, for any block size with
// blockDim.x * MAXVEC * 8 >= hidden.
// mode 0: residual_out = sum (+ residual_in); y = rmsnorm(residual_out) * w.   mode 1: y = sum.
template <int MAXVEC>
__device__ inline void tp_reduce_rows(const TpComm& c, long long buf_offset, const __nv_bfloat16* __restrict__ residual_in,
                                      __nv_bfloat16* __restrict__ residual_out, const __nv_bfloat16* __restrict__ w,
                                      __nv_bfloat16* __restrict__ y, int rows, int hidden, float eps, int mode,
                                      float* scratch /* 32 floats of shared memory */) {
  const int nvec = hidden >> 3;
  const int nthreads = blockDim.x;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long off = buf_offset + static_cast<long long>(row) * hidden * 2;
    float vals[MAXVEC][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXVEC; ++i) {
      const int v = threadIdx.x + i * nthreads;
      if (v < nvec) {
        float acc[8];
        tp_load_sum8(c, off + v * 16, acc);
        if (mode == 0) {
          if (residual_in != nullptr) {
            float rr[8];
            unpack8(*reinterpret_cast<const uint4*>(residual_in + static_cast<size_t>(row) * hidden + v * 8), rr);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += rr[j];
          }
          *reinterpret_cast<uint4*>(residual_out + static_cast<size_t>(row) * hidden + v * 8) = pack8(acc);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            acc[j] = __bfloat162float(__float2bfloat16(acc[j]));
            ss += acc[j] * acc[j];
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[i][j] = acc[j];
      }
    }
    float inv = 1.f;
    if (mode == 0) {
      ss = warp_sum(ss);
      const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
      if (lane == 0) scratch[warp] = ss;
      __syncthreads();
      float t = lane < (nthreads >> 5) ? scratch[lane] : 0.f;
      t = warp_sum(t);
      __syncthreads();
      inv = rsqrtf(t / static_cast<float>(hidden) + eps);
    }
#pragma unroll
    for (int i = 0; i < MAXVEC; ++i) {
      const int v = threadIdx.x + i * nthreads;
      if (v < nvec) {
        float o[8];
        if (mode == 0) {
          float g[8];
          unpack8(*reinterpret_cast<const uint4*>(w + v * 8), g);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * inv * g[j];
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = vals[i][j];
        }
        *reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * hidden + v * 8) = pack8(o);
      }
    }
  }
}

// Everything a GEMM needs to finish with the cross-rank reduction in the same kernel.
struct TpTail {
  int enabled;
  TpComm comm;
  long long buf_offset;                 // byte offset of the [rows, hidden] bf16 partial in the symmetric buffer
  const __nv_bfloat16* residual_in;
  __nv_bfloat16* residual_out;
  const __nv_bfloat16* norm_w;
  __nv_bfloat16* y;
  int rows, hidden;
  float eps;
  int mode;
  uint32_t* grid_sync;                  // two words of local device memory, zero-initialised once
  const float* partials;                // split-K planes to fold first (splits > 1)
  int splits;
  long long split_stride;
};

}  // namespace xv
