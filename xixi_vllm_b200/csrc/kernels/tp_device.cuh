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

// ---- push protocol: GEMM epilogue -> row owners' slots -> sum + residual + RMSNorm -> broadcast ----------
//
// A row-parallel projection under tensor parallelism is ONE kernel. Its GEMM epilogue writes every
// finished tile of this rank's partial product straight into the memory of the ranks that will reduce
// it ("slots": one copy of the rows per source), then raises an arrival counter there. Rows are dealt
// round-robin: rank r owns rows r, r + world, ... (two-shot form; traffic per GPU does not grow with the
// number of ranks). The owner sums the sources in a fixed order, adds its rows of the residual stream,
// normalises and broadcasts the result into every rank's activation buffer (multimem.st through
// NVSwitch, or one peer store per rank), then raises a second counter. With few rows the one-shot form
// is cheaper: every rank receives all rows from all sources and reduces all of them itself; there is no
// broadcast and no second wait.
//
// Counters only grow. Each rank keeps, in local device memory, the value every counter had reached
// when the previous call ended; a call waits for that value plus the number of arrivals it expects.
// A rank cannot leave call k before every rank has delivered its part of call k, so arrivals that
// belong to call k + 1 can only come on top of a complete call k and never satisfy a wait early.
// Every wait is bounded by `spin_limit`; on expiry the kernel records a status code and carries on to
// its end (its output is then garbage, the host raises).
//
// Slot array of one call, at byte `slot_offset` of the symmetric buffer of the reducing rank:
//   [world * splits sources][cap_rows][hidden] bf16, source index = rank * splits + k_split.
// The caller alternates between two arrays, so the array written in call k is not written again
// before call k + 2, by which time its owner has finished reading it (same argument as above).
constexpr int kPushArriveWord = 32;   // flag words [32, 40): tiles arrived from source rank s
constexpr int kPushBcastWord = 64;    // flag words [64, 72): rows arrived from owner rank o
constexpr int kPushTicketWord = 6;    // TpComm::epoch word: CTAs of the running call that have finished
constexpr int kPushArriveBase = 8;    // TpComm::epoch words [8, 16): arrive counters at the end of the last call
constexpr int kPullDoneChannel = 2;   // flag words [16, 24): the row-sharded reduction's "my rows are broadcast" epoch flags
constexpr int kPullTargetWord = 26;   // TpComm::epoch word: epoch of the last row-sharded reduction that left its wait to the consumer
constexpr int kPushBcastBase = 16;    // TpComm::epoch words [16, 24): broadcast counters at the end of the last call
constexpr int kTpPushKernelId = 4;

struct TpPush {
  int enabled;
  int two_shot;                        // 1: rows dealt to owners; 0: every rank reduces every row
  TpComm comm;
  long long slot_offset;
  int cap_rows;                        // rows per source in the slot array
  int splits;                          // K splits of the GEMM, pushed as separate sources
  long long h_offset;                  // two-shot: byte offset (symmetric buffer) the finished rows are broadcast to
  __nv_bfloat16* y;                    // one-shot: local [rows, hidden] output
  const __nv_bfloat16* residual_in;    // [rows, hidden] local; two-shot touches only this rank's rows; may be null
  __nv_bfloat16* residual_out;
  const __nv_bfloat16* norm_w;
  int rows, hidden;
  float eps;
  int mode;                            // 0: residual add + RMSNorm; 1: plain sum
  int signal_ctas;                     // CTAs of this launch that own GEMM work (each raises its counter once)
  unsigned long long* prof;            // optional: 8 global-timer stamps per CTA (see xv_tp_profile_buffer)
  int defer_row_wait;                  // two-shot: do not hold the kernel open until every owner's rows have arrived;
                                       // the kernel that reads the activation waits for them itself (GemmRowWait)
};

// What a GEMM needs to wait, before its first activation tile, for the rows that the one-kernel projection
// before it has other ranks broadcast into this rank's activation buffer (all-gather -> GEMM): the per-owner
// arrival counters in this rank's flag array and the values they must reach (the projection's last CTA
// wrote those into the communicator's history words before it ended).
struct GemmRowWait {
  const uint32_t* flags;     // this rank's flag array: one word per source rank
  const uint32_t* targets;   // values the flags must reach (local device memory)
  int n;                     // ranks (0: nothing to wait for)
  unsigned spin_us;
  int target_stride;         // 1: one target per rank (monotonic counters); 0: all ranks reach the same value (an epoch)
};



__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Polls until the counter at `f` has reached `target` (signed distance, so wrap-around is harmless).
__device__ __forceinline__ bool tp_wait_counter(const uint32_t* f, uint32_t target, unsigned spin_us) {
  unsigned long long t0 = 0;
  const unsigned long long limit = static_cast<unsigned long long>(spin_us) * 1000ull;
  for (int polls = 0;; ++polls) {
    if (static_cast<int32_t>(ld_acquire_sys(f) - target) >= 0) return true;
    if (polls == 64) t0 = global_timer_ns();
    if (polls > 64) {
      if (global_timer_ns() - t0 > limit) return false;
      __nanosleep(32);
    }
  }
}

// Called by the one thread that issues the GEMM's TMA loads. The loads that follow read memory that peers wrote
// through NVLink, so the acquire is followed by a cross-proxy fence.
__device__ __forceinline__ bool gemm_wait_rows(const GemmRowWait& w) {
  bool ok = true;
  for (int r = 0; r < w.n; ++r) {
    const uint32_t target = *reinterpret_cast<const volatile uint32_t*>(w.targets + r * w.target_stride);
    ok = tp_wait_counter(w.flags + r, target, w.spin_us) && ok;
  }
  if (w.n > 0) asm volatile("fence.proxy.async;" ::: "memory");
  return ok;
}

// Phase stamps of the one-kernel projection, per CTA: 0 kernel entry, 1 GEMM roles done (tiles pushed, arrival
// raised), 2 all sources' tiles arrived, 3 this CTA's rows reduced and stored / broadcast, 4 broadcast raised,
// 5 every owner's rows arrived (CTA 0 only), 6 exit.
__device__ __forceinline__ void tp_prof(const TpPush& t, int slot) {
  if (t.prof != nullptr && threadIdx.x == 0) t.prof[blockIdx.x * 8 + slot] = global_timer_ns();
}

__device__ __forceinline__ int tp_rows_owned(int rows, int owner, int world) {
  return rows > owner ? (rows - owner + world - 1) / world : 0;
}

// Eight bf16 values of row `row`, columns col .. col + 7, of this rank's partial (K split `split`)
// to wherever they will be reduced.
__device__ __forceinline__ void tp_push_store8(const TpPush& t, int row, int col, int split, const uint4& v) {
  const int src = t.comm.rank * t.splits + split;
  if (t.two_shot) {
    const int owner = row % t.comm.world;
    const int slot_row = row / t.comm.world;
    char* dst = const_cast<char*>(static_cast<const char*>(t.comm.peer_buf[owner])) + t.slot_offset +
                ((static_cast<long long>(src) * t.cap_rows + slot_row) * t.hidden + col) * 2;
    st_relaxed_sys_v4(dst, v);
  } else {
    const long long off = t.slot_offset + ((static_cast<long long>(src) * t.cap_rows + row) * t.hidden + col) * 2;
    if (t.comm.mc_buf != nullptr) {
      multimem_st_bf16x8(const_cast<char*>(static_cast<const char*>(t.comm.mc_buf)) + off, v);
    } else {
      for (int r = 0; r < t.comm.world; ++r)
        st_relaxed_sys_v4(const_cast<char*>(static_cast<const char*>(t.comm.peer_buf[r])) + off, v);
    }
  }
}

// Called by threads 0 .. world-1 of the group that pushed, after a barrier among that group:
// "this CTA's tiles have been written" on every rank.
__device__ __forceinline__ void tp_push_signal_tiles(const TpPush& t, int peer) {
  // the release orders this thread's earlier stores and, through the barrier it follows, the group's
  red_release_sys_add(t.comm.peer_flags[peer] + kPushArriveWord + t.comm.rank, 1u);
}

// Second half of the kernel, run by all threads of every CTA once the CTA's GEMM work is done.
template <int MAXVEC>
__device__ __noinline__ void tp_push_tail(const TpPush& t) {
  __shared__ float scratch[32];
  const int world = t.comm.world, rank = t.comm.rank;
  const int nthreads = blockDim.x;
  volatile uint32_t* st = t.comm.epoch;
  const int n_mine = t.two_shot ? tp_rows_owned(t.rows, rank, world) : t.rows;
  // rows go to the CTAs from the end of the grid first: those are the ones without GEMM tiles
  const int first = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  tp_prof(t, 1);
  if (first < n_mine) {
    const int nvec = t.hidden >> 3;
    // What does not depend on the peers is fetched before the wait: the norm weights and the first row's residual.
    uint4 wv[MAXVEC], rv[MAXVEC];
    {
      const int row0 = t.two_shot ? rank + first * world : first;
#pragma unroll
      for (int u = 0; u < MAXVEC; ++u) {
        const int v = threadIdx.x + u * nthreads;
        wv[u] = make_uint4(0u, 0u, 0u, 0u);
        rv[u] = make_uint4(0u, 0u, 0u, 0u);
        if (v < nvec && t.mode == 0) {
          wv[u] = *reinterpret_cast<const uint4*>(t.norm_w + v * 8);
          if (t.residual_in != nullptr)
            rv[u] = *reinterpret_cast<const uint4*>(t.residual_in + static_cast<size_t>(row0) * t.hidden + v * 8);
        }
      }
    }
    if (threadIdx.x < world) {
      const uint32_t target = st[kPushArriveBase + threadIdx.x] + static_cast<uint32_t>(t.signal_ctas);
      if (!tp_wait_counter(t.comm.peer_flags[rank] + kPushArriveWord + threadIdx.x, target, t.comm.spin_limit))
        report_status(t.comm.status, kTpPushKernelId, kPeerFlagTimeout);
    }
    __syncthreads();
    tp_prof(t, 2);
    const char* slots = static_cast<const char*>(t.comm.peer_buf[rank]) + t.slot_offset;
    const int n_src = world;          // K splits are summed before the push
    for (int i = first; i < n_mine; i += gridDim.x) {
      const int row = t.two_shot ? rank + i * world : i;
      float vals[MAXVEC][8];
      float ss = 0.f;
      const long long src_stride = static_cast<long long>(t.cap_rows) * t.hidden * 2;
      // two 16-byte columns of the row at a time: all their sources' loads are issued before the first sum,
      // so a round costs one memory round trip instead of one per source
#pragma unroll
      for (int u0 = 0; u0 < MAXVEC; u0 += 2) {
        if (threadIdx.x + u0 * nthreads < nvec) {
          uint4 raw[2][kMaxRanks];
#pragma unroll
          for (int du = 0; du < 2; ++du) {
            const int v = threadIdx.x + (u0 + du) * nthreads;
            const char* p0 = slots + (static_cast<long long>(i) * t.hidden + (v < nvec ? v : 0) * 8) * 2;
#pragma unroll
            for (int s = 0; s < kMaxRanks; ++s)
              raw[du][s] = (s < n_src && v < nvec) ? ld_relaxed_sys_v4(p0 + s * src_stride) : make_uint4(0u, 0u, 0u, 0u);
          }
#pragma unroll
          for (int du = 0; du < 2; ++du) {
            const int u = u0 + du;
            const int v = threadIdx.x + u * nthreads;
            if (v < nvec) {
              float acc[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
              for (int s = 0; s < kMaxRanks; ++s) {     // fixed order, fp32: the result does not depend on arrival order
                if (s < n_src) {
                  float x[8];
                  unpack8(raw[du][s], x);
#pragma unroll
                  for (int j = 0; j < 8; ++j) acc[j] += x[j];
                }
              }
              if (t.mode == 0) {
                const size_t ro = static_cast<size_t>(row) * t.hidden + v * 8;
                if (t.residual_in != nullptr) {
                  float rr[8];
                  unpack8(i == first ? rv[u] : *reinterpret_cast<const uint4*>(t.residual_in + ro), rr);
#pragma unroll
                  for (int j = 0; j < 8; ++j) acc[j] += rr[j];
                }
                *reinterpret_cast<uint4*>(t.residual_out + ro) = pack8(acc);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  acc[j] = __bfloat162float(__float2bfloat16(acc[j]));
                  ss += acc[j] * acc[j];
                }
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) vals[u][j] = acc[j];
            }
          }
        }
      }
      float inv = 1.f;
      if (t.mode == 0) {
        ss = warp_sum(ss);
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (lane == 0) scratch[warp] = ss;
        __syncthreads();
        float tot = lane < (nthreads >> 5) ? scratch[lane] : 0.f;
        tot = warp_sum(tot);
        __syncthreads();
        inv = rsqrtf(tot / static_cast<float>(t.hidden) + t.eps);
      }
#pragma unroll
      for (int u = 0; u < MAXVEC; ++u) {
        const int v = threadIdx.x + u * nthreads;
        if (v < nvec) {
          float o[8];
          if (t.mode == 0) {
            float g[8];
            unpack8(wv[u], g);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = vals[u][j] * inv * g[j];
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = vals[u][j];
          }
          const uint4 packed = pack8(o);
          if (!t.two_shot) {
            *reinterpret_cast<uint4*>(t.y + static_cast<size_t>(row) * t.hidden + v * 8) = packed;
          } else {
            const long long off = t.h_offset + (static_cast<long long>(row) * t.hidden + v * 8) * 2;
            if (t.comm.mc_buf != nullptr) {
              multimem_st_bf16x8(const_cast<char*>(static_cast<const char*>(t.comm.mc_buf)) + off, packed);
            } else {
              for (int r = 0; r < world; ++r)
                st_relaxed_sys_v4(const_cast<char*>(static_cast<const char*>(t.comm.peer_buf[r])) + off, packed);
            }
          }
        }
      }
    }
    tp_prof(t, 3);
    if (t.two_shot) {
      __syncthreads();
      if (threadIdx.x < world) red_release_sys_add(t.comm.peer_flags[threadIdx.x] + kPushBcastWord + rank, 1u);
    }
    tp_prof(t, 4);
  }
  // One CTA keeps the kernel open until every owner's rows have landed in this rank's activation
  // buffer: the kernel's end then means "the whole [rows, hidden] activation is here".
  if (t.two_shot && !t.defer_row_wait && blockIdx.x == 0 && threadIdx.x < world) {
    const int owned = tp_rows_owned(t.rows, threadIdx.x, world);
    const int expect = owned < static_cast<int>(gridDim.x) ? owned : static_cast<int>(gridDim.x);
    const uint32_t target = st[kPushBcastBase + threadIdx.x] + static_cast<uint32_t>(expect);
    if (!tp_wait_counter(t.comm.peer_flags[rank] + kPushBcastWord + threadIdx.x, target, t.comm.spin_limit))
      report_status(t.comm.status, kTpPushKernelId, kPeerFlagTimeout);
  }
  // The last CTA to get here moves the per-counter bases on for the next call.
  __syncthreads();
  if (t.two_shot && blockIdx.x == 0) tp_prof(t, 5);
  tp_prof(t, 6);
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(t.comm.epoch + kPushTicketWord, 1u) == gridDim.x - 1) {
      t.comm.epoch[kPushTicketWord] = 0;
      for (int r = 0; r < world; ++r) {
        t.comm.epoch[kPushArriveBase + r] += static_cast<uint32_t>(t.signal_ctas);
        if (t.two_shot) {
          const int owned = tp_rows_owned(t.rows, r, world);
          t.comm.epoch[kPushBcastBase + r] +=
              static_cast<uint32_t>(owned < static_cast<int>(gridDim.x) ? owned : static_cast<int>(gridDim.x));
        }
      }
      __threadfence();
    }
  }
}

}  // namespace xv
