// Tensor-parallel reductions over NVLink peer memory, fused with what follows them.
//
// Every rank keeps its partial results in a *symmetric* buffer: the same allocation exists on
// each GPU and every rank has all peers' copies mapped into its address space (and, when the
// fabric supports it, one multicast address that reaches all copies through NVSwitch).
//
//   tp_reduce_norm_kernel   - sum of the ranks' partial [T,H] tiles + residual add + RMSNorm in
//                             one pass. Peers are read with plain system-scope loads from their
//                             mapped buffers, or the sum is fetched already reduced inside the
//                             switch with multimem.ld_reduce. The producing GEMM (or embedding
//                             lookup) writes straight into the symmetric buffer, so there is no
//                             NCCL call, no staging copy and no separate add+norm kernel.
//   tp_argmax_kernel        - vocab-parallel greedy sampling: local argmax of this rank's logit
//                             shard, (value, id) pushed into every peer's slot, global pick.
//   tp_allgather_cols_kernel - full logits for sampled requests: every rank pushes its vocabulary
//                             shard into all ranks' logits matrix (multimem.st or peer stores).
//
// Synchronisation: a monotonically increasing epoch per communicator, kept in device memory
// (so a captured CUDA graph advances it on every replay). A rank announces "my partial for
// epoch e is complete" by storing e into its slot of every peer's flag array with a
// system-scope release; consumers poll their own flag array with acquire loads. Polls are
// bounded: after `spin_limit` microseconds the kernel records a status code and returns.
//
// Buffer reuse rule (enforced by the caller): the buffer written for call k may be rewritten
// only after the caller has passed the barrier of call k+1, i.e. never in two consecutive calls.
//
// The reference does these steps as NCCL all-reduce / all-gather calls followed by separate
// kernels (reference: src/compute/layers/linear.py:141-154, src/compute/layers/vocab_parallel.py:171-216).

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "tp_device.cuh"
#include "xv_cuda.h"

namespace xv {

constexpr int kTpMaxVec = 4;   // hidden <= 256 * 4 * 8 = 8192

// mode 0: y = rmsnorm(sum + residual) * w, residual (in/out) updated; residual_in may be null,
//         in which case residual_out receives the plain sum.
// mode 1: y = sum (all-reduce only).
__global__ void __launch_bounds__(kTpThreads)
tp_reduce_norm_kernel(const TpComm c, long long buf_offset, const __nv_bfloat16* __restrict__ residual_in,
                      __nv_bfloat16* __restrict__ residual_out, const __nv_bfloat16* __restrict__ w,
                      __nv_bfloat16* __restrict__ y, int rows, int hidden, float eps, int mode) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ float scratch[32];
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(c.epoch);
  const bool ok = tp_barrier(c, epoch, 0);
  if (ok)
    tp_reduce_rows<kTpMaxVec>(c, buf_offset, residual_in, residual_out, w, y, rows, hidden, eps, mode, scratch);
  tp_finish(c);
}

// Row-sharded ("two-shot") form of the reduction point, used by the native forward:
//   barrier -> rank r sums rows r, r + world, ... of all ranks' partials (in-switch or by peer
//   loads), adds its shard of the residual stream (which stays sharded by rows: only the owner
//   ever reads a residual row), normalises, and broadcasts the normalised rows into every rank's
//   activation buffer (multimem.st or peer stores) -> barrier, so the kernel's end means the full
//   [rows, hidden] activation is present on every rank.
// Per reduction each GPU sends and receives about rows*hidden*2 bytes regardless of the number
// of ranks; the one-shot kernel above moves world times more and is kept for small worlds and
// for callers that need the full residual on every rank (pipeline hand-off).
__global__ void __launch_bounds__(kTpThreads, 4)
tp_reduce_norm_sharded_kernel(const TpComm c, long long buf_offset, long long h_offset, int has_residual,
                              __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ w, int rows,
                              int hidden, float eps, int defer_wait) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ float scratch[32];
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(c.epoch);
  bool ok = tp_barrier(c, epoch, 0);
  const int nvec = hidden >> 3;
  if (ok) {
    for (int row = c.rank + c.world * static_cast<int>(blockIdx.x); row < rows; row += c.world * gridDim.x) {
      const long long off = buf_offset + static_cast<long long>(row) * hidden * 2;
      float vals[kTpMaxVec][8];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < kTpMaxVec; ++i) {
        const int v = threadIdx.x + i * kTpThreads;
        if (v < nvec) {
          float acc[8];
          tp_load_sum8(c, off + v * 16, acc);
          __nv_bfloat16* rr = residual + static_cast<size_t>(row) * hidden + v * 8;
          if (has_residual) {
            float t[8];
            unpack8(*reinterpret_cast<const uint4*>(rr), t);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += t[j];
          }
          *reinterpret_cast<uint4*>(rr) = pack8(acc);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            acc[j] = __bfloat162float(__float2bfloat16(acc[j]));
            ss += acc[j] * acc[j];
            vals[i][j] = acc[j];
          }
        }
      }
      ss = warp_sum(ss);
      const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
      if (lane == 0) scratch[warp] = ss;
      __syncthreads();
      float t = lane < (kTpThreads >> 5) ? scratch[lane] : 0.f;
      t = warp_sum(t);
      __syncthreads();
      const float inv = rsqrtf(t / static_cast<float>(hidden) + eps);
      const long long hoff = h_offset + static_cast<long long>(row) * hidden * 2;
#pragma unroll
      for (int i = 0; i < kTpMaxVec; ++i) {
        const int v = threadIdx.x + i * kTpThreads;
        if (v < nvec) {
          float g[8], o[8];
          unpack8(*reinterpret_cast<const uint4*>(w + v * 8), g);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * inv * g[j];
          const uint4 packed = pack8(o);
          if (c.mc_buf != nullptr) {
            multimem_st_bf16x8(const_cast<char*>(static_cast<const char*>(c.mc_buf)) + hoff + v * 16, packed);
          } else {
            for (int r = 0; r < c.world; ++r)
              st_relaxed_sys_v4(const_cast<char*>(static_cast<const char*>(c.peer_buf[r])) + hoff + v * 16, packed);
          }
        }
      }
    }
  }
  // second barrier: my rows are on every rank / every rank's rows are here. With defer_wait the second half is
  // left to the kernel that reads the activation (a GEMM waits for the peers' flags in its TMA producer, see
  // gemm_wait_rows): this kernel ends as soon as its own rows are out.
  __shared__ int last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    last = atomicAdd(c.epoch + 2, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (last && threadIdx.x < c.world) {
    c.epoch[2] = 0;
    if (defer_wait && threadIdx.x == 0) c.epoch[kPullTargetWord] = epoch;
    __threadfence_system();
    st_release_sys(c.peer_flags[threadIdx.x] + kPullDoneChannel * kMaxRanks + c.rank, epoch);
  }
  if (!defer_wait && threadIdx.x < c.world) {
    const uint32_t* f = c.peer_flags[c.rank] + kPullDoneChannel * kMaxRanks + threadIdx.x;
    const unsigned long long t0 = global_timer_ns();
    const unsigned long long limit = static_cast<unsigned long long>(c.spin_limit) * 1000ull;
    for (;;) {
      if (static_cast<int32_t>(ld_acquire_sys(f) - epoch) >= 0) break;
      if (global_timer_ns() - t0 > limit) {
        report_status(c.status, kTpKernelId, kPeerFlagTimeout);
        break;
      }
      __nanosleep(20);
    }
  }
  tp_finish(c);
}

struct ArgSlot {
  float v;
  int i;
};

// slots: symmetric [world][rows] ArgSlot array; each rank writes its local best of every row into slot
// [rank][row] of every peer, then all ranks pick the same winner. The grid is capped at what can be
// resident at once (every CTA waits for the peers before it picks) and walks the rows with its stride.
__global__ void __launch_bounds__(1024)
tp_argmax_kernel(const TpComm c, long long slots_offset, const __nv_bfloat16* __restrict__ logits, long long ld,
                 int local_vocab, int valid_vocab, int vocab_start, long long* __restrict__ out, int rows) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(c.epoch);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool vec_ok = (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* lr = logits + static_cast<size_t>(row) * ld;
    float bv = -CUDART_INF_F;
    int bi = 0x7fffffff;
    const int n = valid_vocab < local_vocab ? valid_vocab : local_vocab;
    // eight logits per 16-byte load where the rows allow it (a thread meets its ids in ascending order, so
    // "greater than" keeps the lowest id among equals)
    const int nvec = vec_ok ? n / 8 : 0;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 raw = *reinterpret_cast<const uint4*>(lr + v * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        if (f.x > bv) { bv = f.x; bi = v * 8 + 2 * j; }
        if (f.y > bv) { bv = f.y; bi = v * 8 + 2 * j + 1; }
      }
    }
    for (int i = nvec * 8 + threadIdx.x; i < n; i += blockDim.x) {
      const float x = __bfloat162float(lr[i]);
      if (x > bv || (x == bv && i < bi)) { bv = x; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
      bv = lane < (blockDim.x >> 5) ? sv[lane] : -CUDART_INF_F;
      bi = lane < (blockDim.x >> 5) ? si[lane] : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (lane < c.world) {
        // push (value, global id) into slot [my rank][row] on peer `lane`
        ArgSlot* dst = reinterpret_cast<ArgSlot*>(const_cast<char*>(static_cast<const char*>(c.peer_buf[lane])) +
                                                  slots_offset) + static_cast<size_t>(c.rank) * rows + row;
        const int gi = bi == 0x7fffffff ? -1 : bi + vocab_start;
        asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(bv)), "r"(gi)
                     : "memory");
      }
    }
    __syncthreads();
  }
  // one flag per kernel: raised by whichever CTA finishes last, after a grid-wide ticket says every row
  // has been pushed
  __shared__ int last;
  if (threadIdx.x < 32 && threadIdx.x < c.world) __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    last = atomicAdd(c.epoch + 2, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (last && threadIdx.x < c.world) {
    c.epoch[2] = 0;
    __threadfence_system();
    st_release_sys(c.peer_flags[threadIdx.x] + 1 * kMaxRanks + c.rank, epoch);
  }
  // wait for every rank's pushes
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    const uint32_t* f = c.peer_flags[c.rank] + 1 * kMaxRanks + threadIdx.x;
    bool seen = false;
    const unsigned long long t0 = global_timer_ns();
    const unsigned long long limit = static_cast<unsigned long long>(c.spin_limit) * 1000ull;
    for (;;) {
      if (static_cast<int32_t>(ld_acquire_sys(f) - epoch) >= 0) { seen = true; break; }
      if (global_timer_ns() - t0 > limit) break;
      __nanosleep(20);
    }
    if (!seen) { report_status(c.status, kTpKernelId, kPeerFlagTimeout); ok_flag = 0; }
  }
  __syncthreads();
  const ArgSlot* mine = reinterpret_cast<const ArgSlot*>(static_cast<const char*>(c.peer_buf[c.rank]) + slots_offset);
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < rows; row += gridDim.x * blockDim.x) {
    long long pick = 0;
    if (ok_flag) {
      float best = -CUDART_INF_F;
      int id = 0x7fffffff;
      for (int r = 0; r < c.world; ++r) {
        const volatile uint32_t* raw = reinterpret_cast<const volatile uint32_t*>(mine + static_cast<size_t>(r) * rows + row);
        const float v = __uint_as_float(raw[0]);
        const int i = static_cast<int>(raw[1]);
        if (i >= 0 && (v > best || (v == best && i < id))) { best = v; id = i; }
      }
      pick = id == 0x7fffffff ? 0 : id;
    }
    out[row] = pick;
  }
  tp_finish(c);
}

// All-gather along columns: every rank owns `local_cols` columns of a [rows, total_cols] matrix
// (its LM-head logit shard) and pushes them into that position of the matrix on every rank:
// one multimem.st per 16 bytes when the buffer has a multicast mapping (the switch replicates the
// store), else one peer store per rank. The last CTA to finish raises this rank's flag; every CTA
// then waits until all ranks have raised theirs, so when the kernel ends the full matrix is local.
// The destination lives in a symmetric buffer of its own (base pointers in c.peer_buf / c.mc_buf).
__global__ void __launch_bounds__(kTpThreads, 4)
tp_allgather_cols_kernel(const TpComm c, const __nv_bfloat16* __restrict__ src, long long ld, int local_cols,
                         long long total_cols, int rows) {
  grid_dep_launch();
  grid_dep_wait();
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(c.epoch);
  const int vec_per_row = local_cols >> 3;
  const long long total = static_cast<long long>(rows) * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / vec_per_row;
    const int v = static_cast<int>(i - row * vec_per_row);
    const uint4 val = *reinterpret_cast<const uint4*>(src + row * ld + v * 8);
    const long long off = (row * total_cols + static_cast<long long>(c.rank) * local_cols + v * 8) * 2;
    if (c.mc_buf != nullptr) {
      multimem_st_bf16x8(const_cast<char*>(static_cast<const char*>(c.mc_buf)) + off, val);
    } else {
      for (int r = 0; r < c.world; ++r)
        st_relaxed_sys_v4(const_cast<char*>(static_cast<const char*>(c.peer_buf[r])) + off, val);
    }
  }
  __shared__ int last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    last = atomicAdd(c.epoch + 2, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (last && threadIdx.x < c.world) {
    c.epoch[2] = 0;
    st_release_sys(c.peer_flags[threadIdx.x] + 1 * kMaxRanks + c.rank, epoch);
  }
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    const uint32_t* f = c.peer_flags[c.rank] + 1 * kMaxRanks + threadIdx.x;
    bool seen = false;
    const unsigned long long t0 = global_timer_ns();
    const unsigned long long limit = static_cast<unsigned long long>(c.spin_limit) * 1000ull;
    for (;;) {
      if (static_cast<int32_t>(ld_acquire_sys(f) - epoch) >= 0) { seen = true; break; }
      if (global_timer_ns() - t0 > limit) break;
      __nanosleep(20);
    }
    if (!seen) { report_status(c.status, kTpKernelId, kPeerFlagTimeout); ok_flag = 0; }
  }
  tp_finish(c);
}

}  // namespace xv

using namespace xv;

static int fill_comm(TpComm* c, const void* const* peer_bufs, void* const* peer_flags, const void* mc_buf,
                     void* epoch, int rank, int world, unsigned spin_limit, int* status) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return XV_ERR_SHAPE;
  for (int r = 0; r < kMaxRanks; ++r) {
    c->peer_buf[r] = r < world ? peer_bufs[r] : nullptr;
    c->peer_flags[r] = r < world ? static_cast<uint32_t*>(peer_flags[r]) : nullptr;
  }
  c->mc_buf = mc_buf;
  c->epoch = static_cast<uint32_t*>(epoch);
  c->rank = rank;
  c->world = world;
  c->spin_limit = spin_limit;
  c->status = status;
  return 0;
}

// How many CTAs of `kernel` can be resident on the current device at once (0 on error). Kernels whose CTAs
// wait for one another must not be launched with more; the figure comes from the occupancy calculator and
// the device's SM count, cached per device and kernel.
template <typename K>
static int resident_ctas(K kernel, int threads, int slot) {
  constexpr int kMaxDev = 64;
  static int cache[4][kMaxDev] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return 0;
  if (cache[slot][dev] > 0) return cache[slot][dev];
  int per_sm = 0, sms = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  cache[slot][dev] = per_sm * sms;
  return cache[slot][dev];
}

extern "C" {

// peer_bufs / peer_flags: HOST arrays of `world` device pointers (as mapped on this rank).
// epoch: 4 uint32 words of local device memory, zero-initialised except epoch[0] = 1.
int xv_tp_reduce_norm(const void* const* peer_bufs, void* const* peer_flags, const void* mc_buf, void* epoch,
                      int rank, int world, long long buf_offset, const void* residual_in, void* residual_out,
                      const void* w, void* y, int rows, int hidden, float eps, int mode, unsigned spin_limit,
                      int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden % 8 || hidden > kTpThreads * kTpMaxVec * 8 || (buf_offset & 15)) return XV_ERR_SHAPE;
  TpComm c;
  int rc = fill_comm(&c, peer_bufs, peer_flags, mc_buf, epoch, rank, world, spin_limit, status);
  if (rc) return rc;
  const int cap = resident_ctas(tp_reduce_norm_kernel, kTpThreads, 0);
  if (cap < 1) return XV_ERR_LAUNCH;
  int grid = rows < cap ? rows : cap;
  launch_pdl(tp_reduce_norm_kernel, dim3(grid), dim3(kTpThreads), 0, stream, 
      c, buf_offset, static_cast<const __nv_bfloat16*>(residual_in), static_cast<__nv_bfloat16*>(residual_out),
      static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), rows, hidden, eps, mode);
  return cudaGetLastError() == cudaSuccess ? 0 : XV_ERR_LAUNCH;
}

// Row-sharded reduction point: partial at `buf_offset`, normalised activations broadcast to
// `h_offset` (both byte offsets inside the symmetric buffer). `residual` holds this rank's rows
// of the residual stream (rows rank, rank + world, ...); has_residual == 0 starts the stream.
static int reduce_norm_sharded_impl(const void* const* peer_bufs, void* const* peer_flags, const void* mc_buf,
                                    void* epoch, int rank, int world, long long buf_offset, long long h_offset,
                                    int has_residual, void* residual, const void* w, int rows, int hidden, float eps,
                                    unsigned spin_limit, int* status, cudaStream_t stream, int defer_wait) {
  if (rows <= 0) return 0;
  if (hidden % 8 || hidden > kTpThreads * kTpMaxVec * 8 || (buf_offset & 15) || (h_offset & 15)) return XV_ERR_SHAPE;
  TpComm c;
  int rc = fill_comm(&c, peer_bufs, peer_flags, mc_buf, epoch, rank, world, spin_limit, status);
  if (rc) return rc;
  const int cap = resident_ctas(tp_reduce_norm_sharded_kernel, kTpThreads, 1);
  if (cap < 1) return XV_ERR_LAUNCH;
  int mine = (rows + world - 1) / world;
  int grid = mine < cap ? mine : cap;     // every CTA waits at the end: keep the grid resident
  if (grid < 1) grid = 1;
  launch_pdl(tp_reduce_norm_sharded_kernel, dim3(grid), dim3(kTpThreads), 0, stream, 
      c, buf_offset, h_offset, has_residual, static_cast<__nv_bfloat16*>(residual),
      static_cast<const __nv_bfloat16*>(w), rows, hidden, eps, defer_wait);
  return cudaGetLastError() == cudaSuccess ? 0 : XV_ERR_LAUNCH;
}

int xv_tp_reduce_norm_sharded(const void* const* peer_bufs, void* const* peer_flags, const void* mc_buf, void* epoch,
                              int rank, int world, long long buf_offset, long long h_offset, int has_residual,
                              void* residual, const void* w, int rows, int hidden, float eps, unsigned spin_limit,
                              int* status, cudaStream_t stream) {
  return reduce_norm_sharded_impl(peer_bufs, peer_flags, mc_buf, epoch, rank, world, buf_offset, h_offset,
                                  has_residual, residual, w, rows, hidden, eps, spin_limit, status, stream, 0);
}

// Same, but the kernel ends once its own rows are broadcast: the caller must make the next kernel that reads the
// activation wait for the other ranks' rows (xv_gemm_wait_for_epoch before the GEMM that consumes it).
int xv_tp_reduce_norm_sharded_nowait(const void* const* peer_bufs, void* const* peer_flags, const void* mc_buf,
                                     void* epoch, int rank, int world, long long buf_offset, long long h_offset,
                                     int has_residual, void* residual, const void* w, int rows, int hidden,
                                     float eps, unsigned spin_limit, int* status, cudaStream_t stream) {
  return reduce_norm_sharded_impl(peer_bufs, peer_flags, mc_buf, epoch, rank, world, buf_offset, h_offset,
                                  has_residual, residual, w, rows, hidden, eps, spin_limit, status, stream, 1);
}
int xv_tp_pull_done_word(void) { return kPullDoneChannel * kMaxRanks; }
int xv_tp_pull_target_word(void) { return kPullTargetWord; }

int xv_tp_argmax(const void* const* peer_bufs, void* const* peer_flags, void* epoch, int rank, int world,
                 long long slots_offset, const void* logits, long long ld, int local_vocab, int valid_vocab,
                 int vocab_start, long long* out, int rows, unsigned spin_limit, int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  TpComm c;
  int rc = fill_comm(&c, peer_bufs, peer_flags, nullptr, epoch, rank, world, spin_limit, status);
  if (rc) return rc;
  const int cap = resident_ctas(tp_argmax_kernel, 1024, 2);
  if (cap < 1) return XV_ERR_LAUNCH;
  launch_pdl(tp_argmax_kernel, dim3(rows < cap ? rows : cap), dim3(1024), 0, stream, c, slots_offset, static_cast<const __nv_bfloat16*>(logits), ld,
                                              local_vocab, valid_vocab, vocab_start, out, rows);
  return cudaGetLastError() == cudaSuccess ? 0 : XV_ERR_LAUNCH;
}

// Column all-gather into the symmetric matrix whose per-rank base pointers are `peer_bufs`
// (`mc_buf`: its multicast mapping or null). src: this rank's [rows, local_cols] shard with row
// stride ld; the gathered matrix is [rows, total_cols] with this rank's shard at column rank * local_cols.
int xv_tp_allgather_cols(const void* const* peer_bufs, void* const* peer_flags, const void* mc_buf, void* epoch,
                         int rank, int world, const void* src, long long ld, int local_cols, long long total_cols,
                         int rows, unsigned spin_limit, int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (local_cols % 8 || ld % 8 || total_cols % 8 || static_cast<long long>(local_cols) * world > total_cols ||
      (reinterpret_cast<uintptr_t>(src) & 15))
    return XV_ERR_SHAPE;
  TpComm c;
  int rc = fill_comm(&c, peer_bufs, peer_flags, mc_buf, epoch, rank, world, spin_limit, status);
  if (rc) return rc;
  const long long vecs = static_cast<long long>(rows) * (local_cols / 8);
  long long want = (vecs + kTpThreads - 1) / kTpThreads;
  const int cap = resident_ctas(tp_allgather_cols_kernel, kTpThreads, 3);
  if (cap < 1) return XV_ERR_LAUNCH;
  const int grid = static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));   // every CTA waits: stay resident
  launch_pdl(tp_allgather_cols_kernel, dim3(grid), dim3(kTpThreads), 0, stream, c, static_cast<const __nv_bfloat16*>(src), ld, local_cols,
                                                            total_cols, rows);
  return cudaGetLastError() == cudaSuccess ? 0 : XV_ERR_LAUNCH;
}

}  // extern "C"
