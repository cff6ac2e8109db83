// bf16 GEMM for sm_100a on the 5th-generation tensor cores: Y[M,N] = X[M,K] * W[N,K]^T.
//
// Structure of one CTA (192 threads):
//   warp 0      - TMA producer: cp.async.bulk.tensor 2-D tile loads of both operands into a
//                 ring of shared-memory stages (128-byte swizzle), completion on mbarriers.
//   warp 1      - allocates TMEM and issues tcgen05.mma (one elected thread); accumulator
//                 D[128 x BN] stays in tensor memory for the whole K loop.
//   warps 2..5  - epilogue: tcgen05.ld the accumulator (each warp owns 32 TMEM lanes),
//                 convert and store.
//
// Two orientations share the kernel. "Normal" puts tokens on the MMA M axis (A = X) and
// output features on N (B = W); it is used when M is large (prefill). "Swapped" puts output
// features on M (A = W) and tokens on N (B = X, BN = tokens rounded up to 16), so a decode
// step with a handful of tokens still issues full 128-row MMAs and streams each weight byte
// exactly once; the epilogue writes the transposed tile. Split-K (grid.z) spreads the K loop
// over more CTAs when there are too few output tiles to fill 148 SMs; partial sums go to an
// fp32 workspace that a second small kernel reduces.
//
// The reference calls cuBLAS through torch.nn.functional.linear for all of these
// (reference: src/compute/layers/linear.py:87,148,268,307).

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "tp_device.cuh"
#include "xv_cuda.h"

namespace xv {

constexpr int kBM = 128;          // MMA M (rows of operand A per CTA)
constexpr int kBK = 64;           // K elements per stage = one 128-byte swizzle row
constexpr int kUmmaK = 16;        // K per tcgen05.mma for 16-bit inputs
constexpr int kGemmThreads = 192;
constexpr int kMaxStages = 8;
constexpr int kGemmKernelId = 1;

struct GemmParams {
  int rows_a;        // valid rows of operand A (M axis of the MMA)
  int rows_b;        // valid rows of operand B (N axis of the MMA)
  int k;             // reduction length
  int bn;            // MMA N = rows of B per CTA (multiple of 16, <= 256)
  int stages;
  int k_blocks_per_split;
  int tiles_a, tiles_b, splits;
  int a_fastest;     // work order: 1 = consecutive work items walk the A tiles, 0 = the B tiles
  int transposed;    // 1: out[(b_row) * ldc + a_row], 0: out[a_row * ldc + b_row]
  int out_fp32;      // 1: fp32 partials at out + split * split_stride, 0: bf16
  int act;           // 1: SiLU-mul epilogue. Operand rows of the weight matrix come in groups of 16 =
                     //    [8 gate rows | 8 up rows]; output has half as many features (bf16 only)
  long long ldc;
  long long split_stride;   // elements between split-K partial planes
  void* out;
  int* status;
  uint32_t idesc;
  uint32_t tmem_cols;       // total allocation (two accumulators)
  uint32_t acc_stride;      // column offset of the second accumulator
};

struct WorkItem {
  int tile_a, tile_b, split;
};

__device__ __forceinline__ WorkItem decode_work(const GemmParams& p, int w) {
  WorkItem it;
  const int tiles = p.tiles_a * p.tiles_b;
  it.split = w / tiles;
  const int r = w - it.split * tiles;
  if (p.a_fastest) {
    it.tile_b = r / p.tiles_a;
    it.tile_a = r - it.tile_b * p.tiles_a;
  } else {
    it.tile_a = r / p.tiles_b;
    it.tile_b = r - it.tile_a * p.tiles_b;
  }
  return it;
}

// Persistent kernel: every CTA walks work items (output tile x K split) with stride gridDim.x.
// The shared-memory stage ring and its phases run on across work items, and the accumulator
// is double buffered in TMEM, so the epilogue of one tile overlaps the main loop of the next.
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmParams p, const __grid_constant__ TpTail tail) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  grid_dep_launch();           // the next kernel of the stream may start its prologue (see launch.cuh)
  // Dynamic shared memory is only guaranteed 16-byte alignment; the swizzled tiles need 1024.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const uint32_t a_bytes = kBM * kBK * 2;
  const uint32_t b_bytes = static_cast<uint32_t>(p.bn) * kBK * 2;
  const uint32_t stage_bytes = a_bytes + b_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(p.stages) * stage_bytes);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* acc_full = empty_bar + kMaxStages;     // [2] accumulator ready for the epilogue
  uint64_t* acc_empty = acc_full + 2;              // [2] accumulator drained, MMA may overwrite
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_work = p.tiles_a * p.tiles_b * p.splits;
  const int total_kb = (p.k + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);      // one arrival per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Everything up to here touched only this CTA's shared and tensor memory. The producer thread first
  // starts the weight stream, which no earlier kernel writes; every other thread waits now for the
  // previous kernel of the stream (its outputs are this kernel's activations, and this kernel's
  // outputs may overwrite buffers it still reads).
  if (threadIdx.x != 0) grid_dep_wait();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      // In the swapped orientation operand A is the weight matrix, streamed once; B (the
      // activations) is re-read by every CTA. Hints follow that.
      const uint64_t hint_a = p.transposed ? l2_policy_evict_first() : l2_policy_evict_normal();
      const uint64_t hint_b = p.transposed ? l2_policy_evict_last() : l2_policy_evict_normal();
      // Weight tiles of the first stages of the first work item go out before the wait.
      uint32_t pre = 0;
      if (static_cast<int>(blockIdx.x) < total_work) {
        const WorkItem wi = decode_work(p, blockIdx.x);
        const int kb_begin = wi.split * p.k_blocks_per_split;
        const int kb_end = min(kb_begin + p.k_blocks_per_split, total_kb);
        pre = static_cast<uint32_t>(min(kb_end - kb_begin, p.stages));
        for (uint32_t i = 0; i < pre; ++i) {
          uint8_t* sa = smem + static_cast<size_t>(i) * stage_bytes;
          mbar_expect_tx(&full_bar[i], stage_bytes);
          if (p.transposed)
            tma_load_2d(sa, &map_a, &full_bar[i], (kb_begin + i) * kBK, wi.tile_a * kBM, hint_a);
          else
            tma_load_2d(sa + a_bytes, &map_b, &full_bar[i], (kb_begin + i) * kBK, wi.tile_b * p.bn, hint_b);
        }
      }
      grid_dep_wait();
      uint32_t it = 0;                   // K blocks issued so far by this CTA, across work items
      for (int w = blockIdx.x; w < total_work && !*abort_flag; w += gridDim.x) {
        const WorkItem wi = decode_work(p, w);
        const int kb_begin = wi.split * p.k_blocks_per_split;
        const int kb_end = min(kb_begin + p.k_blocks_per_split, total_kb);
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const uint32_t s = it % p.stages;
          const uint32_t round = it / p.stages;
          if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1)) {
            report_status(p.status, kGemmKernelId, kWaitEmptyTimeout);
            *abort_flag = 1;
            break;
          }
          uint8_t* sa = smem + static_cast<size_t>(s) * stage_bytes;
          const bool weights_out = it < pre;      // expect_tx and the weight tile were issued above
          if (!weights_out) mbar_expect_tx(&full_bar[s], stage_bytes);
          if (!(weights_out && p.transposed))
            tma_load_2d(sa, &map_a, &full_bar[s], kb * kBK, wi.tile_a * kBM, hint_a);
          if (!(weights_out && !p.transposed))
            tma_load_2d(sa + a_bytes, &map_b, &full_bar[s], kb * kBK, wi.tile_b * p.bn, hint_b);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t it = 0, t = 0;
      for (int w = blockIdx.x; w < total_work && !*abort_flag; w += gridDim.x, ++t) {
        const WorkItem wi = decode_work(p, w);
        const int kb_begin = wi.split * p.k_blocks_per_split;
        const int kb_end = min(kb_begin + p.k_blocks_per_split, total_kb);
        const uint32_t buf = t & 1, use = t >> 1;
        if (use > 0 && !mbar_wait(&acc_empty[buf], (use - 1) & 1)) {
          report_status(p.status, kGemmKernelId, kWaitAccumTimeout);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * p.acc_stride;
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const uint32_t s = it % p.stages;
          const uint32_t round = it / p.stages;
          if (!mbar_wait(&full_bar[s], round & 1)) {
            report_status(p.status, kGemmKernelId, kWaitFullTimeout);
            *abort_flag = 1;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + static_cast<size_t>(s) * stage_bytes);
          const uint32_t sb = sa + a_bytes;
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            const uint64_t da = umma_desc_sw128(sa + kk * kUmmaK * 2);
            const uint64_t db = umma_desc_sw128(sb + kk * kUmmaK * 2);
            umma_bf16(d_tmem, da, db, p.idesc, (kb > kb_begin || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);   // stage is free once these MMAs have read it
        }
        umma_commit(&acc_full[buf]);     // accumulator complete
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;                       // TMEM lane quarter this warp may read
    uint32_t t = 0;
    for (int w = blockIdx.x; w < total_work; w += gridDim.x, ++t) {
      const WorkItem wi = decode_work(p, w);
      const uint32_t buf = t & 1, use = t >> 1;
      bool ok = mbar_wait(&acc_full[buf], use & 1);
      if (!ok) {
        report_status(p.status, kGemmKernelId, kWaitAccumTimeout);
        *abort_flag = 1;
      }
      tc_fence_after_sync();
      // warp-uniform: the aligned TMEM loads below must be executed by all 32 lanes or none
      ok = __all_sync(0xffffffffu, ok && (*abort_flag == 0));
      if (!ok) break;
      const int a_row = wi.tile_a * kBM + quarter * 32 + lane;
      const uint32_t lane_addr = tmem_base + buf * p.acc_stride + (static_cast<uint32_t>(quarter * 32) << 16);
      const int b0 = wi.tile_b * p.bn;
      for (int c = 0; c < p.bn; c += 16) {
        uint32_t r[16];
        tmem_ld16(lane_addr + static_cast<uint32_t>(c), r);
        tmem_ld_wait();
        if (p.act && p.transposed) {
          // lanes are weight rows laid out [8 gate | 8 up | 8 gate | 8 up]: lane l pairs with l ^ 8
          __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out);
          const int out_col = (a_row >> 4) * 8 + (a_row & 7);
          const bool writer = (lane & 8) == 0 && a_row < p.rows_a;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float v = __uint_as_float(r[j]);
            const float up = __shfl_xor_sync(0xffffffffu, v, 8);
            const int b_row = b0 + c + j;
            if (writer && b_row < p.rows_b)
              o[static_cast<size_t>(b_row) * p.ldc + out_col] = __float2bfloat16(v / (1.f + __expf(-v)) * up);
          }
        } else if (p.act) {
          // this thread's 16 columns are [8 gate | 8 up] of one feature group
          if (a_row < p.rows_a) {
            const int col = b0 + c;
            if (col + 16 <= p.rows_b) {
              float ov[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float gte = __uint_as_float(r[j]);
                ov[j] = gte / (1.f + __expf(-gte)) * __uint_as_float(r[8 + j]);
              }
              uint4 v0;
              v0.x = pack_bf16(ov[0], ov[1]);
              v0.y = pack_bf16(ov[2], ov[3]);
              v0.z = pack_bf16(ov[4], ov[5]);
              v0.w = pack_bf16(ov[6], ov[7]);
              *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(a_row) * p.ldc +
                                        (col >> 1)) = v0;
            }
          }
        } else if (p.transposed) {
          // lanes hold consecutive output columns (a_row); tokens run along the registers
          if (a_row < p.rows_a) {
            if (p.out_fp32) {
              float* o = static_cast<float*>(p.out) + static_cast<size_t>(wi.split) * p.split_stride;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int b_row = b0 + c + j;
                if (b_row < p.rows_b) o[static_cast<size_t>(b_row) * p.ldc + a_row] = __uint_as_float(r[j]);
              }
            } else {
              __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int b_row = b0 + c + j;
                if (b_row < p.rows_b)
                  o[static_cast<size_t>(b_row) * p.ldc + a_row] = __float2bfloat16(__uint_as_float(r[j]));
              }
            }
          }
        } else if (a_row < p.rows_a) {
          const int col = b0 + c;
          if (p.out_fp32) {
            float* o = static_cast<float*>(p.out) + static_cast<size_t>(wi.split) * p.split_stride +
                       static_cast<size_t>(a_row) * p.ldc + col;
            if (col + 16 <= p.rows_b && (p.ldc & 3) == 0) {
#pragma unroll
              for (int j = 0; j < 16; j += 4)
                *reinterpret_cast<float4*>(o + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                                __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            } else {
              for (int j = 0; j < 16; ++j)
                if (col + j < p.rows_b) o[j] = __uint_as_float(r[j]);
            }
          } else {
            __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(a_row) * p.ldc + col;
            if (col + 16 <= p.rows_b && (p.ldc & 7) == 0) {
              uint4 v0, v1;
              v0.x = pack_bf16(__uint_as_float(r[0]), __uint_as_float(r[1]));
              v0.y = pack_bf16(__uint_as_float(r[2]), __uint_as_float(r[3]));
              v0.z = pack_bf16(__uint_as_float(r[4]), __uint_as_float(r[5]));
              v0.w = pack_bf16(__uint_as_float(r[6]), __uint_as_float(r[7]));
              v1.x = pack_bf16(__uint_as_float(r[8]), __uint_as_float(r[9]));
              v1.y = pack_bf16(__uint_as_float(r[10]), __uint_as_float(r[11]));
              v1.z = pack_bf16(__uint_as_float(r[12]), __uint_as_float(r[13]));
              v1.w = pack_bf16(__uint_as_float(r[14]), __uint_as_float(r[15]));
              *reinterpret_cast<uint4*>(o) = v0;
              *reinterpret_cast<uint4*>(o + 8) = v1;
            } else {
              for (int j = 0; j < 16; ++j)
                if (col + j < p.rows_b) o[j] = __float2bfloat16(__uint_as_float(r[j]));
            }
          }
        }
      }
      // this warp has drained its quarter of the accumulator
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }

  // ---------------- tensor-parallel tail: all-reduce + residual + RMSNorm in this kernel ----------------
  // The whole grid is resident (the host clamps it to the occupancy), so grid-wide barriers
  // are safe. Phase order: [fold split-K planes into the symmetric buffer] -> announce to
  // peers -> wait for peers -> every CTA reduces, adds the residual and normalises its rows.
  if (tail.enabled) {
    __shared__ float tail_scratch[32];
    bool ok = *abort_flag == 0;
    if (tail.splits > 1) {
      ok = grid_barrier(tail.grid_sync, kDefaultWaitNs) && ok;
      if (ok) {
        __nv_bfloat16* mine = reinterpret_cast<__nv_bfloat16*>(
            const_cast<char*>(static_cast<const char*>(tail.comm.peer_buf[tail.comm.rank])) + tail.buf_offset);
        const long long elems = static_cast<long long>(tail.rows) * tail.hidden;
        for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < elems;
             i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
          float4 acc = *reinterpret_cast<const float4*>(tail.partials + i);
          for (int sp = 1; sp < tail.splits; ++sp) {
            const float4 v = *reinterpret_cast<const float4*>(tail.partials + sp * tail.split_stride + i);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
          }
          uint2 o;
          o.x = pack_bf16(acc.x, acc.y);
          o.y = pack_bf16(acc.z, acc.w);
          *reinterpret_cast<uint2*>(mine + i) = o;
        }
      }
    }
    ok = grid_barrier(tail.grid_sync, kDefaultWaitNs) && ok;
    if (!ok) report_status(p.status, kGemmKernelId, kPeerFlagTimeout);
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(tail.comm.epoch);
    ok = tp_barrier(tail.comm, epoch, 0) && ok;
    if (ok)
      tp_reduce_rows<6>(tail.comm, tail.buf_offset, tail.residual_in, tail.residual_out, tail.norm_w, tail.y,
                        tail.rows, tail.hidden, tail.eps, tail.mode, tail_scratch);
    tp_finish(tail.comm);
  }
}

// ---- CTA-pair variant --------------------------------------------------------------------------------
// Two CTAs of a 2-wide cluster compute one 256 x 256 output tile with tcgen05.mma cta_group::2.
// Each CTA loads 128 rows of A and 128 rows of B per K block (32 KB instead of the 48 KB a lone
// CTA needs for its 128 x 256 tile), so the shared-memory fill traffic per FLOP drops by a third
// and six stages fit. CTA rank 0 issues the MMAs for the pair; each CTA drains its own 128
// accumulator rows. Used for the large-M (prefill) orientation.
constexpr int kPairStages = 6;
constexpr int kPairStageBytes = 2 * kBM * kBK * 2;   // A 16 KB + B 16 KB
constexpr int kPairSmem = kPairStages * kPairStageBytes + 1024 + 256;

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr uint32_t a_bytes = kBM * kBK * 2;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes);   // used in the leader
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* acc_full = empty_bar + kMaxStages;
  uint64_t* acc_empty = acc_full + 2;                                                       // used in the leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int total_work = p.tiles_a * p.tiles_b * p.splits;
  const int total_kb = (p.k + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&full_bar[s], 2);       // one arrive.expect_tx from each CTA's producer
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);      // four epilogue warps in each of the two CTAs
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      const uint64_t hint = l2_policy_evict_normal();
      uint32_t it = 0;
      for (int w = pair; w < total_work && !*abort_flag; w += num_pairs) {
        const WorkItem wi = decode_work(p, w);
        const int kb_begin = wi.split * p.k_blocks_per_split;
        const int kb_end = min(kb_begin + p.k_blocks_per_split, total_kb);
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const uint32_t s = it % kPairStages;
          const uint32_t round = it / kPairStages;
          if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1)) {
            report_status(p.status, kGemmKernelId, kWaitEmptyTimeout);
            *abort_flag = 1;
            break;
          }
          uint8_t* sa = smem + static_cast<size_t>(s) * kPairStageBytes;
          const uint32_t leader_full = map_to_cta(smem_u32(&full_bar[s]), 0);
          mbar_expect_tx_cluster(leader_full, kPairStageBytes);
          tma_load_2d_pair(sa, &map_a, leader_full, kb * kBK, wi.tile_a * 256 + static_cast<int>(rank) * kBM, hint);
          tma_load_2d_pair(sa + a_bytes, &map_b, leader_full, kb * kBK,
                           wi.tile_b * 256 + static_cast<int>(rank) * kBM, hint);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && rank == 0) {
      uint32_t it = 0, t = 0;
      for (int w = pair; w < total_work && !*abort_flag; w += num_pairs, ++t) {
        const WorkItem wi = decode_work(p, w);
        const int kb_begin = wi.split * p.k_blocks_per_split;
        const int kb_end = min(kb_begin + p.k_blocks_per_split, total_kb);
        const uint32_t buf = t & 1, use = t >> 1;
        if (use > 0 && !mbar_wait(&acc_empty[buf], (use - 1) & 1)) {
          report_status(p.status, kGemmKernelId, kWaitAccumTimeout);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * 256;
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const uint32_t s = it % kPairStages;
          const uint32_t round = it / kPairStages;
          if (!mbar_wait(&full_bar[s], round & 1)) {
            report_status(p.status, kGemmKernelId, kWaitFullTimeout);
            *abort_flag = 1;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + static_cast<size_t>(s) * kPairStageBytes);
          const uint32_t sb = sa + a_bytes;
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            umma_bf16_pair(d_tmem, umma_desc_sw128(sa + kk * kUmmaK * 2), umma_desc_sw128(sb + kk * kUmmaK * 2),
                           p.idesc, (kb > kb_begin || kk > 0) ? 1u : 0u);
          }
          // the stage is free in both CTAs once these MMAs have read it
          umma_commit_pair(map_to_cta(smem_u32(&empty_bar[s]), 0));
          umma_commit_pair(map_to_cta(smem_u32(&empty_bar[s]), 1));
        }
        umma_commit_pair(map_to_cta(smem_u32(&acc_full[buf]), 0));
        umma_commit_pair(map_to_cta(smem_u32(&acc_full[buf]), 1));
      }
    }
  } else {
    // ---------------- epilogue (both CTAs, own 128 accumulator rows) ----------------
    const int quarter = warp & 3;
    uint32_t t = 0;
    for (int w = pair; w < total_work; w += num_pairs, ++t) {
      const WorkItem wi = decode_work(p, w);
      const uint32_t buf = t & 1, use = t >> 1;
      bool ok = mbar_wait(&acc_full[buf], use & 1);
      if (!ok) {
        report_status(p.status, kGemmKernelId, kWaitAccumTimeout);
        *abort_flag = 1;
      }
      tc_fence_after_sync();
      ok = __all_sync(0xffffffffu, ok && (*abort_flag == 0));
      if (!ok) break;
      const int a_row = wi.tile_a * 256 + static_cast<int>(rank) * kBM + quarter * 32 + lane;
      const uint32_t lane_addr = tmem_base + buf * 256 + (static_cast<uint32_t>(quarter * 32) << 16);
      const int b0 = wi.tile_b * 256;
      for (int c = 0; c < 256; c += 16) {
        uint32_t r[16];
        tmem_ld16(lane_addr + static_cast<uint32_t>(c), r);
        tmem_ld_wait();
        const int col = b0 + c;
        if (a_row >= p.rows_a || col >= p.rows_b) continue;
        if (p.act) {
          if (col + 16 <= p.rows_b) {
            float ov[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float gte = __uint_as_float(r[j]);
              ov[j] = gte / (1.f + __expf(-gte)) * __uint_as_float(r[8 + j]);
            }
            uint4 v0;
            v0.x = pack_bf16(ov[0], ov[1]);
            v0.y = pack_bf16(ov[2], ov[3]);
            v0.z = pack_bf16(ov[4], ov[5]);
            v0.w = pack_bf16(ov[6], ov[7]);
            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(a_row) * p.ldc +
                                      (col >> 1)) = v0;
          }
        } else if (p.out_fp32) {
          float* o = static_cast<float*>(p.out) + static_cast<size_t>(wi.split) * p.split_stride +
                     static_cast<size_t>(a_row) * p.ldc + col;
          for (int j = 0; j < 16; ++j)
            if (col + j < p.rows_b) o[j] = __uint_as_float(r[j]);
        } else {
          __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(a_row) * p.ldc + col;
          if (col + 16 <= p.rows_b && (p.ldc & 7) == 0) {
            uint4 v0, v1;
            v0.x = pack_bf16(__uint_as_float(r[0]), __uint_as_float(r[1]));
            v0.y = pack_bf16(__uint_as_float(r[2]), __uint_as_float(r[3]));
            v0.z = pack_bf16(__uint_as_float(r[4]), __uint_as_float(r[5]));
            v0.w = pack_bf16(__uint_as_float(r[6]), __uint_as_float(r[7]));
            v1.x = pack_bf16(__uint_as_float(r[8]), __uint_as_float(r[9]));
            v1.y = pack_bf16(__uint_as_float(r[10]), __uint_as_float(r[11]));
            v1.z = pack_bf16(__uint_as_float(r[12]), __uint_as_float(r[13]));
            v1.w = pack_bf16(__uint_as_float(r[14]), __uint_as_float(r[15]));
            *reinterpret_cast<uint4*>(o) = v0;
            *reinterpret_cast<uint4*>(o + 8) = v1;
          } else {
            for (int j = 0; j < 16; ++j)
              if (col + j < p.rows_b) o[j] = __float2bfloat16(__uint_as_float(r[j]));
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
    }
  }

  // Both CTAs stay alive until the pair is done: the leader's MMAs read the peer's shared
  // memory and write the peer's tensor memory.
  tc_fence_before_sync();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// out[m, n] = sum_s partial[s, m, n], rounded to bf16.
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                     long long elems, int splits, long long split_stride) {
  grid_dep_launch();
  grid_dep_wait();
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i >= elems) return;
  if (i + 4 <= elems) {
    float4 acc = *reinterpret_cast<const float4*>(partial + i);
    for (int s = 1; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(partial + s * split_stride + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    uint2 o;
    o.x = pack_bf16(acc.x, acc.y);
    o.y = pack_bf16(acc.z, acc.w);
    *reinterpret_cast<uint2*>(out + i) = o;
  } else {
    for (long long j = i; j < elems; ++j) {
      float acc = 0.f;
      for (int s = 0; s < splits; ++s) acc += partial[s * split_stride + j];
      out[j] = __float2bfloat16(acc);
    }
  }
}

// ---- host side --------------------------------------------------------------------------------

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn get_encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  long long rows, k, ld;
  int box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && k == o.k && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h ^= static_cast<size_t>(k.rows) * 0x9E3779B97F4A7C15ULL + (h << 6) + (h >> 2);
    h ^= static_cast<size_t>(k.k) * 0xC2B2AE3D27D4EB4FULL + (h << 6) + (h >> 2);
    h ^= static_cast<size_t>(k.ld * 31 + k.box_rows) + (h << 6) + (h >> 2);
    return h;
  }
};

// Tensor maps depend only on (address, shape, box); weights never move and the caching
// allocator hands activations the same addresses step after step, so encodes are cached.
static int get_tensor_map(CUtensorMap* out, const void* ptr, long long rows, long long k, long long ld,
                          int box_rows) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{ptr, rows, k, ld, box_rows};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  EncodeFn enc = get_encode_fn();
  if (!enc) return XV_ERR_DRIVER;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return XV_ERR_TENSORMAP;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 65536) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

static int round_up(int x, int m) { return (x + m - 1) / m * m; }

static uint32_t pow2_cols(int n) {
  uint32_t c = 32;
  while (c < static_cast<uint32_t>(n)) c <<= 1;
  return c;
}

}  // namespace xv

using namespace xv;

static bool g_disable_pair = false;

extern "C" {

// Test hook: 1 forces the single-CTA kernel for every shape (A/B comparisons), 0 restores.
void xv_gemm_disable_pair(int disable) { g_disable_pair = disable != 0; }

// Chooses orientation, tile and split-K for a problem; fills *plan. Pure host arithmetic so
// callers (and CPU tests) can size the workspace before launching.
static int gemm_plan_impl(int m, int n, int k, int num_sms, XvGemmPlan* plan, bool allow_pair) {
  if (m <= 0 || n <= 0 || k <= 0 || (k % 8) != 0) return XV_ERR_SHAPE;
  if (num_sms <= 0) num_sms = 148;
  XvGemmPlan pl;
  std::memset(&pl, 0, sizeof(pl));
  const int total_kb = (k + kBK - 1) / kBK;
  if (m <= 256) {
    pl.swapped = 1;
    // above 128 tokens the batch is cut into two token tiles: twice as many (half-size) work
    // items balance better over 148 SMs and halve the per-stage activation bytes
    pl.tiles_b = m > 128 ? 2 : 1;
    pl.bn = round_up((m + pl.tiles_b - 1) / pl.tiles_b, 16);
    pl.tiles_a = (n + kBM - 1) / kBM;
  } else {
    pl.swapped = 0;
    pl.bn = n >= 256 ? 256 : round_up(n, 16);
    pl.tiles_a = (m + kBM - 1) / kBM;
    pl.tiles_b = (n + pl.bn - 1) / pl.bn;
  }
  const int tiles = pl.tiles_a * pl.tiles_b;
  const int stage_bytes = kBM * kBK * 2 + pl.bn * kBK * 2;
  // small-token tiles leave room for two resident CTAs per SM (more loads in flight while
  // another CTA drains its epilogue); big tiles take the whole SM
  const int smem_budget = (pl.swapped && pl.bn <= 128) ? 100 * 1024 : 200 * 1024;
  int stages = smem_budget / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) stages = 2;
  const int smem_bytes = stages * stage_bytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
  pl.ctas_per_sm = (smem_bytes <= 110 * 1024 && 2 * pow2_cols(pl.bn) <= 256) ? 2 : 1;
  // Split K when the output tiles alone cannot occupy the machine. Bounds: at least 4 K blocks
  // per split, at most 16 splits, and fp32 partials (written and read back once) no larger
  // than about a quarter of the weight bytes.
  const int slots = num_sms * pl.ctas_per_sm;
  int splits = 1;
  if (tiles < num_sms) {
    splits = slots / tiles;
    // partial planes cost splits * m * n * 4 bytes written and read back: allow them up to a quarter of
    // the weight bytes, or up to 16 MB in absolute terms (they stay in the 126 MB L2), whichever is more
    int by_traffic = k / (8 * m) > 1 ? k / (8 * m) : 1;
    const long long plane = static_cast<long long>(m) * n * 4;
    const int by_bytes = static_cast<int>((16ll << 20) / (plane > 0 ? plane : 1));
    if (by_bytes > by_traffic) by_traffic = by_bytes;
    if (splits > by_traffic) splits = by_traffic;
    while (splits > 1 && total_kb / splits < 4) --splits;
    static const int max_splits = [] {
      const char* e = std::getenv("XV_GEMM_MAX_SPLITS");      // experiment knob: cap on split-K
      return e ? std::atoi(e) : 16;
    }();
    if (splits > max_splits) splits = max_splits;
    if (splits > 16) splits = 16;
    if (splits < 1) splits = 1;
  }
  pl.k_blocks_per_split = (total_kb + splits - 1) / splits;
  pl.splits = (total_kb + pl.k_blocks_per_split - 1) / pl.k_blocks_per_split;
  if (stages > pl.k_blocks_per_split && pl.k_blocks_per_split >= 2) stages = pl.k_blocks_per_split;
  pl.stages = stages;
  pl.smem_bytes = stages * stage_bytes + 1024 + 256;
  pl.workspace_bytes = pl.splits > 1 ? static_cast<long long>(pl.splits) * m * n * 4 : 0;
  // CTA pairs (256 x 256 tiles, cta_group::2) instead of the plan above? Both kernels are persistent with one
  // tile per SM (pair of SMs), so time goes in whole waves, and a pair tile takes about 0.88 of the time of a
  // 128 x 256 tile (measured: 35 us against 39 us at K = 4096). Pairs win unless they need more waves
  // (M = 1100, N = 4096: 80 pair tiles on 74 pairs are two waves, 144 single tiles on 148 SMs one: measured 156
  // against 109 us). With fewer pair tiles than SM pairs they still win by 5-13 % (M = 384..832, N = 4096 or 6144)
  // as long as the single-CTA plan would not split K; where it does (M <= 512 with K = 12288), split-K is faster.
  if (!pl.swapped && allow_pair && n >= 256) {
    const int pair_tiles = ((m + 255) / 256) * ((n + 255) / 256);
    const int pair_waves = (pair_tiles + num_sms / 2 - 1) / (num_sms / 2);
    const int single_waves = (tiles + num_sms - 1) / num_sms;
    const bool enough = pair_tiles >= num_sms / 2 || (pl.splits == 1 && pair_tiles >= 24);
    if (enough && pair_waves * 0.88 <= single_waves) {
      pl.pair = 1;
      pl.bn = 256;
      pl.tiles_a = (m + 255) / 256;
      pl.tiles_b = (n + 255) / 256;
      pl.splits = 1;
      pl.k_blocks_per_split = total_kb;
      pl.stages = kPairStages;
      pl.smem_bytes = kPairSmem;
      pl.ctas_per_sm = 1;
      pl.workspace_bytes = 0;
    }
  }
  *plan = pl;
  return 0;
}

int xv_gemm_plan(int m, int n, int k, int num_sms, XvGemmPlan* plan) {
  return gemm_plan_impl(m, n, k, num_sms, plan, !g_disable_pair);
}

// Y[m,n] (bf16, row stride ldy) = X[m,k] (row stride ldx) * W[n,k]^T (row stride ldw).
// `workspace` must hold plan.workspace_bytes when the plan splits K. `status` may be null.
static int gemm_impl(const void* x, const void* w, void* y, int m, int n, int k, long long ldx, long long ldw,
                     long long ldy, void* workspace, long long workspace_bytes, int num_sms, int* status,
                     cudaStream_t stream, bool defer_reduce, int* splits_out, int act = 0,
                     const TpTail* tail_in = nullptr) {
  XvGemmPlan pl;
  // the fused tensor-parallel tail lives in the single-CTA kernel
  int rc = gemm_plan_impl(m, n, k, num_sms, &pl, tail_in == nullptr && !g_disable_pair);
  if (rc) return rc;
  if ((ldx % 8) || (ldw % 8) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return XV_ERR_ALIGN;
  if (pl.workspace_bytes > workspace_bytes || (pl.workspace_bytes && !workspace)) return XV_ERR_WORKSPACE;

  CUtensorMap map_a, map_b;
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  if (pl.pair) {
    if ((rc = get_tensor_map(&map_a, x, m, k, ldx, kBM))) return rc;
    if ((rc = get_tensor_map(&map_b, w, n, k, ldw, kBM))) return rc;
    p.rows_a = m;
    p.rows_b = n;
    p.transposed = 0;
  } else if (pl.swapped) {
    if ((rc = get_tensor_map(&map_a, w, n, k, ldw, kBM))) return rc;
    if ((rc = get_tensor_map(&map_b, x, m, k, ldx, pl.bn))) return rc;
    p.rows_a = n;
    p.rows_b = m;
    p.transposed = 1;
  } else {
    if ((rc = get_tensor_map(&map_a, x, m, k, ldx, kBM))) return rc;
    if ((rc = get_tensor_map(&map_b, w, n, k, ldw, pl.bn))) return rc;
    p.rows_a = m;
    p.rows_b = n;
    p.transposed = 0;
  }
  p.k = k;
  p.bn = pl.bn;
  p.stages = pl.stages;
  p.k_blocks_per_split = pl.k_blocks_per_split;
  p.status = status;
  p.idesc = umma_idesc_bf16(pl.pair ? 256 : kBM, pl.bn);
  p.acc_stride = pow2_cols(pl.bn);
  p.tmem_cols = 2 * p.acc_stride;
  p.tiles_a = pl.tiles_a;
  p.tiles_b = pl.tiles_b;
  p.splits = pl.splits;
  p.a_fastest = pl.swapped ? 0 : 1;
  if (pl.splits > 1) {
    p.out = workspace;
    p.out_fp32 = 1;
    p.ldc = n;
    p.split_stride = static_cast<long long>(m) * n;
  } else {
    p.out = y;
    p.out_fp32 = 0;
    p.ldc = ldy;
    p.split_stride = 0;
    p.act = act;
    if (act && ((n % 16) || (ldy % 8))) return XV_ERR_SHAPE;
  }

  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
    if (e != cudaSuccess) return XV_ERR_LAUNCH;
    attr_set = true;
  }
  if (pl.pair) {
    static bool pair_attr = false;
    if (!pair_attr) {
      if (cudaFuncSetAttribute(gemm_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024) !=
          cudaSuccess)
        return XV_ERR_LAUNCH;
      pair_attr = true;
    }
    const int pairs_avail = (num_sms > 0 ? num_sms : 148) / 2;
    const int work = pl.tiles_a * pl.tiles_b;
    const int pairs = work < pairs_avail ? work : pairs_avail;
    gemm_tcgen05_pair_kernel<<<2 * pairs, kGemmThreads, kPairSmem, stream>>>(map_a, map_b, p);
    return cudaGetLastError() == cudaSuccess ? 0 : XV_ERR_LAUNCH;
  }
  const int total_work = pl.tiles_a * pl.tiles_b * pl.splits;
  int slots = (num_sms > 0 ? num_sms : 148) * pl.ctas_per_sm;
  TpTail tail;
  std::memset(&tail, 0, sizeof(tail));
  int grid = total_work < slots ? total_work : slots;
  if (tail_in) {
    tail = *tail_in;
    tail.enabled = 1;
    tail.partials = static_cast<const float*>(workspace);
    tail.splits = pl.splits;
    tail.split_stride = p.split_stride;
    // grid-wide barriers need every CTA resident at once
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_tcgen05_kernel, kGemmThreads, pl.smem_bytes) !=
            cudaSuccess || per_sm < 1)
      return XV_ERR_LAUNCH;
    if (per_sm > pl.ctas_per_sm) per_sm = pl.ctas_per_sm;
    slots = (num_sms > 0 ? num_sms : 148) * per_sm;
    // all CTAs take part in the row phase, so launch the full resident grid even for few tiles
    grid = slots;
    if (grid > 4 * (tail.rows > total_work ? tail.rows : total_work)) grid = 4 * (tail.rows > total_work ? tail.rows : total_work);
    if (grid > slots) grid = slots;
    if (grid < 1) grid = 1;
  }
  launch_pdl(gemm_tcgen05_kernel, dim3(grid), dim3(kGemmThreads), pl.smem_bytes, stream, map_a, map_b, p, tail);
  if (cudaGetLastError() != cudaSuccess) return XV_ERR_LAUNCH;
  if (tail_in) return 0;
  if (splits_out) *splits_out = pl.splits;
  if (act && pl.splits > 1) return XV_ERR_UNSUPPORTED;   // callers check the plan first
  if (pl.splits > 1 && !defer_reduce) {
    const long long elems = static_cast<long long>(m) * n;
    if (ldy != n) return XV_ERR_SHAPE;   // split-K output must be dense
    const int threads = 256;
    const long long blocks = (elems / 4 + threads) / threads;
    launch_pdl(splitk_reduce_kernel, dim3(static_cast<unsigned>(blocks)), dim3(threads), 0, stream,
        static_cast<const float*>(workspace), static_cast<__nv_bfloat16*>(y), elems, pl.splits, p.split_stride);
    if (cudaGetLastError() != cudaSuccess) return XV_ERR_LAUNCH;
  }
  return 0;
}

int xv_gemm_bf16(const void* x, const void* w, void* y, int m, int n, int k, long long ldx, long long ldw,
                 long long ldy, void* workspace, long long workspace_bytes, int num_sms, int* status,
                 cudaStream_t stream) {
  return gemm_impl(x, w, y, m, n, k, ldx, ldw, ldy, workspace, workspace_bytes, num_sms, status, stream, false,
                   nullptr);
}

// RowParallel GEMM + all-reduce + residual add + RMSNorm as ONE kernel. The GEMM writes this
// rank's partial [m, n] into its symmetric buffer at `buf_offset` (peer_bufs[rank]); the same
// kernel then announces it to the peers, waits for theirs and finishes rows (see tp_fused.cu
// for the flag protocol and the buffer-reuse rule). grid_sync: 2 zero-initialised uint32.
int xv_gemm_bf16_tp(const void* x, const void* w, int m, int n, int k, long long ldx, long long ldw, void* workspace,
                    long long workspace_bytes, int num_sms, const void* const* peer_bufs, void* const* peer_flags,
                    const void* mc_buf, void* epoch, int rank, int world, long long buf_offset, void* grid_sync,
                    const void* residual_in, void* residual_out, const void* norm_w, void* y_out, float eps, int mode,
                    unsigned spin_us, int* status, cudaStream_t stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || (n % 8) || n > 192 * 6 * 8 || (buf_offset & 15))
    return XV_ERR_SHAPE;
  TpTail tail;
  std::memset(&tail, 0, sizeof(tail));
  for (int r = 0; r < kMaxRanks; ++r) {
    tail.comm.peer_buf[r] = r < world ? peer_bufs[r] : nullptr;
    tail.comm.peer_flags[r] = r < world ? static_cast<uint32_t*>(peer_flags[r]) : nullptr;
  }
  tail.comm.mc_buf = mc_buf;
  tail.comm.epoch = static_cast<uint32_t*>(epoch);
  tail.comm.rank = rank;
  tail.comm.world = world;
  tail.comm.spin_limit = spin_us;
  tail.comm.status = status;
  tail.buf_offset = buf_offset;
  tail.residual_in = static_cast<const __nv_bfloat16*>(residual_in);
  tail.residual_out = static_cast<__nv_bfloat16*>(residual_out);
  tail.norm_w = static_cast<const __nv_bfloat16*>(norm_w);
  tail.y = static_cast<__nv_bfloat16*>(y_out);
  tail.rows = m;
  tail.hidden = n;
  tail.eps = eps;
  tail.mode = mode;
  tail.grid_sync = static_cast<uint32_t*>(grid_sync);
  void* local = const_cast<char*>(static_cast<const char*>(peer_bufs[rank])) + buf_offset;
  return gemm_impl(x, w, local, m, n, k, ldx, ldw, n, workspace, workspace_bytes, num_sms, status, stream, true,
                   nullptr, 0, &tail);
}

// Y[m, n/2] = silu(gate) * up, with W's rows interleaved in groups of 16 = [8 gate | 8 up].
// Only for plans that do not split K (XV_ERR_UNSUPPORTED otherwise; see xv_gemm_plan).
int xv_gemm_bf16_silu_mul(const void* x, const void* w, void* y, int m, int n, int k, long long ldx, long long ldw,
                          long long ldy, int num_sms, int* status, cudaStream_t stream) {
  return gemm_impl(x, w, y, m, n, k, ldx, ldw, ldy, nullptr, 0, num_sms, status, stream, false, nullptr, 1);
}

// Same, but when the plan splits K the fp32 partial planes [splits][m][n] are left in
// `workspace` for the consumer kernel to sum (y is not written); *splits_out tells which.
int xv_gemm_bf16_defer(const void* x, const void* w, void* y, int m, int n, int k, long long ldx, long long ldw,
                       long long ldy, void* workspace, long long workspace_bytes, int num_sms, int* status,
                       cudaStream_t stream, int* splits_out) {
  return gemm_impl(x, w, y, m, n, k, ldx, ldw, ldy, workspace, workspace_bytes, num_sms, status, stream, true,
                   splits_out);
}

}  // extern "C"

// ---- allocation-free entry point ------------------------------------------------------------------
// Split-K scratch for xv_gemm_bf16_noalloc lives in the library image itself. Every GPU that
// loads this library carries these bytes until the process exits.
#define XV_NOALLOC_SCRATCH_BYTES (16ll << 20)
static __device__ __align__(256) unsigned char g_noalloc_scratch[XV_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void* g_scratch_ptr[kMaxDevices] = {nullptr};
int g_scratch_sms[kMaxDevices] = {0};
std::mutex g_scratch_mu;

// Resolves the device address of g_noalloc_scratch for the current device (once per device).
// In host code the symbol's name is only a handle; the address kernels may use comes from
// cudaGetSymbolAddress.
int noalloc_setup(int* dev_out, void** ptr_out, int* sms_out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return XV_ERR_DRIVER;
  std::lock_guard<std::mutex> g(g_scratch_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) return XV_ERR_DRIVER;
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return XV_ERR_DRIVER;
    g_scratch_ptr[dev] = p;
    g_scratch_sms[dev] = sms;
  }
  *dev_out = dev;
  *ptr_out = g_scratch_ptr[dev];
  *sms_out = g_scratch_sms[dev];
  return 0;
}
}  // namespace

extern "C" {

long long xv_gemm_noalloc_max_scratch_bytes(void) { return XV_NOALLOC_SCRATCH_BYTES; }

int xv_gemm_bf16_noalloc(const void* x, const void* w, void* y, int m, int n, int k, long long ldx, long long ldw,
                         long long ldy, int* status, cudaStream_t stream) {
  int dev = 0, sms = 0;
  void* scratch = nullptr;
  int rc = noalloc_setup(&dev, &scratch, &sms);
  if (rc) return rc;
  XvGemmPlan pl;
  if ((rc = xv_gemm_plan(m, n, k, sms, &pl))) return rc;
  if (pl.workspace_bytes > XV_NOALLOC_SCRATCH_BYTES) {
    std::fprintf(stderr,
                 "xv_gemm_bf16_noalloc: %d x %d x %d needs %lld bytes of split-K scratch, the built-in buffer "
                 "holds %lld; use xv_gemm_bf16 with a caller-provided workspace\n",
                 m, n, k, pl.workspace_bytes, static_cast<long long>(XV_NOALLOC_SCRATCH_BYTES));
    return XV_ERR_WORKSPACE;
  }
  return xv_gemm_bf16(x, w, y, m, n, k, ldx, ldw, ldy, scratch, XV_NOALLOC_SCRATCH_BYTES, sms, status, stream);
}

}  // extern "C"
