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
constexpr int kStagingBytes = 4 * 2048;   // per epilogue warp: transpose buffer, [32 tokens][32 features] bf16 or [16][32] fp32
constexpr int kTailMaxVec = 4;            // hidden <= 192 * 4 * 8 = 6144 in the tensor-parallel tail

struct GemmParams {
  int rows_a;        // valid rows of operand A (M axis of the MMA)
  int rows_b;        // valid rows of operand B (N axis of the MMA)
  int k;             // reduction length
  int bn;            // MMA N = rows of B per CTA (pair: per CTA pair); multiple of 16, <= 256
  int stages;
  int k_blocks_per_split;
  int tiles_a, tiles_b, splits;
  int a_fastest;     // work order: 1 = consecutive work items walk the A tiles, 0 = the B tiles
  int transposed;    // 1: out[(b_row) * ldc + a_row], 0: out[a_row * ldc + b_row]
  int out_fp32;      // 1: fp32 partials at out + split * split_stride, 0: bf16
  int act;           // 1: SiLU-mul epilogue. Operand rows of the weight matrix come in groups of 16 =
                     //    [8 gate rows | 8 up rows]; output has half as many features (bf16 only)
  int vec_ok;        // output rows may be written with 16-byte stores (alignment and row stride allow it)
  int fixup;         // swapped orientation with split-K: partial planes go to fix_planes, and the CTA that
                     // brings a tile's last partial sums them and runs the normal epilogue (no second kernel)
  float* fix_planes;        // [splits][rows_b][rows_a] fp32
  uint32_t* fix_counters;   // one per output tile, zero between launches
  unsigned long long* prof; // optional: 8 global-timer stamps per CTA (see xv_gemm_profile_buffer)
  int cluster_split;        // > 1: the K splits of a tile are the CTAs of one thread-block cluster, which sum their
                            // accumulators through distributed shared memory (swapped orientation, one tile per CTA)
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
  int r;
  if (p.cluster_split > 1) {          // consecutive CTAs (one cluster) share a tile
    it.split = w % p.cluster_split;
    r = w / p.cluster_split;
  } else {
    it.split = w / tiles;
    r = w - it.split * tiles;
  }
  if (p.a_fastest) {
    it.tile_b = r / p.tiles_a;
    it.tile_a = r - it.tile_b * p.tiles_a;
  } else {
    it.tile_a = r / p.tiles_b;
    it.tile_b = r - it.tile_a * p.tiles_b;
  }
  return it;
}

// Phase stamps of the single-CTA kernel, per CTA: 0 entry, 1 barriers + TMEM ready, 2 first tile load issued,
// 3 first stage landed, 4 last MMA of the first work item issued, 5 its accumulator complete, 6 epilogue of the
// CTA's last work item done, 7 exit.
__device__ __forceinline__ void gemm_prof(const GemmParams& p, int slot) {
  if (p.prof != nullptr) p.prof[blockIdx.x * 8 + slot] = global_timer_ns();
}

__device__ __forceinline__ uint4 pack8_regs(const uint32_t* r) {
  uint4 v;
  v.x = pack_bf16(__uint_as_float(r[0]), __uint_as_float(r[1]));
  v.y = pack_bf16(__uint_as_float(r[2]), __uint_as_float(r[3]));
  v.z = pack_bf16(__uint_as_float(r[4]), __uint_as_float(r[5]));
  v.w = pack_bf16(__uint_as_float(r[6]), __uint_as_float(r[7]));
  return v;
}

__device__ __forceinline__ float silu_mul_f(float gate, float up) { return gate / (1.f + __expf(-gate)) * up; }

// One thread's share of an accumulator tile in the normal orientation: 32 consecutive output columns
// (col .. col + 31) of output row `a_row`, in registers. Stores them as bf16, as an fp32 split-K plane,
// through the SiLU-mul epilogue, or into the reducing ranks' slots (tensor-parallel push).
__device__ __forceinline__ void store_row32(const GemmParams& p, const TpPush& push, int a_row, int col, int b_end,
                                            int split, const uint32_t (&r)[32]) {
  // b_end: first column that is not this tile's (the accumulator holds nothing valid from there on)
  if (a_row >= p.rows_a || col >= b_end) return;
  if (push.enabled) {
#pragma unroll
    for (int g = 0; g < 4; ++g)
      if (col + g * 8 < b_end) tp_push_store8(push, a_row, col + g * 8, split, pack8_regs(r + g * 8));
  } else if (p.act) {
    // 16 columns are [8 gate | 8 up] of one feature group -> 8 outputs
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(a_row) * p.ldc + (col >> 1);
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      if (col + g * 16 + 16 <= b_end) {
        float ov[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          ov[j] = silu_mul_f(__uint_as_float(r[g * 16 + j]), __uint_as_float(r[g * 16 + 8 + j]));
        uint4 v;
        v.x = pack_bf16(ov[0], ov[1]);
        v.y = pack_bf16(ov[2], ov[3]);
        v.z = pack_bf16(ov[4], ov[5]);
        v.w = pack_bf16(ov[6], ov[7]);
        *reinterpret_cast<uint4*>(o + g * 8) = v;
      }
    }
  } else if (p.out_fp32) {
    float* o = static_cast<float*>(p.out) + static_cast<size_t>(split) * p.split_stride +
               static_cast<size_t>(a_row) * p.ldc + col;
    if (col + 32 <= b_end && (p.ldc & 3) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(o + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                        __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col + j < b_end) o[j] = __uint_as_float(r[j]);
    }
  } else {
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(a_row) * p.ldc + col;
    if (col + 32 <= b_end && p.vec_ok) {
#pragma unroll
      for (int g = 0; g < 4; ++g) *reinterpret_cast<uint4*>(o + g * 8) = pack8_regs(r + g * 8);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col + j < b_end) o[j] = __float2bfloat16(__uint_as_float(r[j]));
    }
  }
}

// One warp's share of an accumulator tile in the swapped orientation: lane = output feature
// (a_row0 + lane), registers = 32 consecutive tokens (tok0 ..). The tile is turned through a
// per-warp shared-memory buffer so that global (or peer) memory sees 16-byte stores of eight
// consecutive features of one token instead of 2-byte stores.
__device__ __forceinline__ void store_swapped32(const GemmParams& p, const TpPush& push, uint8_t* stage_w, int lane,
                                                int a_row0, int tok0, int b_end, int split,
                                                const uint32_t (&r)[32]) {
  const int a_row = a_row0 + lane;
  if (p.out_fp32) {
    float* o = static_cast<float*>(p.out) + static_cast<size_t>(split) * p.split_stride;
    if ((p.ldc & 3) == 0 && a_row0 + 32 <= p.rows_a) {
      // through shared memory, 16 tokens at a time: eight lanes then write a token's 32 features as 16-byte
      // pieces (four tokens per store instruction instead of one)
      float* st = reinterpret_cast<float*>(stage_w);                  // [16 tokens][32 features]
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 16; ++j) st[j * 32 + lane] = __uint_as_float(r[half * 16 + j]);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int tl = (lane >> 3) + 4 * i;
          const int tok = tok0 + half * 16 + tl;
          const float4 v = *reinterpret_cast<const float4*>(st + tl * 32 + (lane & 7) * 4);
          if (tok < b_end)
            *reinterpret_cast<float4*>(o + static_cast<size_t>(tok) * p.ldc + a_row0 + (lane & 7) * 4) = v;
        }
      }
    } else if (a_row < p.rows_a) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (tok0 + j < b_end) o[static_cast<size_t>(tok0 + j) * p.ldc + a_row] = __uint_as_float(r[j]);
    }
    return;
  }
  if (p.act) {
    // lanes are weight rows laid out [8 gate | 8 up | 8 gate | 8 up]: lane l pairs with l ^ 8;
    // the 16 lanes with (l & 8) == 0 end up with one output feature each
    __nv_bfloat16* st = reinterpret_cast<__nv_bfloat16*>(stage_w);     // [32 tokens][16 features]
    const bool writer = (lane & 8) == 0;
    const int of = ((lane >> 4) << 3) + (lane & 7);
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float v = __uint_as_float(r[j]);
      const float up = __shfl_xor_sync(0xffffffffu, v, 8);
      if (writer) st[j * 16 + of] = __float2bfloat16(silu_mul_f(v, up));
    }
    __syncwarp();
    const int out_col = (a_row0 >> 1) + (lane & 1) * 8;
    if (p.vec_ok && a_row0 + 32 <= p.rows_a) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int tl = (lane >> 1) + 16 * i;
        const uint4 v = *reinterpret_cast<const uint4*>(stage_w + tl * 32 + (lane & 1) * 16);
        if (tok0 + tl < b_end)
          *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(tok0 + tl) * p.ldc +
                                    out_col) = v;
      }
    } else if (writer && a_row < p.rows_a) {
      __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out);
      const int oc = (a_row >> 4) * 8 + (a_row & 7);
      for (int j = 0; j < 32; ++j)
        if (tok0 + j < b_end) o[static_cast<size_t>(tok0 + j) * p.ldc + oc] = st[j * 16 + of];
    }
    return;
  }
  if (!(p.vec_ok || push.enabled)) {
    if (a_row < p.rows_a) {
      __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (tok0 + j < b_end) o[static_cast<size_t>(tok0 + j) * p.ldc + a_row] = __float2bfloat16(__uint_as_float(r[j]));
    }
    return;
  }
  __nv_bfloat16* st = reinterpret_cast<__nv_bfloat16*>(stage_w);       // [32 tokens][32 features]
  __syncwarp();                  // the readers of the previous chunk are done with the buffer
#pragma unroll
  for (int j = 0; j < 32; ++j) st[j * 32 + lane] = __float2bfloat16(__uint_as_float(r[j]));
  __syncwarp();
  const int col = a_row0 + (lane & 3) * 8;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int tl = (lane >> 2) + 8 * i;
    const int tok = tok0 + tl;
    const uint4 v = *reinterpret_cast<const uint4*>(stage_w + tl * 64 + (lane & 3) * 16);
    if (tok < b_end && col < p.rows_a) {       // rows_a is a multiple of 8 on this path
      if (push.enabled)
        tp_push_store8(push, tok, col, split, v);
      else
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(tok) * p.ldc + col) = v;
    }
  }
}

// Persistent kernel: every CTA walks work items (output tile x K split) with stride gridDim.x.
// The shared-memory stage ring and its phases run on across work items, and the accumulator
// is double buffered in TMEM, so the epilogue of one tile overlaps the main loop of the next.
__global__ void __launch_bounds__(kGemmThreads, 2)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmParams p, const __grid_constant__ TpPush push, const GemmRowWait row_wait) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  grid_dep_launch();           // the next kernel of the stream may start its prologue (see launch.cuh)
  if (push.enabled) tp_prof(push, 0);
  if (threadIdx.x == 0) gemm_prof(p, 0);
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
  uint64_t* peers_done = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(full_bar) + 176);   // cluster split-K
  uint64_t* recv_full = peers_done + 1;
  uint8_t* staging = reinterpret_cast<uint8_t*>(full_bar) + 256;   // kStagingBytes, swapped orientation only

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
    if (p.cluster_split > 1) {
      // peers_done: every CTA of the cluster reports that its MMAs no longer read shared memory;
      // recv_full: the other CTAs' partial sums for the accumulator columns this CTA finishes have landed
      const int cs = p.cluster_split, nch = (p.bn + 31) >> 5, crank = static_cast<int>(cluster_ctarank());
      const int owned = crank < nch ? (nch - crank + cs - 1) / cs : 0;
      mbar_init(peers_done, static_cast<uint32_t>(cs));
      mbar_init(recv_full, 1);
      mbar_fence_init();
      mbar_expect_tx(recv_full, static_cast<uint32_t>((cs - 1) * owned) * 16384u);
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
  if (p.cluster_split > 1) cluster_arrive_wait();      // the barriers above exist in every CTA of the cluster
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) gemm_prof(p, 1);
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
      gemm_prof(p, 2);
      grid_dep_wait();
      // all-gather -> GEMM: the activation rows other ranks broadcast into this rank's buffer
      if (row_wait.n > 0 && !gemm_wait_rows(row_wait)) report_status(p.status, kGemmKernelId, kPeerFlagTimeout);
      // K blocks issued so far by this CTA, across work items: `it` counts them, `s` is the stage the
      // next one goes to and `round` how often the ring has wrapped (kept incrementally: no division
      // in the loop)
      uint32_t it = 0, s = 0, round = 0;
      const uint32_t nst = static_cast<uint32_t>(p.stages);
      for (int w = blockIdx.x; w < total_work && !*abort_flag; w += gridDim.x) {
        const WorkItem wi = decode_work(p, w);
        const int kb_begin = wi.split * p.k_blocks_per_split;
        const int kb_end = min(kb_begin + p.k_blocks_per_split, total_kb);
        const int ya = wi.tile_a * kBM, yb = wi.tile_b * p.bn;
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1)) {
            report_status(p.status, kGemmKernelId, kWaitEmptyTimeout);
            *abort_flag = 1;
            break;
          }
          uint8_t* sa = smem + static_cast<size_t>(s) * stage_bytes;
          const bool weights_out = it < pre;      // expect_tx and the weight tile were issued above
          if (!weights_out) mbar_expect_tx(&full_bar[s], stage_bytes);
          if (!(weights_out && p.transposed))
            tma_load_2d(sa, &map_a, &full_bar[s], kb * kBK, ya, hint_a);
          if (!(weights_out && !p.transposed))
            tma_load_2d(sa + a_bytes, &map_b, &full_bar[s], kb * kBK, yb, hint_b);
          if (++s == nst) {
            s = 0;
            ++round;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t t = 0, s = 0, parity = 0;
      const uint32_t nst = static_cast<uint32_t>(p.stages);
      // descriptors of stage 0; a stage further on adds stage_bytes / 16, a K step of 16 elements adds 2
      const uint64_t desc_a0 = umma_desc_sw128(smem_u32(smem));
      const uint64_t desc_b0 = umma_desc_sw128(smem_u32(smem) + a_bytes);
      const uint32_t idesc = p.idesc;
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
        uint32_t accumulate = 0;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(&full_bar[s], parity)) {
            report_status(p.status, kGemmKernelId, kWaitFullTimeout);
            *abort_flag = 1;
            break;
          }
          tc_fence_after_sync();
          if (t == 0 && kb == kb_begin) gemm_prof(p, 3);
          const uint64_t soff = static_cast<uint64_t>((s * stage_bytes) >> 4);
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            umma_bf16(d_tmem, desc_a0 + soff + kk * 2, desc_b0 + soff + kk * 2, idesc, accumulate);
            accumulate = 1;
          }
          umma_commit(&empty_bar[s]);   // stage is free once these MMAs have read it
          if (++s == nst) {
            s = 0;
            parity ^= 1;
          }
        }
        umma_commit(&acc_full[buf]);     // accumulator complete
        if (t == 0) gemm_prof(p, 4);
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;                       // TMEM lane quarter this warp may read
    uint8_t* stage_w = staging + quarter * 2048;
    const int nchunks = (p.bn + 31) >> 5;               // 32 accumulator columns per tcgen05.ld
    uint32_t t = 0;
    bool dead = false;     // a wait ran out: no more data work, but this warp still meets the others at the barriers
    volatile int* fix_last = abort_flag + 1;
    for (int w = blockIdx.x; w < total_work; w += gridDim.x, ++t) {
      const WorkItem wi = decode_work(p, w);
      const uint32_t buf = t & 1, use = t >> 1;
      if (!dead) {
        bool ok = mbar_wait(&acc_full[buf], use & 1);
        if (!ok) {
          report_status(p.status, kGemmKernelId, kWaitAccumTimeout);
          *abort_flag = 1;
        }
        tc_fence_after_sync();
        // warp-uniform: the aligned TMEM loads below must be executed by all 32 lanes or none
        dead = !__all_sync(0xffffffffu, ok && (*abort_flag == 0));
        if (t == 0 && threadIdx.x == 64) gemm_prof(p, 5);
      }
      const int a_row0 = wi.tile_a * kBM + quarter * 32;
      const int b0 = wi.tile_b * p.bn;
      const int b_end = min(p.rows_b, b0 + p.bn);
      if (p.cluster_split > 1) {
        // ---- split-K inside a cluster: accumulator columns are dealt to the cluster's CTAs in chunks of 32;
        // every CTA sends the chunks it does not own to their owners' shared memory (the stage ring, free once
        // all MMAs of the cluster are done) and finishes the ones it owns ----
        const int cs = p.cluster_split;
        const int crank = static_cast<int>(cluster_ctarank());
        const int owned_max = (nchunks + cs - 1) / cs;
        if (threadIdx.x == 64)
          for (int q = 0; q < cs; ++q) mbar_arrive_cluster(map_to_cta(smem_u32(peers_done), static_cast<uint32_t>(q)));
        if (!dead) {
          bool ok = true;
          if (lane == 0) ok = mbar_wait(peers_done, 0);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) {
            report_status(p.status, kGemmKernelId, kWaitAccumTimeout);
            dead = true;
          }
        }
        if (!dead) {
          const uint32_t lane_addr = tmem_base + buf * p.acc_stride + (static_cast<uint32_t>(quarter * 32) << 16);
          const uint32_t recv_local = smem_u32(smem);
          for (int c = 0; c < nchunks; ++c) {
            const int owner = c % cs;
            if (owner == crank) continue;
            uint32_t r[32];
            tmem_ld32(lane_addr + static_cast<uint32_t>(c * 32), r);
            tmem_ld_wait();
            tmem_ld_fence_regs(r);
            const int src_idx = crank < owner ? crank : crank - 1;
            const uint32_t slot = static_cast<uint32_t>(src_idx * owned_max + c / cs) * 16384u;
            const uint32_t dst = map_to_cta(recv_local + slot, static_cast<uint32_t>(owner));
            const uint32_t bar = map_to_cta(smem_u32(recv_full), static_cast<uint32_t>(owner));
            // through this warp's staging buffer, 16 tokens at a time, so that the stores into the owner's
            // shared memory are 16 bytes each: [32 tokens][128 features] fp32 there, this warp's 32 features
            float* st = reinterpret_cast<float*>(stage_w);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 16; ++j) st[j * 32 + lane] = __uint_as_float(r[half * 16 + j]);
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int tl = (lane >> 3) + 4 * i;
                const float4 v = *reinterpret_cast<const float4*>(st + tl * 32 + (lane & 7) * 4);
                st_async_v4(dst + static_cast<uint32_t>(((half * 16 + tl) * 128 + quarter * 32 + (lane & 7) * 4) * 4), v, bar);
              }
            }
          }
          const bool owns = crank < nchunks;
          if (owns) {
            bool ok = true;
            if (lane == 0) ok = mbar_wait(recv_full, 0);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) report_status(p.status, kGemmKernelId, kWaitAccumTimeout);
            const float* recv = reinterpret_cast<const float*>(smem);
            for (int c = crank; c < nchunks; c += cs) {
              uint32_t r[32];
              tmem_ld32(lane_addr + static_cast<uint32_t>(c * 32), r);
              tmem_ld_wait();
              tmem_ld_fence_regs(r);
              for (int sidx = 0; sidx < cs - 1; ++sidx) {       // source order: the sum does not depend on arrival order
                const float* src = recv + static_cast<size_t>(sidx * owned_max + c / cs) * 4096 + quarter * 32 + lane;
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + src[j * 128]);
              }
              store_swapped32(p, push, stage_w, lane, a_row0, b0 + c * 32, b_end, 0, r);
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
        if (threadIdx.x == 64) gemm_prof(p, 6);
        continue;
      }
      if (!dead) {
        const uint32_t lane_addr = tmem_base + buf * p.acc_stride + (static_cast<uint32_t>(quarter * 32) << 16);
        float* plane = p.fixup ? p.fix_planes + static_cast<size_t>(wi.split) * p.rows_a * p.rows_b : nullptr;
        // Two register sets: the load of the next 32 columns is in flight while this one is stored.
        uint32_t ra[32], rb[32];
        tmem_ld32(lane_addr, ra);
        for (int ch = 0; ch < nchunks; ch += 2) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            if (ch + half < nchunks) {
              uint32_t(&r)[32] = half == 0 ? ra : rb;
              uint32_t(&rn)[32] = half == 0 ? rb : ra;
              tmem_ld_wait();
              tmem_ld_fence_regs(r);
              if (ch + half + 1 < nchunks) tmem_ld32(lane_addr + static_cast<uint32_t>((ch + half + 1) * 32), rn);
              const int c0 = b0 + (ch + half) * 32;
              if (p.fixup) {
                if (a_row0 + lane < p.rows_a) {
#pragma unroll
                  for (int j = 0; j < 32; ++j)
                    if (c0 + j < b_end)
                      plane[static_cast<size_t>(c0 + j) * p.rows_a + a_row0 + lane] = __uint_as_float(r[j]);
                }
              } else if (p.transposed) {
                store_swapped32(p, push, stage_w, lane, a_row0, c0, b_end, wi.split, r);
              } else {
                store_row32(p, push, a_row0 + lane, c0, b_end, wi.split, r);
              }
            }
          }
        }
        // this warp has drained its quarter of the accumulator
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
      }
      if (p.fixup) {
        // Whoever brings the tile's last partial plane sums the planes (in split order, so the result does
        // not depend on who that is) and runs the normal epilogue. Nobody waits for anybody.
        __threadfence();
        named_barrier(3, 128);
        if (threadIdx.x == 64) {
          uint32_t* ctr = p.fix_counters + wi.tile_a * p.tiles_b + wi.tile_b;
          const unsigned ticket = atomicAdd(ctr, 1u);
          const int last = ticket == static_cast<unsigned>(p.splits - 1);
          if (last) *ctr = 0u;                     // every split has arrived: ready for the next launch
          *fix_last = last;
        }
        named_barrier(3, 128);
        if (*fix_last && !dead) {
          // The planes hold [token][feature] rows, the layout of the output: 16 threads take a token row of
          // the tile (8 features each), four rows and two planes at a time to keep enough loads in flight.
          __threadfence();
          const size_t plane_stride = static_cast<size_t>(p.rows_a) * p.rows_b;
          const int et = static_cast<int>(threadIdx.x) - 64;
          const int col = wi.tile_a * kBM + (et & 15) * 8;
          if (col < p.rows_a) {
            for (int tb = b0 + (et >> 4); tb < b_end; tb += 32) {
              float acc[4][8];
#pragma unroll
              for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
              for (int sp = 0; sp < p.splits; sp += 2) {
                float4 v[2][4][2];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                  for (int u = 0; u < 4; ++u) {
                    const int tok = tb + 8 * u;
                    const bool on = sp + h < p.splits && tok < b_end;
                    const float4* src = reinterpret_cast<const float4*>(
                        p.fix_planes + (sp + h) * plane_stride + static_cast<size_t>(on ? tok : b0) * p.rows_a + col);
                    v[h][u][0] = on ? ld_cg_f4(src) : make_float4(0.f, 0.f, 0.f, 0.f);
                    v[h][u][1] = on ? ld_cg_f4(src + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
                  }
#pragma unroll
                for (int h = 0; h < 2; ++h)       // plane order: the sum does not depend on which CTA came last
#pragma unroll
                  for (int u = 0; u < 4; ++u) {
                    acc[u][0] += v[h][u][0].x; acc[u][1] += v[h][u][0].y; acc[u][2] += v[h][u][0].z; acc[u][3] += v[h][u][0].w;
                    acc[u][4] += v[h][u][1].x; acc[u][5] += v[h][u][1].y; acc[u][6] += v[h][u][1].z; acc[u][7] += v[h][u][1].w;
                  }
              }
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int tok = tb + 8 * u;
                if (tok < b_end) {
                  uint4 o;
                  o.x = pack_bf16(acc[u][0], acc[u][1]);
                  o.y = pack_bf16(acc[u][2], acc[u][3]);
                  o.z = pack_bf16(acc[u][4], acc[u][5]);
                  o.w = pack_bf16(acc[u][6], acc[u][7]);
                  if (push.enabled)
                    tp_push_store8(push, tok, col, 0, o);
                  else
                    *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(tok) * p.ldc + col) = o;
                }
              }
            }
          }
        }
        named_barrier(3, 128);                    // fix_last is rewritten for the next tile
      }
      if (threadIdx.x == 64) gemm_prof(p, 6);
    }
    if (push.enabled) {
      // "this CTA's tiles are in the reducing ranks' slots": once per CTA that had GEMM work, also when the
      // pipeline gave up (the peers' waits then still end; the status word says what happened)
      if (static_cast<int>(blockIdx.x) < total_work) {
        named_barrier(1, 128);                        // all four epilogue warps have issued their stores
        const int et = static_cast<int>(threadIdx.x) - 64;
        if (et < push.comm.world) tp_push_signal_tiles(push, et);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
  // no CTA of a cluster leaves while another may still be writing into its shared memory
  if (p.cluster_split > 1) cluster_arrive_wait();
  if (threadIdx.x == 0) gemm_prof(p, 7);
  if (push.enabled) tp_push_tail<kTailMaxVec>(push);
}

// ---- CTA-pair variant --------------------------------------------------------------------------------
// Two CTAs of a 2-wide cluster compute 256 x BN output tiles with tcgen05.mma cta_group::2 (BN a
// multiple of 16 up to 256). Each CTA loads 128 rows of A and BN/2 rows of B per K block, so the
// shared-memory fill traffic per FLOP is a third lower than for a lone CTA's 128 x BN tile. CTA rank 0
// issues the MMAs for the pair; each CTA drains its own 128 accumulator rows.
//
// Tiles are dealt whole and round-robin. When the last wave would leave more than half of the SM pairs idle,
// its tiles are cut into two or three K parts, one part per pair ("stream-K tail"): the pairs holding a
// tile's first parts store their fp32 accumulators into their own slots of the workspace and raise the
// counter of the pair that holds the last part; that pair adds the slots to its own accumulator in part
// order (the sum does not depend on timing), runs the normal epilogue and clears its counter for the next
// launch. The parts run first, the whole tiles after them.
constexpr int kPairAccStride = 256;
constexpr long long kSkReserveBytes = 20ll << 20;   // tail of the workspace kept zero for partial tiles + counters
constexpr long long kSkCounterBytes = 4096;         // the very end of it: two counters per SM pair, then one per tile
constexpr int kFixCounterFirst = 256;               // first counter word of the single-CTA kernel's split-K fix-up
constexpr int kFixCounterTiles = 768;

struct StreamK {
  int parts;               // K parts every tile of the stream-K region is cut into (2 or 3; 1: no such region)
  int units_per_pair;      // K blocks of a part
  int dp_tiles;            // tiles [0, dp_tiles) are dealt whole, round-robin over the pairs
  int sk_tiles;            // the tiles after them, one part per pair
  int slot_floats;         // floats per slot: 256 rows x BN rounded up to whole 32-column chunks
  float* slots;            // [pairs][slot_floats], indexed by the pair that wrote it (a tile's earlier K parts)
  uint32_t* counters;      // [pairs][2] (finishing pair, CTA rank); zero between launches
};

struct Segment {
  int tile, kb_begin, kb_end;
  int sk_tile;             // index of the tile inside the stream-K region, -1 for a whole tile dealt round-robin
};

// A pair's work: first its part of a tile of the stream-K region (pair p holds part p % parts of that region's
// tile p / parts; the last part finishes the tile), then its whole tiles pair, pair + pairs, ... of the
// round-robin region, so that the pairs running at the same time work on neighbouring tiles there.
struct PairWork {
  int total_kb, dp_next, dp_tiles, stride;
  int sk_tile, kb_begin, kb_end;      // sk_tile < 0: no stream-K part (left)
  __device__ PairWork(const GemmParams& p, const StreamK& sk, int pair, int num_pairs, int kb_per_tile) {
    total_kb = kb_per_tile;
    dp_next = pair;
    dp_tiles = sk.dp_tiles;
    stride = num_pairs;
    sk_tile = -1;
    kb_begin = kb_end = 0;
    if (sk.parts > 1 && pair < sk.sk_tiles * sk.parts) {
      sk_tile = pair / sk.parts;
      const int part = pair - sk_tile * sk.parts;
      kb_begin = part * sk.units_per_pair;
      kb_end = min(total_kb, kb_begin + sk.units_per_pair);
    }
  }
  __device__ bool any() const { return sk_tile >= 0 || dp_next < dp_tiles; }
  __device__ bool next(Segment& sg) {
    if (sk_tile >= 0) {
      sg.sk_tile = sk_tile;
      sg.tile = dp_tiles + sk_tile;
      sg.kb_begin = kb_begin;
      sg.kb_end = kb_end;
      sk_tile = -1;
      return true;
    }
    if (dp_next < dp_tiles) {
      sg.tile = dp_next;
      sg.sk_tile = -1;
      sg.kb_begin = 0;
      sg.kb_end = total_kb;
      dp_next += stride;
      return true;
    }
    return false;
  }
};
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& tile_a, int& tile_b) {
  tile_b = tile / p.tiles_a;            // consecutive tiles walk the A (row) tiles and share the B tile
  tile_a = tile - tile_b * p.tiles_a;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const GemmParams p, const StreamK sk, const __grid_constant__ TpPush push,
                         const GemmRowWait row_wait) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  grid_dep_launch();
  if (push.enabled) tp_prof(push, 0);
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr uint32_t a_bytes = kBM * kBK * 2;
  const uint32_t half_bn = static_cast<uint32_t>(p.bn) >> 1;
  const uint32_t stage_bytes = a_bytes + half_bn * kBK * 2;      // this CTA's share of a K block
  const uint32_t nstages = static_cast<uint32_t>(p.stages);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(nstages) * stage_bytes);   // used in the leader
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
  const int total_kb = (p.k + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < nstages; ++s) {
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
  grid_dep_wait();

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      // swapped: the weights (A) stream through once, the few activation rows (B) are re-read by every tile
      const uint64_t hint_a = p.transposed ? l2_policy_evict_first() : l2_policy_evict_normal();
      const uint64_t hint_b = p.transposed ? l2_policy_evict_last() : l2_policy_evict_normal();
      uint32_t s = 0, round = 0;
      const uint32_t leader_full0 = map_to_cta(smem_u32(&full_bar[0]), 0);
      if (row_wait.n > 0 && !gemm_wait_rows(row_wait)) report_status(p.status, kGemmKernelId, kPeerFlagTimeout);
      PairWork work(p, sk, pair, num_pairs, total_kb);
      Segment sg;
      while (!*abort_flag && work.next(sg)) {
        int tile_a, tile_b;
        tile_coords(p, sg.tile, tile_a, tile_b);
        const int ya = tile_a * 256 + static_cast<int>(rank) * kBM;
        const int yb = tile_b * p.bn + static_cast<int>(rank * half_bn);
        for (int kb = sg.kb_begin; kb < sg.kb_end; ++kb) {
          if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1)) {
            report_status(p.status, kGemmKernelId, kWaitEmptyTimeout);
            *abort_flag = 1;
            break;
          }
          uint8_t* sa = smem + static_cast<size_t>(s) * stage_bytes;
          const uint32_t leader_full = leader_full0 + s * 8;
          mbar_expect_tx_cluster(leader_full, stage_bytes);
          tma_load_2d_pair(sa, &map_a, leader_full, kb * kBK, ya, hint_a);
          tma_load_2d_pair(sa + a_bytes, &map_b, leader_full, kb * kBK, yb, hint_b);
          if (++s == nstages) {
            s = 0;
            ++round;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && rank == 0) {
      uint32_t t = 0, s = 0, parity = 0;
      const uint64_t desc_a0 = umma_desc_sw128(smem_u32(smem));
      const uint64_t desc_b0 = umma_desc_sw128(smem_u32(smem) + a_bytes);
      const uint32_t idesc = p.idesc;
      const uint32_t empty0_cta0 = map_to_cta(smem_u32(&empty_bar[0]), 0);
      const uint32_t empty0_cta1 = map_to_cta(smem_u32(&empty_bar[0]), 1);
      PairWork work(p, sk, pair, num_pairs, total_kb);
      Segment sg;
      for (; !*abort_flag && work.next(sg); ++t) {
        const uint32_t buf = t & 1, use = t >> 1;
        if (use > 0 && !mbar_wait(&acc_empty[buf], (use - 1) & 1)) {
          report_status(p.status, kGemmKernelId, kWaitAccumTimeout);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * kPairAccStride;
        uint32_t accumulate = 0;
        for (int kb = sg.kb_begin; kb < sg.kb_end; ++kb) {
          if (!mbar_wait(&full_bar[s], parity)) {
            report_status(p.status, kGemmKernelId, kWaitFullTimeout);
            *abort_flag = 1;
            break;
          }
          tc_fence_after_sync();
          const uint64_t soff = static_cast<uint64_t>((s * stage_bytes) >> 4);
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            umma_bf16_pair(d_tmem, desc_a0 + soff + kk * 2, desc_b0 + soff + kk * 2, idesc, accumulate);
            accumulate = 1;
          }
          // the stage is free in both CTAs once these MMAs have read it
          umma_commit_pair(empty0_cta0 + s * 8);
          umma_commit_pair(empty0_cta1 + s * 8);
          if (++s == nstages) {
            s = 0;
            parity ^= 1;
          }
        }
        umma_commit_pair(map_to_cta(smem_u32(&acc_full[buf]), 0));
        umma_commit_pair(map_to_cta(smem_u32(&acc_full[buf]), 1));
      }
    }
  } else {
    // ---------------- epilogue (both CTAs, own 128 accumulator rows) ----------------
    const int quarter = warp & 3;
    const int nchunks = (p.bn + 31) >> 5;
    const int row_in_tile = static_cast<int>(rank) * kBM + quarter * 32 + lane;
    // swapped orientation (weights on the MMA's M axis, tokens on N): per-warp transpose buffer after the barriers
    uint8_t* stage_w = reinterpret_cast<uint8_t*>(full_bar) + 256 + quarter * 2048;
    uint32_t t = 0;
    bool dead = false;      // a wait ran out: no more data work, but this warp keeps meeting the others at the barriers
    PairWork work(p, sk, pair, num_pairs, total_kb);
    const bool has_work = work.any();
    Segment sg;
    for (; work.next(sg); ++t) {
      int tile_a, tile_b;
      tile_coords(p, sg.tile, tile_a, tile_b);
      const uint32_t buf = t & 1, use = t >> 1;
      const bool contributes = sg.sk_tile >= 0 && sg.kb_end < total_kb;     // the tile's end belongs to another pair
      const bool finishes = sg.sk_tile >= 0 && !contributes;                // other pairs hold the tile's beginning
      if (!dead) {
        bool ok = mbar_wait(&acc_full[buf], use & 1);
        if (!ok) {
          report_status(p.status, kGemmKernelId, kWaitAccumTimeout);
          *abort_flag = 1;
        }
        tc_fence_after_sync();
        // warp-uniform: the aligned TMEM loads below must be executed by all 32 lanes or none
        dead = !__all_sync(0xffffffffu, ok && (*abort_flag == 0));
      }
      if (!dead) {
        const int a_row = tile_a * 256 + row_in_tile;
        const uint32_t lane_addr = tmem_base + buf * kPairAccStride + (static_cast<uint32_t>(quarter * 32) << 16);
        const int b0 = tile_b * p.bn;
        const int b_end = min(p.rows_b, b0 + p.bn);
        // The pair that holds the tile's last K part finishes the tile: the pairs with the earlier parts store
        // their fp32 accumulators into their own slots (plain 16-byte stores: an order of magnitude faster
        // than red.add through the L2 atomic units), the finisher adds them in part order.
        // Slot layout: [32-column chunk][4-float group j][256 rows][4 floats]: the 32 rows of a warp are
        // consecutive 16-byte pieces, so every vector access of a warp is 512 contiguous bytes.
        const int first_pair = sg.sk_tile * sk.parts;
        const int fin_pair = first_pair + sk.parts - 1;
        float* slot = sk.slots + static_cast<size_t>(contributes ? pair : first_pair) * sk.slot_floats;
        if (finishes) {
          const uint32_t want = static_cast<uint32_t>(sk.parts - 1);
          const uint32_t* ctr = sk.counters + 2 * pair + rank;
          if (lane == 0) {
            const unsigned long long t0 = global_timer_ns();
            while (ld_acquire_gpu(ctr) < want) {
              if (global_timer_ns() - t0 > kDefaultWaitNs) {
                report_status(p.status, kGemmKernelId, kWaitAccumTimeout);
                break;
              }
              __nanosleep(64);
            }
          }
          __syncwarp();
        }
        uint32_t ra[32], rb[32];
        tmem_ld32(lane_addr, ra);
        for (int ch = 0; ch < nchunks; ch += 2) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            if (ch + half < nchunks) {
              uint32_t(&r)[32] = half == 0 ? ra : rb;
              uint32_t(&rn)[32] = half == 0 ? rb : ra;
              tmem_ld_wait();
              tmem_ld_fence_regs(r);
              if (ch + half + 1 < nchunks) tmem_ld32(lane_addr + static_cast<uint32_t>((ch + half + 1) * 32), rn);
              float* sl = slot + (static_cast<size_t>(ch + half) * 8 * 256 + row_in_tile) * 4;
              if (contributes) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  *reinterpret_cast<float4*>(sl + j * 1024) =
                      make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                  __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
              } else {
                if (finishes) {
                  for (int part = 0; part + 1 < sk.parts; ++part) {
                    const float* sp = sl + static_cast<size_t>(part) * sk.slot_floats;
                    float4 v[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = ld_cg_f4(reinterpret_cast<const float4*>(sp + j * 1024));
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                      r[4 * j] = __float_as_uint(__uint_as_float(r[4 * j]) + v[j].x);
                      r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + v[j].y);
                      r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + v[j].z);
                      r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + v[j].w);
                    }
                  }
                }
                if (p.transposed)
                  store_swapped32(p, push, stage_w, lane, a_row - lane, b0 + (ch + half) * 32, b_end, 0, r);
                else
                  store_row32(p, push, a_row, b0 + (ch + half) * 32, b_end, 0, r);
              }
            }
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
      }
      if (contributes || finishes) {
        // all four epilogue warps of this CTA are done with the slot / the counter (also after a failed wait:
        // the other pairs' waits must still end, the status word says that the numbers are not to be used)
        __threadfence();
        named_barrier(2, 128);
        if (threadIdx.x == 64) {
          const int fin_pair = sg.sk_tile * sk.parts + sk.parts - 1;
          uint32_t* ctr = sk.counters + 2 * fin_pair + rank;
          if (contributes)
            red_release_gpu_add(ctr, 1u);
          else
            *reinterpret_cast<volatile uint32_t*>(ctr) = 0u;     // ready for the next launch
        }
      }
    }
    if (push.enabled && has_work) {
      named_barrier(1, 128);
      const int et = static_cast<int>(threadIdx.x) - 64;
      if (et < push.comm.world) tp_push_signal_tiles(push, et);
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
  if (push.enabled) tp_push_tail<kTailMaxVec>(push);
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
static thread_local GemmRowWait g_pending_wait = {nullptr, nullptr, 0, 0, 1};
static unsigned long long* g_tp_prof = nullptr;
static unsigned long long* g_gemm_prof = nullptr;

namespace {

constexpr int kMaxDevices = 64;

struct PlanOverride {
  int active, kind, bn, splits, stages;
};
PlanOverride g_override = {0, 0, 0, 0, 0};

constexpr unsigned kPlanNoPair = 1u;     // single-CTA kernels only
constexpr unsigned kPlanNoSplit = 2u;    // the caller cannot take fp32 partial planes
constexpr unsigned kPlanDeep = 4u;       // few CTAs: give each the whole SM's shared memory for stages
constexpr unsigned kPlanNoCluster = 8u;  // K splits as fp32 planes in global memory, not summed inside a cluster

struct PlanKey {
  int m, n, k, sms;
  unsigned flags;
  int max_splits;
  bool operator==(const PlanKey& o) const {
    return m == o.m && n == o.n && k == o.k && sms == o.sms && flags == o.flags && max_splits == o.max_splits;
  }
};
struct PlanKeyHash {
  size_t operator()(const PlanKey& k) const {
    size_t h = static_cast<size_t>(k.m) * 0x9E3779B97F4A7C15ULL;
    h ^= static_cast<size_t>(k.n) * 0xC2B2AE3D27D4EB4FULL + (h << 6) + (h >> 2);
    h ^= static_cast<size_t>(k.k) * 0x165667B19E3779F9ULL + (h << 6) + (h >> 2);
    h ^= static_cast<size_t>(k.sms * 131 + k.flags * 7 + k.max_splits) + (h << 6) + (h >> 2);
    return h;
  }
};

int env_int(const char* name, int dflt) {
  const char* e = std::getenv(name);
  return e ? std::atoi(e) : dflt;
}

void fill_single_smem(XvGemmPlan& pl, int stages) {
  const int stage_bytes = kBM * kBK * 2 + pl.bn * kBK * 2;
  pl.stages = stages;
  pl.smem_bytes = stages * stage_bytes + 256 + (pl.swapped ? kStagingBytes : 0) + 1024;
}

// Swapped (weights on the MMA M axis) or normal single-CTA plan, with split-K when the output tiles
// alone cannot occupy the machine.
void plan_single(int m, int n, int k, int num_sms, unsigned flags, int max_splits, XvGemmPlan& pl) {
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
  const int extra = 256 + (pl.swapped ? kStagingBytes : 0) + 1024;
  static const int small_budget_kb = env_int("XV_GEMM_SWAPPED_SMEM_KB", 112);     // experiment knob
  const int smem_budget = (pl.swapped && pl.bn <= 128 && !(flags & kPlanDeep)) ? small_budget_kb * 1024 : 220 * 1024;
  int stages = (smem_budget - extra) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) stages = 2;
  const int smem_bytes = stages * stage_bytes + extra;
  pl.ctas_per_sm = (smem_bytes <= 113 * 1024 && 2 * pow2_cols(pl.bn) <= 256) ? 2 : 1;
  // Split K bounds: at least 4 K blocks per split, at most 16 splits, and fp32 partials (written and
  // read back once) no larger than about a quarter of the weight bytes or 16 MB (they stay in L2).
  const int slots = num_sms * pl.ctas_per_sm;
  int splits = 1;
  if (tiles < num_sms && !(flags & kPlanNoSplit)) {
    splits = slots / tiles;
    int by_traffic = k / (8 * m) > 1 ? k / (8 * m) : 1;
    const long long plane = static_cast<long long>(m) * n * 4;
    const int by_bytes = static_cast<int>((16ll << 20) / (plane > 0 ? plane : 1));
    if (by_bytes > by_traffic) by_traffic = by_bytes;
    if (splits > by_traffic) splits = by_traffic;
    while (splits > 1 && total_kb / splits < 4) --splits;
    static const int env_max = env_int("XV_GEMM_MAX_SPLITS", 16);      // experiment knob: cap on split-K
    if (splits > env_max) splits = env_max;
    if (splits > 16) splits = 16;
    if (max_splits > 0 && splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
  }
  // Swapped orientation: up to four K splits of a tile form one thread-block cluster and sum their accumulators
  // through distributed shared memory: no fp32 planes in global memory, the output is final (bf16, activation
  // or pushed tiles). The receive buffers alias the stage ring, which must hold them.
  static const int cluster_on = env_int("XV_GEMM_CLUSTER", 1);
  pl.cluster = 0;
  if (cluster_on && pl.swapped && splits > 1 && !(flags & kPlanNoCluster)) {
    int cs = splits > 4 ? 4 : splits;
    const int nch = (pl.bn + 31) / 32;
    while (cs > 1 && (cs - 1) * ((nch + cs - 1) / cs) * 16384 > stages * stage_bytes) --cs;
    if (cs > 1) {
      splits = cs;
      pl.cluster = 1;
    }
  }
  pl.k_blocks_per_split = (total_kb + splits - 1) / splits;
  pl.splits = (total_kb + pl.k_blocks_per_split - 1) / pl.k_blocks_per_split;
  if (pl.cluster && pl.splits < 2) pl.cluster = 0;
  if (stages > pl.k_blocks_per_split && pl.k_blocks_per_split >= 2 && !pl.cluster) stages = pl.k_blocks_per_split;
  fill_single_smem(pl, stages);
  pl.workspace_bytes = (pl.splits > 1 && !pl.cluster) ? static_cast<long long>(pl.splits) * m * n * 4 : 0;
}

// Parts a tile of the last, `rest`-tile wave is cut into: as many as there are idle pairs per tile, at most
// three (two contributions to a slot commute), none when more than half of the pairs would be busy anyway.
int sk_parts_for(int rest, int pairs, int total_kb) {
  if (rest <= 0 || total_kb < 16) return 1;
  int parts = pairs / rest;
  if (parts > 3) parts = 3;
  return parts < 2 ? 1 : parts;
}

// CTA-pair plan: 256 x bn tiles dealt whole and round-robin, with the last wave's tiles cut into K parts when
// `stream_k` is set and that wave is less than half full. bn <= 0 picks the widest tile that splits N evenly.
void fill_pair(int m, int n, int k, int bn, int num_sms, int stream_k, XvGemmPlan& pl, bool swapped = false) {
  const int total_kb = (k + kBK - 1) / kBK;
  if (swapped) {
    // weights on the 256-row M axis, the (at most 256) tokens on N: every weight byte is read once and a
    // pair's K block carries as many FLOPs per operand byte as a 256 x 256 tile of a large GEMM
    bn = round_up(m, 16);
    const int t = m;
    m = n;
    n = t;
  }
  if (bn <= 0) {
    const int tiles_b = (n + 255) / 256;
    bn = round_up((n + tiles_b - 1) / tiles_b, 16);
  }
  if (bn > 256) bn = 256;
  if (bn < 16) bn = 16;
  pl.pair = 1;
  pl.swapped = swapped ? 1 : 0;
  pl.bn = bn;
  pl.tiles_a = (m + 255) / 256;
  pl.tiles_b = (n + bn - 1) / bn;
  pl.splits = 1;
  pl.k_blocks_per_split = total_kb;
  const int stage_bytes = kBM * kBK * 2 + (bn / 2) * kBK * 2;
  int stages = (200 * 1024) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  pl.stages = stages;
  pl.smem_bytes = stages * stage_bytes + 256 + (swapped ? kStagingBytes : 0) + 1024;
  pl.ctas_per_sm = 1;
  const int pairs = num_sms / 2;
  const int tiles = pl.tiles_a * pl.tiles_b;
  pl.sk_tiles = 0;
  pl.sk_parts = 1;
  pl.units_per_pair = 0;
  pl.workspace_bytes = 0;
  const int parts = stream_k > 0 ? sk_parts_for(tiles % pairs, pairs, total_kb) : 1;
  if (parts < 2) return;
  pl.sk_tiles = tiles % pairs;
  pl.sk_parts = parts;
  pl.units_per_pair = (total_kb + parts - 1) / parts;
  const int chunks = (bn + 31) / 32;
  pl.workspace_bytes = static_cast<long long>(pairs) * chunks * 256 * 32 * 4 + kSkCounterBytes;
}

std::unordered_map<PlanKey, XvGemmPlan, PlanKeyHash> g_plan_cache;
std::mutex g_plan_mu;

// Chooses kernel, orientation, tile and split-K for a problem. Pure host arithmetic so callers (and
// CPU tests) can size the workspace before launching.
int gemm_plan_impl(int m, int n, int k, int num_sms, XvGemmPlan* plan, unsigned flags, int max_splits) {
  if (m <= 0 || n <= 0 || k <= 0 || (k % 8) != 0) return XV_ERR_SHAPE;
  if (num_sms <= 0) num_sms = 148;
  if (g_disable_pair) flags |= kPlanNoPair;
  const PlanKey key{m, n, k, num_sms, flags, max_splits};
  if (!g_override.active) {
    std::lock_guard<std::mutex> g(g_plan_mu);
    auto it = g_plan_cache.find(key);
    if (it != g_plan_cache.end()) {
      *plan = it->second;
      return 0;
    }
  }
  XvGemmPlan pl;
  std::memset(&pl, 0, sizeof(pl));
  if (g_override.active) {
    // test and tuning hook: a fixed kernel / tile / split instead of the planner's choice
    const int total_kb = (k + kBK - 1) / kBK;
    int sp = g_override.splits > 0 ? g_override.splits : 1;
    if (sp > total_kb) sp = total_kb;
    if (g_override.kind == 3 && m <= 256) {
      fill_pair(m, n, k, 0, num_sms, g_override.splits >= 0 ? 1 : 0, pl, true);
    } else if (g_override.kind == 2 || g_override.kind == 3) {
      // `splits` of the hook: > 0 cuts the last wave's tiles into K parts (stream-K tail), else whole tiles only
      const int bn = g_override.bn > 0 ? round_up(g_override.bn, 16) : 0;
      fill_pair(m, n, k, bn, num_sms, g_override.splits > 0 ? 1 : 0, pl);
      if (g_override.stages > 1 && g_override.stages <= pl.stages) {
        pl.smem_bytes -= (pl.stages - g_override.stages) * (kBM * kBK * 2 + (pl.bn / 2) * kBK * 2);
        pl.stages = g_override.stages;
      }
    } else {
      plan_single(m, n, k, num_sms, flags | kPlanNoSplit | kPlanNoCluster, 0, pl);
      if (g_override.kind == 1 && m <= 256) {       // normal orientation for a small batch
        pl.swapped = 0;
        pl.bn = n >= 256 ? 256 : round_up(n, 16);
        pl.tiles_a = (m + kBM - 1) / kBM;
        pl.tiles_b = (n + pl.bn - 1) / pl.bn;
      }
      if (g_override.bn > 0 && !pl.swapped) {
        pl.bn = round_up(g_override.bn > 256 ? 256 : g_override.bn, 16);
        pl.tiles_b = (n + pl.bn - 1) / pl.bn;
      }
      pl.k_blocks_per_split = (total_kb + sp - 1) / sp;
      pl.splits = (total_kb + pl.k_blocks_per_split - 1) / pl.k_blocks_per_split;
      const int stage_bytes = kBM * kBK * 2 + pl.bn * kBK * 2;
      int stages = g_override.stages > 1 ? g_override.stages : (200 * 1024) / stage_bytes;
      if (stages > kMaxStages) stages = kMaxStages;
      while (stages > 2 && stages * stage_bytes + 256 + kStagingBytes + 1024 > 222 * 1024) --stages;
      fill_single_smem(pl, stages);
      pl.ctas_per_sm = (pl.smem_bytes <= 113 * 1024 && 2 * pow2_cols(pl.bn) <= 256) ? 2 : 1;
      pl.workspace_bytes = pl.splits > 1 ? static_cast<long long>(pl.splits) * m * n * 4 : 0;
    }
    *plan = pl;
    return 0;
  }
  plan_single(m, n, k, num_sms, flags, max_splits, pl);
  // CTA pairs (cta_group::2, 256-row tiles) instead? Measured on a B200 (bench/gemm_sweep.py): a pair's K block
  // takes 0.30 us + 0.55 ns per tile column almost independently of the shape (the operand stream from L2
  // bounds it, not the MMA), pairs work in waves of SMs / 2 tiles, so the tile width is picked to make the
  // tile count fit the waves; among equal costs the wider tile wins (fewer operand bytes per FLOP).
  //  * above 256 rows the pairs beat lone CTAs on every measured shape;
  //  * from 161 to 256 rows (a decode batch) the swapped single-CTA kernel with split-K wins unless there
  //    are enough output columns for the pairs to fill the machine without splitting K.
  static const int pair_min_m = env_int("XV_GEMM_PAIR_MIN_M", 161);
  static const int streamk = env_int("XV_GEMM_STREAMK", 1);
  const int total_kb = (k + kBK - 1) / kBK;
  // From pair_swap_min_m to 256 rows (a decode batch) the pairs run swapped: weights on the 256-row M axis, all
  // tokens in one N tile. Every weight byte then crosses L2 -> SM once and the activation is re-read once per
  // 256 weight rows, where the unswapped 256 x BN tiling re-read it once per BN weight rows and was bound
  // by that stream; too few weight tiles for the SM pairs are cut along K (stream-K tail).
  static const int pair_swap_min_m = env_int("XV_GEMM_PAIR_SWAP_MIN_M", 161);
  static const int pair_swap_min_n = env_int("XV_GEMM_PAIR_SWAP_MIN_N", 6144);
  if (!(flags & kPlanNoPair) && m >= pair_swap_min_m && m <= 256 && n >= pair_swap_min_n && (n % 8) == 0 &&
      total_kb >= 8) {
    std::memset(&pl, 0, sizeof(pl));
    fill_pair(m, n, k, 0, num_sms, streamk, pl, true);
  } else if (!(flags & kPlanNoPair) && m >= pair_min_m && n >= 64 && (m > 256 || (n >= 6144 && total_kb <= 80))) {
    const int pairs = num_sms / 2;
    const int tiles_a = (m + 255) / 256;
    double best = 1e30, widest = 0.0;
    int best_bn = 256;
    for (int bn = 256; bn >= 96; bn -= 16) {
      if (bn > round_up(n, 16) && bn != 256) continue;
      const int tiles = tiles_a * ((n + bn - 1) / bn);
      const int waves = tiles / pairs, rest = tiles % pairs;
      const double t_kb = 0.30 + 0.00055 * bn;
      double cost = waves * (total_kb * t_kb + 1.5);
      if (rest > 0) {
        const int parts = streamk ? sk_parts_for(rest, pairs, total_kb) : 1;
        // a part costs its K blocks plus the exchange of a 256 x bn fp32 tile through L2
        cost += parts > 1 ? ((total_kb + parts - 1) / parts) * t_kb + 1.5 + 4.0 * bn / 256.0 : total_kb * t_kb + 1.5;
      }
      if (bn == 256) widest = cost;
      // a narrower tile has to win by more than the run-to-run spread of the measurements
      if (cost < best && (bn == 256 || cost < 0.94 * widest)) {
        best = cost;
        best_bn = bn;
      }
    }
    if (n < 256) best_bn = round_up(n, 16);
    std::memset(&pl, 0, sizeof(pl));
    fill_pair(m, n, k, best_bn, num_sms, streamk, pl);
  }
  *plan = pl;
  std::lock_guard<std::mutex> g(g_plan_mu);
  if (g_plan_cache.size() > (1u << 18)) g_plan_cache.clear();
  g_plan_cache.emplace(key, pl);
  return 0;
}

bool g_attr_single[kMaxDevices] = {false};
bool g_attr_pair[kMaxDevices] = {false};
std::mutex g_attr_mu;

// The opt-in to more than 48 KB of dynamic shared memory is a per-device property of a kernel.
int ensure_smem_attr(bool pair) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return XV_ERR_DRIVER;
  std::lock_guard<std::mutex> g(g_attr_mu);
  bool* done = pair ? g_attr_pair : g_attr_single;
  if (!done[dev]) {
    const cudaError_t e =
        pair ? cudaFuncSetAttribute(gemm_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024)
             : cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
    if (e != cudaSuccess) return XV_ERR_LAUNCH;
    done[dev] = true;
  }
  return 0;
}

}  // namespace

extern "C" {

// Test hook: 1 forces the single-CTA kernel for every shape (A/B comparisons), 0 restores.
void xv_gemm_disable_pair(int disable) { g_disable_pair = disable != 0; }

// All-gather -> GEMM: the next GEMM launched from this thread waits, before its first activation tile, until
// the `n` counters at `flags` (this rank's flag array, word kPushBcastWord on) have reached the values at
// `targets` (the communicator's history words kPushBcastBase on). Used after an xv_gemm_bf16_tp call with
// defer_row_wait: the rows other ranks broadcast are then awaited by the kernel that reads them, not by the
// kernel that caused them.
void xv_gemm_wait_for_rows(const void* flags, const void* targets, int n, unsigned spin_us) {
  g_pending_wait.flags = static_cast<const uint32_t*>(flags);
  g_pending_wait.targets = static_cast<const uint32_t*>(targets);
  g_pending_wait.n = n;
  g_pending_wait.spin_us = spin_us;
  g_pending_wait.target_stride = 1;
}
// Same for epoch-valued flags: the `n` flags at `flags` must all reach the one value at `target`.
void xv_gemm_wait_for_epoch(const void* flags, const void* target, int n, unsigned spin_us) {
  g_pending_wait.flags = static_cast<const uint32_t*>(flags);
  g_pending_wait.targets = static_cast<const uint32_t*>(target);
  g_pending_wait.n = n;
  g_pending_wait.spin_us = spin_us;
  g_pending_wait.target_stride = 0;
}
int xv_tp_bcast_word(void) { return kPushBcastWord; }
int xv_tp_bcast_base_word(void) { return kPushBcastBase; }

// Diagnostics: following xv_gemm_bf16_tp launches write 8 global-timer stamps per CTA into `buf`
// (device memory, 8 * 8 bytes per CTA of the largest grid, i.e. 2 * SM count CTAs); null switches it off.
void xv_tp_profile_buffer(void* buf) { g_tp_prof = static_cast<unsigned long long*>(buf); }
// Same for the single-CTA GEMM kernel's own phases (see gemm_prof); 8 stamps for each of up to 2 * SM count CTAs.
void xv_gemm_profile_buffer(void* buf) { g_gemm_prof = static_cast<unsigned long long*>(buf); }

// Test and tuning hook: kind 0 = single CTA, swapped where the planner would; 1 = single CTA, normal
// orientation; 2 = CTA pairs; 3 = CTA pairs, swapped for at most 256 rows. bn / splits / stages <= 0 keep that
// kernel's default. kind < 0 clears.
void xv_gemm_plan_override(int kind, int bn, int splits, int stages) {
  g_override.active = kind >= 0;
  g_override.kind = kind;
  g_override.bn = bn;
  g_override.splits = splits;
  g_override.stages = stages;
}

int xv_gemm_plan(int m, int n, int k, int num_sms, XvGemmPlan* plan) {
  return gemm_plan_impl(m, n, k, num_sms, plan, 0u, 0);
}
// The plan xv_gemm_bf16_noalloc runs: K splits always as fp32 planes in the scratch buffer.
int xv_gemm_plan_planes(int m, int n, int k, int num_sms, XvGemmPlan* plan) {
  return gemm_plan_impl(m, n, k, num_sms, plan, kPlanNoCluster, 0);
}

// Y[m,n] (bf16, row stride ldy) = X[m,k] (row stride ldx) * W[n,k]^T (row stride ldw).
// `workspace` must hold plan.workspace_bytes when the plan splits K. `status` may be null.
// Every argument is checked before the first launch.
static int gemm_impl(const void* x, const void* w, void* y, int m, int n, int k, long long ldx, long long ldw,
                     long long ldy, void* workspace, long long workspace_bytes, int num_sms, int* status,
                     cudaStream_t stream, bool defer_reduce, int* splits_out, int act = 0,
                     const TpPush* push_in = nullptr, int push_max_splits = 1, unsigned plan_flags = 0u) {
  XvGemmPlan pl;
  if (num_sms <= 0) num_sms = 148;
  // A workspace of at least twice the stream-K reserve has its tail set aside (and kept zero) for counters and
  // the pair kernel's partial tiles; split-K planes use the front part. Smaller workspaces are all planes.
  const bool sk_ok = workspace != nullptr && workspace_bytes >= 2 * kSkReserveBytes;
  unsigned flags = plan_flags;
  int max_splits = 0;
  if (push_in != nullptr) {
    // Pushed tiles must be complete sums: K splits are summed inside the kernel by the CTA that arrives last
    // at a tile, a chain of dependent memory round trips that only pays for a long K.
    (void)push_max_splits;
    const int total_kb = (k + kBK - 1) / kBK;
    if (!sk_ok || total_kb <= 32) flags |= kPlanNoSplit;
    flags |= kPlanDeep;
    max_splits = 4;
  }
  int rc = gemm_plan_impl(m, n, k, num_sms, &pl, flags, max_splits);
  if (rc) return rc;
  if ((ldx % 8) || (ldw % 8) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return XV_ERR_ALIGN;
  // Without the reserve the pair kernel deals whole tiles (its pairs then finish unevenly).
  if (pl.pair && pl.sk_tiles > 0 && (!sk_ok || pl.workspace_bytes > kSkReserveBytes))
    fill_pair(m, n, k, pl.bn, num_sms, 0, pl, pl.swapped != 0);
  // Split-K in the swapped orientation: the planes are summed inside the kernel by the CTA that brings a
  // tile's last one (needs a tile counter from the reserve), unless the caller wants the planes themselves.
  const bool fixup = pl.splits > 1 && !pl.cluster && pl.swapped && !pl.pair && push_in != nullptr && sk_ok &&
                     (n % 8) == 0 && pl.tiles_a * pl.tiles_b <= kFixCounterTiles;
  const bool to_planes = pl.splits > 1 && !fixup && !pl.cluster;
  if (pl.splits > 1 && !pl.cluster &&
      (!workspace || pl.workspace_bytes > (sk_ok ? workspace_bytes - kSkReserveBytes : workspace_bytes)))
    return XV_ERR_WORKSPACE;
  if (act && to_planes) return XV_ERR_UNSUPPORTED;           // callers check the plan first
  if (act && ((n % 16) || (ldy % 8))) return XV_ERR_SHAPE;
  if (to_planes && !defer_reduce && ldy != n) return XV_ERR_SHAPE;   // the reduce kernel writes a dense output
  if (push_in != nullptr && ((n % 8) || to_planes)) return XV_ERR_SHAPE;
  if ((rc = ensure_smem_attr(pl.pair != 0))) return rc;

  CUtensorMap map_a, map_b;
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  if (pl.pair && pl.swapped) {
    if ((rc = get_tensor_map(&map_a, w, n, k, ldw, kBM))) return rc;
    if ((rc = get_tensor_map(&map_b, x, m, k, ldx, pl.bn / 2))) return rc;
    p.rows_a = n;
    p.rows_b = m;
    p.transposed = 1;
  } else if (pl.pair) {
    if ((rc = get_tensor_map(&map_a, x, m, k, ldx, kBM))) return rc;
    if ((rc = get_tensor_map(&map_b, w, n, k, ldw, pl.bn / 2))) return rc;
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
  p.prof = pl.pair ? nullptr : g_gemm_prof;
  p.stages = pl.stages;
  p.k_blocks_per_split = pl.k_blocks_per_split;
  p.status = status;
  p.idesc = umma_idesc_bf16(pl.pair ? 256 : kBM, pl.bn);
  p.acc_stride = pl.pair ? kPairAccStride : pow2_cols(pl.bn);
  p.tmem_cols = 2 * p.acc_stride;
  p.tiles_a = pl.tiles_a;
  p.tiles_b = pl.tiles_b;
  p.splits = pl.splits;
  p.a_fastest = pl.swapped ? 0 : 1;
  p.cluster_split = pl.cluster ? pl.splits : 0;
  if (to_planes) {
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
    p.vec_ok = (ldy % 8 == 0) && ((reinterpret_cast<uintptr_t>(y) & 15) == 0) && (act || (n % 8) == 0);
  }
  if (fixup) {
    p.fixup = 1;
    p.fix_planes = static_cast<float*>(workspace);
    p.fix_counters = reinterpret_cast<uint32_t*>(static_cast<char*>(workspace) + workspace_bytes - kSkCounterBytes) +
                     kFixCounterFirst;
  }

  TpPush push;
  std::memset(&push, 0, sizeof(push));
  // the rows this GEMM's activation still waits for (set by xv_gemm_wait_for_rows just before this call)
  const GemmRowWait row_wait = g_pending_wait;
  g_pending_wait.n = 0;
  const int total_work = pl.tiles_a * pl.tiles_b * pl.splits;
  if (pl.pair) {
    const int pairs_avail = num_sms / 2;
    const int total_kb = (k + kBK - 1) / kBK;
    const int tiles = pl.tiles_a * pl.tiles_b;
    StreamK sk;
    std::memset(&sk, 0, sizeof(sk));
    sk.dp_tiles = tiles - pl.sk_tiles;
    sk.sk_tiles = pl.sk_tiles;
    sk.parts = pl.sk_tiles > 0 ? pl.sk_parts : 1;
    sk.units_per_pair = pl.sk_tiles > 0 ? pl.units_per_pair : total_kb;
    int used_pairs = sk.dp_tiles < pairs_avail ? sk.dp_tiles : pairs_avail;
    if (pl.sk_tiles > 0) {
      const int sk_pairs = pl.sk_tiles * pl.sk_parts;
      if (sk_pairs > pairs_avail) return XV_ERR_SHAPE;
      if (sk_pairs > used_pairs) used_pairs = sk_pairs;
      sk.slot_floats = ((pl.bn + 31) / 32) * 256 * 32;
      char* tail = static_cast<char*>(workspace) + workspace_bytes - kSkReserveBytes;
      sk.slots = reinterpret_cast<float*>(tail);
      sk.counters = reinterpret_cast<uint32_t*>(static_cast<char*>(workspace) + workspace_bytes - kSkCounterBytes);
    }
    int pairs = used_pairs;
    if (push_in) {
      push = *push_in;
      push.enabled = 1;
      push.splits = 1;
      // every CTA takes part in the row phase and waits for the others: the whole grid must be resident
      int per_sm = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_tcgen05_pair_kernel, kGemmThreads,
                                                        pl.smem_bytes) != cudaSuccess || per_sm < 1)
        return XV_ERR_LAUNCH;
      pairs = pairs_avail;
      push.signal_ctas = 2 * used_pairs;
    }
    if (launch_pdl(gemm_tcgen05_pair_kernel, dim3(2 * pairs), dim3(kGemmThreads), pl.smem_bytes, stream, map_a, map_b,
                   p, sk, push, row_wait) != cudaSuccess)
      return XV_ERR_LAUNCH;
  } else {
    int slots = num_sms * pl.ctas_per_sm;
    int grid = total_work < slots ? total_work : slots;
    if (pl.cluster) grid = total_work;          // one tile split per CTA; clusters are consecutive CTAs
    if (push_in) {
      push = *push_in;
      push.enabled = 1;
      push.splits = 1;               // K splits are summed before the push (inside the cluster, or by the fix-up)
      int per_sm = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_tcgen05_kernel, kGemmThreads, pl.smem_bytes) !=
              cudaSuccess || per_sm < 1)
        return XV_ERR_LAUNCH;
      if (per_sm > pl.ctas_per_sm) per_sm = pl.ctas_per_sm;
      slots = num_sms * per_sm;
      // CTAs beyond the GEMM tiles take the rows this rank reduces; every CTA must be resident at once
      const int n_mine = push.two_shot ? (push.rows + push.comm.world - 1) / push.comm.world : push.rows;
      const int cs = pl.cluster ? pl.splits : 1;
      if (pl.cluster && total_work > slots) return XV_ERR_UNSUPPORTED;
      grid = (total_work < slots ? total_work : slots) + n_mine;
      if (grid > slots) grid = slots;
      grid = grid / cs * cs;                       // whole clusters
      if (grid < total_work && pl.cluster) grid = total_work;
      if (grid < 1) grid = 1;
      push.signal_ctas = total_work < grid ? total_work : grid;
    }
    const cudaError_t le =
        pl.cluster ? launch_pdl_cluster(gemm_tcgen05_kernel, dim3(grid), dim3(kGemmThreads), pl.smem_bytes, stream,
                                        static_cast<unsigned>(pl.splits), map_a, map_b, p, push, row_wait)
                   : launch_pdl(gemm_tcgen05_kernel, dim3(grid), dim3(kGemmThreads), pl.smem_bytes, stream, map_a, map_b,
                                p, push, row_wait);
    if (le != cudaSuccess) return XV_ERR_LAUNCH;
  }
  if (cudaGetLastError() != cudaSuccess) return XV_ERR_LAUNCH;
  if (push_in) return 0;
  if (splits_out) *splits_out = to_planes ? pl.splits : 1;
  if (to_planes && !defer_reduce) {
    const long long elems = static_cast<long long>(m) * n;
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

// RowParallel GEMM + cross-rank sum + residual add + RMSNorm as ONE kernel (push protocol, see
// tp_device.cuh). The GEMM epilogue writes this rank's partial [m, n] into the slot array at
// `slot_offset` (`slot_bytes` long) of the symmetric buffers of the ranks that reduce it.
//   two_shot = 1: rank r reduces rows r, r + world, ...; `residual_in` / `residual_out` are local
//                 [m, n] buffers of which only those rows are touched; the finished rows are broadcast to
//                 byte offset `h_offset` of every rank's symmetric buffer (y_out unused).
//   two_shot = 0: every rank reduces all rows into its local `y_out` (and `residual_out`).
//   mode 0: residual_out = sum (+ residual_in, may be null); out = rmsnorm(residual_out) * norm_w.   mode 1: out = sum.
// `epoch`: 32 uint32 words of local device memory, zero-initialised once (the kernels keep their counters'
// history there). Returns XV_ERR_WORKSPACE when the slot array is too small for the problem.
int xv_gemm_bf16_tp(const void* x, const void* w, int m, int n, int k, long long ldx, long long ldw, void* workspace,
                    long long workspace_bytes, int num_sms, const void* const* peer_bufs, void* const* peer_flags,
                    const void* mc_buf, void* epoch, int rank,
                    int world, long long slot_offset, long long slot_bytes, int two_shot, long long h_offset,
                    const void* residual_in, void* residual_out, const void* norm_w, void* y_out, float eps, int mode,
                    int defer_row_wait, unsigned spin_us, int* status, cudaStream_t stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || (n % 8) || n > kGemmThreads * kTailMaxVec * 8 ||
      (slot_offset & 15) || (two_shot && (h_offset & 15)) || m <= 0)
    return XV_ERR_SHAPE;
  if (mode == 0 && (residual_out == nullptr || norm_w == nullptr)) return XV_ERR_SHAPE;
  if (!two_shot && y_out == nullptr) return XV_ERR_SHAPE;
  TpPush t;
  std::memset(&t, 0, sizeof(t));
  for (int r = 0; r < kMaxRanks; ++r) {
    t.comm.peer_buf[r] = r < world ? peer_bufs[r] : nullptr;
    t.comm.peer_flags[r] = r < world ? static_cast<uint32_t*>(peer_flags[r]) : nullptr;
  }
  t.comm.mc_buf = mc_buf;
  t.comm.epoch = static_cast<uint32_t*>(epoch);
  t.comm.rank = rank;
  t.comm.world = world;
  t.comm.spin_limit = spin_us;
  t.comm.status = status;
  t.two_shot = two_shot ? 1 : 0;
  t.slot_offset = slot_offset;
  t.cap_rows = two_shot ? (m + world - 1) / world : m;
  t.h_offset = h_offset;
  t.y = static_cast<__nv_bfloat16*>(y_out);
  t.residual_in = static_cast<const __nv_bfloat16*>(residual_in);
  t.residual_out = static_cast<__nv_bfloat16*>(residual_out);
  t.norm_w = static_cast<const __nv_bfloat16*>(norm_w);
  t.rows = m;
  t.hidden = n;
  t.eps = eps;
  t.mode = mode;
  t.defer_row_wait = (two_shot && defer_row_wait) ? 1 : 0;
  t.prof = g_tp_prof;
  if (static_cast<long long>(world) * t.cap_rows * n * 2 > slot_bytes) return XV_ERR_WORKSPACE;
  return gemm_impl(x, w, nullptr, m, n, k, ldx, ldw, n, workspace, workspace_bytes, num_sms, status, stream, false,
                   nullptr, 0, &t, 1);
}

// Y[m, n/2] = silu(gate) * up, with W's rows interleaved in groups of 16 = [8 gate | 8 up].
// Only for plans that do not split K (XV_ERR_UNSUPPORTED otherwise; see xv_gemm_plan).
int xv_gemm_bf16_silu_mul(const void* x, const void* w, void* y, int m, int n, int k, long long ldx, long long ldw,
                          long long ldy, void* workspace, long long workspace_bytes, int num_sms, int* status,
                          cudaStream_t stream) {
  return gemm_impl(x, w, y, m, n, k, ldx, ldw, ldy, workspace, workspace_bytes, num_sms, status, stream, false,
                   nullptr, 1);
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
  if ((rc = xv_gemm_plan_planes(m, n, k, sms, &pl))) return rc;
  // Split-K planes have to fit; the CTA-pair kernel deals whole tiles when given a buffer this small.
  if (!pl.pair && pl.workspace_bytes > XV_NOALLOC_SCRATCH_BYTES) {
    std::fprintf(stderr,
                 "xv_gemm_bf16_noalloc: %d x %d x %d needs %lld bytes of split-K scratch, the built-in buffer "
                 "holds %lld; use xv_gemm_bf16 with a caller-provided workspace\n",
                 m, n, k, pl.workspace_bytes, static_cast<long long>(XV_NOALLOC_SCRATCH_BYTES));
    return XV_ERR_WORKSPACE;
  }
  return gemm_impl(x, w, y, m, n, k, ldx, ldw, ldy, scratch, XV_NOALLOC_SCRATCH_BYTES, sms, status, stream, false,
                   nullptr, 0, nullptr, 1, kPlanNoCluster);
}

}  // extern "C"
