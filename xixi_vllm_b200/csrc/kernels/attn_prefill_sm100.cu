// Paged causal prefill attention for sm_100a on the 5th-generation tensor cores.
//
// A CTA owns 128 query rows of TWO query heads of one KV group of one sequence ("units": same rows,
// same K/V tiles; 256 TMEM columns and one softmax warpgroup each) and walks the sequence's KV pages
// in tiles of 128 tokens (MMAs narrower than N = 128 leave the tensor pipe waiting on operand reads).
// With an odd group size a CTA carries one head. Warps of the two-head form:
//   warps 0-3 / 4-7 - softmax of unit 0 / 1: thread r owns query row r. tcgen05.ld of the S row
//                 (128 fp32), causal mask on diagonal tiles, three-input max, p = 2^(s*scale - m) with a
//                 packed FMA and one MUFU per score, row sum; P rounded to bf16 and written back over the
//                 first 64 S columns (tcgen05.st), where the second MMA reads it as its A operand from
//                 tensor memory (no shared-memory round trip). The output accumulator lives in TMEM
//                 for the whole sequence; it is rescaled in place (tcgen05.ld/st) only when a row's
//                 maximum grows by more than 2^8, otherwise the stale maximum is kept, which the final
//                 division by the row sum makes exact.
//   warps 8, 9  - TMA producers, one for K tiles and one for V tiles (plus the Q tiles once): per tile
//                 the pages named by the block table, each page and 64-column half its own
//                 cp.async.bulk.tensor box (128-byte swizzle), into rings of 32 KiB shared-memory slots
//                 (K: 3, V: 2). Block-table entries are read 32 pages at a time, one batch ahead of use.
//   warps 10, 11 - one MMA issuer thread per unit (warp 10 also owns the TMEM allocation): per tile
//                 O += P V (M=128, N=128, A from TMEM, V read MN-major exactly as the cache stores it)
//                 as soon as that unit's P is ready, then at once the unit's next S = Q K^T (M=128,
//                 N=128) into the same columns. The two issuers run independently (one thread issuing
//                 for both heads spent the whole tile period issuing and waiting), so one head's softmax
//                 runs under the other head's MMAs.
//
// Every barrier wait is bounded; a wait that runs out records a status code, the CTA stops
// issuing work, frees its TMEM and returns.
//
// The reference calls flash_attn_varlen_func (an Ampere-generation mma.sync kernel) here
// (reference: src/compute/layers/attention.py:80-90).

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>
#include <unordered_map>

#include "../common/ptx.cuh"
#include "xv_cuda.h"

namespace {

using namespace xv;

constexpr int kBM = 128;                       // query rows per CTA
constexpr int kBN = 128;                       // KV tokens per tile
constexpr int kD = 128;                        // head dimension
constexpr int kQBytes = kBM * kD * 2;          // 32 KiB, two 64-column halves of 16 KiB
constexpr int kQHalf = kBM * 128;
constexpr int kSlotBytes = kBN * kD * 2;       // 32 KiB, two 64-column halves of 16 KiB
constexpr int kSlotHalf = kBN * 128;
constexpr int kMaxRing = 3;                    // slots per K or V ring
constexpr int kBarBytes = 256;
// The Q tile of every head plus five 32 KiB ring slots (K: 3, V: 2).
constexpr int kSmemRequest1 = kQBytes + 5 * kSlotBytes + kBarBytes;
constexpr int kSmemRequest2 = 2 * kQBytes + 5 * kSlotBytes + kBarBytes;
// TMEM columns of a unit: S (fp32) in [0,128); P (bf16 pairs) overwrites [0,64) once the S row is in
// registers; the output accumulator in [128,256).
constexpr uint32_t kTmemO = 128;
constexpr int kKernelId = 7;
constexpr float kRescaleThreshold = 8.f;       // log2 units

struct Params {
  const int* block_tables;
  const int* cu_q;
  const int* kv_lens;
  __nv_bfloat16* out;
  int seq_begin, hq, hkv, block_size, max_blocks, num_blocks;
  float scale_log2;
  int* status;
  unsigned long long* prof;      // profiling build only: per-phase cycle totals, see kProf* below
};

// Phase counters of the profiling instantiation (cycles summed over CTAs, one observer thread per role).
enum ProfSlot {
  kProfSoftWaitS = 0, kProfSoftLoad, kProfSoftMax, kProfSoftRescale, kProfSoftExp, kProfSoftWaitO, kProfSoftStore,
  kProfSoftEpilogue, kProfMmaWaitK, kProfMmaWaitP, kProfMmaWaitV, kProfMmaIssue, kProfLoadWaitEmpty, kProfLoadIssue,
  kProfCtaTotal, kProfTiles, kProfSetup, kProfRingSlots, kProfSlots
};

template <bool kProfile>
struct PhaseClock {
  long long t0 = 0;
  unsigned long long acc[kProfSlots] = {};
  __device__ __forceinline__ void start() { t0 = clock64(); }
  __device__ __forceinline__ void tick(int slot) {
    const long long t1 = clock64();
    acc[slot] += static_cast<unsigned long long>(t1 - t0);
    t0 = t1;
  }
  __device__ __forceinline__ void flush(unsigned long long* out, int lo, int hi) {
    for (int i = lo; i <= hi; ++i) atomicAdd(&out[i], acc[i]);
  }
};
template <>
struct PhaseClock<false> {
  __device__ __forceinline__ void start() {}
  __device__ __forceinline__ void tick(int) {}
  __device__ __forceinline__ void flush(unsigned long long*, int, int) {}
};

// kUnits = 2: the CTA handles two query heads of one KV group (same rows, same K/V tiles), one
// softmax warpgroup each. kUnits = 1: one head per CTA (odd group sizes; nothing overlaps its softmax).
template <int kUnits, bool kProfile>
__global__ void __launch_bounds__(kUnits * 160 + 64, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr int kProducerWarp = 4 * kUnits, kMmaWarp = 4 * kUnits + 2;    // producers: K warp, V warp; then one MMA warp per unit
  constexpr int kFixedBytes = kUnits * kQBytes;
  constexpr uint32_t kTmemCols = 256 * kUnits;   // per unit: S [0,128) O [128,256)
  const int b = p.seq_begin + blockIdx.z, head0 = blockIdx.y * kUnits;
  const int q_begin = p.cu_q[b];
  const int q_len = p.cu_q[b + 1] - q_begin;
  const int row0 = (static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x)) * kBM;   // long tiles first
  if (row0 >= q_len) return;
  const int kv_len = p.kv_lens[b];
  const int pos0 = kv_len - q_len;                           // absolute position of query row 0
  const int rows_valid = min(kBM, q_len - row0);
  const int n_tiles = (pos0 + row0 + rows_valid - 1) / kBN + 1;
  const int hk = head0 / (p.hq / p.hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  PhaseClock<kProfile> clk;
  const long long cta_t0 = kProfile ? clock64() : 0;
  clk.start();

  // The swizzled tiles need 1024-byte alignment. Whatever shared memory is left after the Q and P
  // tiles becomes K and V ring slots (at most kMaxRing each).
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw & 1023u)) & 1023u;
  uint32_t dyn;
  asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
  int slots = (static_cast<int>(dyn) - static_cast<int>(pad) - kBarBytes - kFixedBytes) / kSlotBytes;
  slots = slots > 2 * kMaxRing ? 2 * kMaxRing : slots;
  const int nv = slots >= 4 ? 2 : 1, nk = slots - nv;
  uint8_t* smem = smem_raw + pad;
  uint8_t* q_s = smem;                                   // [kUnits][2 halves][128 rows][128 B]
  uint8_t* k_ring = q_s + kUnits * kQBytes;
  uint8_t* v_ring = k_ring + nk * kSlotBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(k_ring + slots * kSlotBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;                   // [kMaxRing]
  uint64_t* v_full = k_full + kMaxRing;          // [kMaxRing]
  uint64_t* k_empty = v_full + kMaxRing;         // [kMaxRing]
  uint64_t* v_empty = k_empty + kMaxRing;        // [kMaxRing]
  uint64_t* s_full = v_empty + kMaxRing;         // [kUnits] S written by the MMA
  uint64_t* p_ready = s_full + kUnits;           // [kUnits] P written (and O rescaled) by the softmax warps
  uint64_t* o_done = p_ready + kUnits;           // [kUnits]
  uint64_t* xu_done = o_done + kUnits;           // [kUnits] a unit's exp phase of the tile is over
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xu_done + kUnits);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (nk < 2 || nv < 1) {                        // cannot happen with the launch below; never index past the rings
    if (threadIdx.x == 0) report_status(p.status, kKernelId, kBadIndex);
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kMaxRing; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], kUnits);       // one commit per unit's MMA issuer
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], kUnits);
    }
    for (int u = 0; u < kUnits; ++u) {
      mbar_init(&s_full[u], 1);
      mbar_init(&p_ready[u], 128);
      mbar_init(&o_done[u], 1);
      mbar_init(&xu_done[u], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) clk.tick(kProfSetup);
  if (kProfile && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0)
    p.prof[kProfRingSlots] = static_cast<unsigned long long>(slots);
  clk.start();

  if (warp == kProducerWarp || warp == kProducerWarp + 1) {
    // ---------------- TMA producers: one warp streams the K tiles, the other the V tiles ----------------
    const int is_v = warp - kProducerWarp;
    const uint64_t pol = l2_policy_evict_normal();
    if (lane == 0 && is_v) prefetch_tensormap(&map_v);
    if (lane == 0 && !is_v) {
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_k);
      mbar_expect_tx(q_full, kUnits * kQBytes);
      for (int u = 0; u < kUnits; ++u) {
        tma_load_2d(q_s + u * kQBytes, &map_q, q_full, (head0 + u) * kD, q_begin + row0, pol);
        tma_load_2d(q_s + u * kQBytes + kQHalf, &map_q, q_full, (head0 + u) * kD + 64, q_begin + row0, pol);
      }
    }
    const int bs = p.block_size;
    const int rows_per_load = bs < kBN ? bs : kBN;
    const int loads = kBN / rows_per_load;               // pages per tile (1 when a page holds a whole tile)
    const int last_page = (kv_len - 1) / bs;
    // Block-table entries are fetched 32 pages at a time (lane l holds page 32*batch + l), one batch
    // ahead of use, so the dependent global load never sits between two TMA issues.
    const int* table = p.block_tables + static_cast<long long>(b) * p.max_blocks;
    auto fetch = [&](int batch) { return __ldg(table + min(batch * 32 + lane, last_page)); };
    int cur_batch = 0;
    int cur = fetch(0), nxt = fetch(1);
    const int i = lane >> 1, half = lane & 1;
    uint64_t* full_bars = is_v ? v_full : k_full;
    uint64_t* empty_bars = is_v ? v_empty : k_empty;
    uint8_t* ring = is_v ? v_ring : k_ring;
    const CUtensorMap* map = is_v ? &map_v : &map_k;
    const int depth = is_v ? nv : nk;
    // A K slot frees as soon as the S = Q K^T that read it finishes, a V slot only after the softmax
    // of that tile, so the K warp runs ahead of the V warp by itself.
    for (int j = 0; j < n_tiles; ++j) {
      const int first_pg = min(j * kBN / bs, last_page);
      while ((first_pg >> 5) > cur_batch) {              // warp-uniform
        cur = nxt;
        ++cur_batch;
        nxt = fetch(cur_batch + 1);
      }
      const int tok = j * kBN + (i < loads ? i : 0) * rows_per_load;
      const int pg = min(tok / bs, last_page);           // past the end: any valid page, the columns are masked
      const int from_cur = __shfl_sync(0xffffffffu, cur, pg & 31);
      const int from_nxt = __shfl_sync(0xffffffffu, nxt, pg & 31);
      int blk = (pg >> 5) == cur_batch ? from_cur : from_nxt;
      if (blk < 0 || blk >= p.num_blocks) {
        report_status(p.status, kKernelId, kBadIndex);
        blk = 0;
      }
      const int y = (blk * p.hkv + hk) * bs + (bs > kBN ? tok % bs : 0);
      const int slot = j % depth, use = j / depth;
      int ok = 1;
      if (lane == 0) {
        ok = mbar_wait(&empty_bars[slot], (use & 1) ^ 1) && *abort_flag == 0;
        if (ok) mbar_expect_tx(&full_bars[slot], kSlotBytes);
        if (!is_v) clk.tick(kProfLoadWaitEmpty);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) {
        if (lane == 0) {
          report_status(p.status, kKernelId, kWaitEmptyTimeout);
          *abort_flag = 1;
        }
        break;
      }
      if (lane < 2 * loads) {
        uint8_t* dst = ring + slot * kSlotBytes + half * kSlotHalf + i * rows_per_load * 128;
        tma_load_2d(dst, map, &full_bars[slot], half * 64, y, pol);
      }
      __syncwarp();
      if (lane == 0 && !is_v) clk.tick(kProfLoadIssue);
    }
    if (kProfile && lane == 0 && !is_v) clk.flush(p.prof, kProfLoadWaitEmpty, kProfLoadIssue);
  } else if (warp >= kMmaWarp && warp < kMmaWarp + kUnits) {
    // ---------------- MMA issuers: one thread per unit ----------------
    // Per tile: O_u += P_u(j) V(j) as soon as the unit's softmax warps have written P (over the S
    // columns), then at once S_u(j+1) = Q_u K(j+1)^T into the same columns; the tensor pipe runs a
    // thread's MMAs in issue order. The units run independently, so one head's softmax overlaps the
    // other head's MMAs; a K or V slot is free when both issuers have committed it.
    const int u = warp - kMmaWarp;
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc_bf16(kBM, kBN);
      const uint32_t idesc_o = umma_idesc_bf16_b_mn(kBM, kD);
      const uint32_t q_addr = smem_u32(q_s) + u * kQBytes;
      const uint32_t k_ring_addr = smem_u32(k_ring), v_ring_addr = smem_u32(v_ring);
      const uint32_t s_tmem = tmem_base + u * 256, o_tmem = s_tmem + kTmemO;
      bool ok = mbar_wait(q_full, 0);
      int reason = kWaitFullTimeout;
      auto issue_s = [&](int j) -> bool {
        const int slot = j % nk;
        if (!mbar_wait(&k_full[slot], (j / nk) & 1)) return false;
        if (u == 0) clk.tick(kProfMmaWaitK);
        tc_fence_after_sync();
        const uint32_t k_addr = k_ring_addr + slot * kSlotBytes;
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks) {
          const uint64_t a = umma_desc_sw128(q_addr + (ks >> 2) * kQHalf + (ks & 3) * 32);
          const uint64_t bd = umma_desc_sw128(k_addr + (ks >> 2) * kSlotHalf + (ks & 3) * 32);
          umma_bf16(s_tmem, a, bd, idesc_s, ks > 0);
        }
        umma_commit(&s_full[u]);
        umma_commit(&k_empty[slot]);
        if (u == 0) clk.tick(kProfMmaIssue);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (!mbar_wait(&p_ready[u], j & 1)) { ok = false; reason = kWaitAccumTimeout; break; }
        if (u == 0) clk.tick(kProfMmaWaitP);
        const int vslot = j % nv;
        if (!mbar_wait(&v_full[vslot], (j / nv) & 1)) { ok = false; break; }
        if (u == 0) clk.tick(kProfMmaWaitV);
        tc_fence_after_sync();
        const uint32_t v_addr = v_ring_addr + vslot * kSlotBytes;
#pragma unroll
        for (int ks = 0; ks < kBN / 16; ++ks) {
          const uint64_t bd = umma_desc_sw128_mn(v_addr + ks * 2048, kSlotHalf, 1024);
          umma_bf16_a_tmem(o_tmem, s_tmem + ks * 8, bd, idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&o_done[u]);
        umma_commit(&v_empty[vslot]);
        if (u == 0) clk.tick(kProfMmaIssue);
        if (j + 1 < n_tiles && !issue_s(j + 1)) ok = false;
      }
      if (kProfile && u == 0) clk.flush(p.prof, kProfMmaWaitK, kProfMmaIssue);
      if (!ok || *abort_flag) {
        if (!ok) report_status(p.status, kKernelId, reason);
        *abort_flag = 1;
      }
    }
  } else {
    // ---------------- softmax + epilogue: thread r of unit u owns query row r of head head0 + u ----------------
    const int u = warp >> 2;
    const int r = threadIdx.x & 127;
    const int head = head0 + u;
    const int pos_row = pos0 + row0 + (r < rows_valid ? r : rows_valid - 1);
    const uint32_t lane_taddr = tmem_base + u * 256 + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    uint64_t* my_s_full = &s_full[u];
    uint64_t* my_p_ready = &p_ready[u];
    uint64_t* my_o_done = &o_done[u];
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(my_s_full, j & 1) && *abort_flag == 0);
      if (!ok) break;
      clk.tick(kProfSoftWaitS);
      tc_fence_after_sync();
      uint32_t sr[8][16];                          // the whole score row: 128 fp32
#pragma unroll
      for (int c = 0; c < 8; ++c) tmem_ld16(lane_taddr + c * 16, sr[c]);
      tmem_ld_wait();
      clk.tick(kProfSoftLoad);
      const int k0 = j * kBN;
      if (k0 + kBN - 1 > pos_row) {              // only tiles that cross the diagonal mask anything
#pragma unroll
        for (int c = 0; c < 8; ++c)
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (k0 + c * 16 + i > pos_row) sr[c][i] = 0xff800000u;      // -inf
      }
      // Row maximum of the raw scores (the scale is positive, so it commutes with max).
      float mx[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float a0 = fmax3(__uint_as_float(sr[c][0]), __uint_as_float(sr[c][1]), __uint_as_float(sr[c][2]));
        const float a1 = fmax3(__uint_as_float(sr[c][3]), __uint_as_float(sr[c][4]), __uint_as_float(sr[c][5]));
        const float a2 = fmax3(__uint_as_float(sr[c][6]), __uint_as_float(sr[c][7]), __uint_as_float(sr[c][8]));
        const float a3 = fmax3(__uint_as_float(sr[c][9]), __uint_as_float(sr[c][10]), __uint_as_float(sr[c][11]));
        const float a4 = fmax3(__uint_as_float(sr[c][12]), __uint_as_float(sr[c][13]), __uint_as_float(sr[c][14]));
        mx[c] = fmax3(fmax3(a0, a1, a2), fmax3(a3, a4, __uint_as_float(sr[c][15])), -INFINITY);
      }
      const float mt = fmax3(fmax3(mx[0], mx[1], mx[2]), fmax3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7])) *
                       p.scale_log2;
      clk.tick(kProfSoftMax);
      if (j == 0) {
        m = mt;                                  // column 0 is never masked, so this is finite
      } else {
        const bool need = mt > m + kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          ok = __all_sync(0xffffffffu, mbar_wait(my_o_done, (j - 1) & 1));
          if (!ok) break;
          tc_fence_after_sync();
          const float m_new = need ? mt : m;
          const float alpha = exp2f(m - m_new);
          l *= alpha;
          m = m_new;
          const uint64_t alpha2 = pack_f32x2(alpha, alpha);
#pragma unroll 1
          for (int ch = 0; ch < kD / 16; ++ch) {
            uint32_t o[16];
            tmem_ld16(lane_taddr + kTmemO + ch * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              float lo, hi;
              unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(o[i]), __uint_as_float(o[i + 1])), alpha2), lo, hi);
              o[i] = __float_as_uint(lo);
              o[i + 1] = __float_as_uint(hi);
            }
            tmem_st16(lane_taddr + kTmemO + ch * 16, o);
          }
          tmem_st_wait();
        }
      }
      clk.tick(kProfSoftRescale);
      // The two units take turns on the MUFU pipe (unit 0 tile j, unit 1 tile j, unit 0 tile j+1, ...):
      // run together, both exp phases take twice as long and nothing overlaps the rest of either chain.
      if (kUnits == 2 && (u == 1 || j > 0)) {
        ok = __all_sync(0xffffffffu, u == 1 ? mbar_wait(&xu_done[0], j & 1) : mbar_wait(&xu_done[1], (j - 1) & 1));
        if (!ok) break;
      }
      clk.tick(kProfSoftWaitO);
      // p = 2^(s * scale - m): one packed FMA per two scores, one MUFU each, four independent sums. P goes
      // back to tensor memory as bf16 pairs over the first 64 columns of S (this thread's own lane), where
      // the second MMA reads it as its A operand.
      const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2), negm2 = pack_f32x2(-m, -m);
      float sums[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 8; c += 2) {
        uint32_t packed[16];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            float x0, x1;
            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sr[c + h][i]), __uint_as_float(sr[c + h][i + 1])),
                                   scale2, negm2),
                         x0, x1);
            const float p0 = exp2f(x0), p1 = exp2f(x1);
            sums[(i >> 1) & 3] += p0 + p1;
            packed[h * 8 + (i >> 1)] = pack_bf16(p0, p1);
          }
        tmem_st16(lane_taddr + (c >> 1) * 16, packed);   // scores 16c .. 16c+31 -> P columns 8c .. 8c+15
      }
      l += (sums[0] + sums[1]) + (sums[2] + sums[3]);
      if (kUnits == 2) mbar_arrive(&xu_done[u]);
      clk.tick(kProfSoftExp);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(my_p_ready);
      clk.tick(kProfSoftStore);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(my_o_done, (n_tiles - 1) & 1) && *abort_flag == 0);
    if (ok) {
      tc_fence_after_sync();
      const float inv = 1.f / l;
      __nv_bfloat16* orow =
          p.out + (static_cast<long long>(q_begin + row0 + r) * p.hq + head) * kD;
#pragma unroll 1
      for (int ch = 0; ch < kD / 16; ++ch) {
        uint32_t o[16];
        tmem_ld16(lane_taddr + kTmemO + ch * 16, o);
        tmem_ld_wait();
        if (r < rows_valid) {
          uint4 v0, v1;
          v0.x = pack_bf16(__uint_as_float(o[0]) * inv, __uint_as_float(o[1]) * inv);
          v0.y = pack_bf16(__uint_as_float(o[2]) * inv, __uint_as_float(o[3]) * inv);
          v0.z = pack_bf16(__uint_as_float(o[4]) * inv, __uint_as_float(o[5]) * inv);
          v0.w = pack_bf16(__uint_as_float(o[6]) * inv, __uint_as_float(o[7]) * inv);
          v1.x = pack_bf16(__uint_as_float(o[8]) * inv, __uint_as_float(o[9]) * inv);
          v1.y = pack_bf16(__uint_as_float(o[10]) * inv, __uint_as_float(o[11]) * inv);
          v1.z = pack_bf16(__uint_as_float(o[12]) * inv, __uint_as_float(o[13]) * inv);
          v1.w = pack_bf16(__uint_as_float(o[14]) * inv, __uint_as_float(o[15]) * inv);
          *reinterpret_cast<uint4*>(orow + ch * 16) = v0;
          *reinterpret_cast<uint4*>(orow + ch * 16 + 8) = v1;
        }
      }
    } else if (lane == 0) {
      report_status(p.status, kKernelId, kWaitAccumTimeout);
      *abort_flag = 1;
    }
    clk.tick(kProfSoftEpilogue);
    if (kProfile && threadIdx.x == 0) {
      clk.flush(p.prof, kProfSoftWaitS, kProfSoftEpilogue);
      atomicAdd(&p.prof[kProfTiles], static_cast<unsigned long long>(n_tiles));
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (kProfile && threadIdx.x == 0)
    atomicAdd(&p.prof[kProfCtaTotal], static_cast<unsigned long long>(clock64() - cta_t0));
}

// ---- host side ----------------------------------------------------------------------------------

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(ptr);
  });
  return fn;
}

struct Key {
  const void* ptr;
  long long rows, cols;
  int box_rows;
  bool operator==(const Key& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows;
  }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr) * 0x9E3779B97F4A7C15ULL;
    h ^= static_cast<size_t>(k.rows) * 0xC2B2AE3D27D4EB4FULL + (h << 6) + (h >> 2);
    h ^= static_cast<size_t>(k.cols * 131 + k.box_rows) + (h << 6) + (h >> 2);
    return h;
  }
};

// Row-major bf16 [rows, cols] viewed through boxes of 64 columns x box_rows rows, 128-byte swizzle.
// Cached: the KV cache and the activation arena keep their addresses.
int tensor_map(CUtensorMap* out, const void* ptr, long long rows, long long cols, int box_rows) {
  static std::unordered_map<Key, CUtensorMap, KeyHash> cache;
  static std::mutex mu;
  const Key key{ptr, rows, cols, box_rows};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  EncodeFn enc = encode_fn();
  if (!enc) return XV_ERR_DRIVER;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  if (enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return XV_ERR_TENSORMAP;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

}  // namespace

static int g_force_single_unit = 0;

extern "C" {

// 1: always one head per CTA (for comparing the two forms); 0: pair heads of a KV group when possible.
void xv_attn_prefill_tc_single_unit(int on) { g_force_single_unit = on; }

int xv_attn_prefill_tc_supported(int d, int block_size) {
  if (d != kD || block_size <= 0 || block_size % 16) return 0;
  return (block_size <= kBN ? kBN % block_size == 0 : block_size % kBN == 0) ? 1 : 0;
}

static int launch_prefill_tc(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                       const int* cu_q, const int* kv_lens, void* out, int seq_begin, int num_seqs, int max_q_len,
                       int total_tokens, int num_blocks, int hq, int hkv, int d, int block_size, int max_blocks,
                       float scale, int* status, unsigned long long* prof, cudaStream_t stream) {
  if (num_seqs <= 0 || max_q_len <= 0) return 0;
  if (!xv_attn_prefill_tc_supported(d, block_size)) return XV_ERR_UNSUPPORTED;
  if (hq % hkv || total_tokens <= 0 || num_blocks <= 0) return XV_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return XV_ERR_SHAPE;
  static bool attr = false;
  if (!attr) {
    const auto at = cudaFuncAttributeMaxDynamicSharedMemorySize;
    if (cudaFuncSetAttribute(attn_prefill_tc_kernel<1, false>, at, kSmemRequest1) != cudaSuccess ||
        cudaFuncSetAttribute(attn_prefill_tc_kernel<1, true>, at, kSmemRequest1) != cudaSuccess ||
        cudaFuncSetAttribute(attn_prefill_tc_kernel<2, false>, at, kSmemRequest2) != cudaSuccess ||
        cudaFuncSetAttribute(attn_prefill_tc_kernel<2, true>, at, kSmemRequest2) != cudaSuccess)
      return XV_ERR_LAUNCH;
    attr = true;
  }
  CUtensorMap map_q, map_k, map_v;
  const long long kv_rows = static_cast<long long>(num_blocks) * hkv * block_size;
  const int box_rows = block_size < kBN ? block_size : kBN;
  if (int rc = tensor_map(&map_q, q, total_tokens, static_cast<long long>(hq) * kD, kBM)) return rc;
  if (int rc = tensor_map(&map_k, k_cache, kv_rows, kD, box_rows)) return rc;
  if (int rc = tensor_map(&map_v, v_cache, kv_rows, kD, box_rows)) return rc;
  Params p;
  p.block_tables = block_tables;
  p.cu_q = cu_q;
  p.kv_lens = kv_lens;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.seq_begin = seq_begin; p.hq = hq; p.hkv = hkv; p.block_size = block_size; p.max_blocks = max_blocks;
  p.num_blocks = num_blocks;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.prof = prof;
  // Two heads of a KV group per CTA whenever the group size is even: K/V tiles are fetched once for both.
  const int units = ((hq / hkv) % 2 == 0 && g_force_single_unit == 0) ? 2 : 1;
  dim3 grid((max_q_len + kBM - 1) / kBM, hq / units, num_seqs);
  if (units == 2) {
    if (prof)
      attn_prefill_tc_kernel<2, true><<<grid, 384, kSmemRequest2, stream>>>(map_q, map_k, map_v, p);
    else
      attn_prefill_tc_kernel<2, false><<<grid, 384, kSmemRequest2, stream>>>(map_q, map_k, map_v, p);
  } else {
    if (prof)
      attn_prefill_tc_kernel<1, true><<<grid, 224, kSmemRequest1, stream>>>(map_q, map_k, map_v, p);
    else
      attn_prefill_tc_kernel<1, false><<<grid, 224, kSmemRequest1, stream>>>(map_q, map_k, map_v, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : XV_ERR_LAUNCH;
}

int xv_attn_prefill_tc(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                       const int* cu_q, const int* kv_lens, void* out, int seq_begin, int num_seqs, int max_q_len,
                       int total_tokens, int num_blocks, int hq, int hkv, int d, int block_size, int max_blocks,
                       float scale, int* status, cudaStream_t stream) {
  return launch_prefill_tc(q, k_cache, v_cache, block_tables, cu_q, kv_lens, out, seq_begin, num_seqs, max_q_len,
                           total_tokens, num_blocks, hq, hkv, d, block_size, max_blocks, scale, status, nullptr, stream);
}

// Same launch with per-phase cycle counters: `prof` points to xv_attn_prefill_tc_profile_slots() zeroed
// 64-bit device counters that the kernel adds to (softmax, MMA-issue and load warps: time waiting vs working).
int xv_attn_prefill_tc_profile_slots(void) { return kProfSlots; }
int xv_attn_prefill_tc_profile(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                               const int* cu_q, const int* kv_lens, void* out, int seq_begin, int num_seqs,
                               int max_q_len, int total_tokens, int num_blocks, int hq, int hkv, int d, int block_size,
                               int max_blocks, float scale, int* status, unsigned long long* prof,
                               cudaStream_t stream) {
  if (!prof) return XV_ERR_SHAPE;
  return launch_prefill_tc(q, k_cache, v_cache, block_tables, cu_q, kv_lens, out, seq_begin, num_seqs, max_q_len,
                           total_tokens, num_blocks, hq, hkv, d, block_size, max_blocks, scale, status, prof, stream);
}

}  // extern "C"
