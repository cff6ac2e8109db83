// Paged-KV attention for head_dim 128, GQA, pages of 16 tokens (or multiples), causal.
//
//   attn_decode_kernel  - one query row per sequence. A CTA owns (sequence, KV head, KV split);
//                         the GQA group's query heads are stacked as the M rows of the MMA, so
//                         one pass over a KV page serves the whole group. Each of the 4 warps
//                         streams its own pages through a private 3-stage cp.async ring (no
//                         block-wide barriers in the main loop), keeps an online-softmax state,
//                         and the warps are merged through shared memory at the end. With
//                         several KV splits the partial outputs and log-sum-exps go to a
//                         workspace that attn_combine_kernel reduces.
//   attn_prefill_kernel - packed varlen queries; a CTA owns 64 query rows of one head, 4 warps
//                         x 16 rows, and walks the KV in 64-token tiles (4 pages) with double
//                         buffering; sequences with a cached prefix simply have kv_len > q_len.
//
// Matrix products use mma.sync m16n8k16 (bf16 in, fp32 out) with ldmatrix from XOR-swizzled
// shared memory. KV cache layout: [blocks, kv_heads, block_size, 128] per layer, so a page of
// one head is a contiguous 4 KiB run.
//
// The reference calls flash-attn 2 for both phases and needs 256-token pages for it
// (reference: src/compute/layers/attention.py:43-100).

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "xv_cuda.h"

namespace xv {

constexpr int kD = 128;               // head_dim
constexpr int kRowBytes = kD * 2;     // 256 B per token row
constexpr int kTile = 16;             // tokens per decode tile (= smallest page)
constexpr int kTileBytes = kTile * kRowBytes;   // 4 KiB
constexpr float kLog2e = 1.4426950408889634f;

// Byte offset of 16-byte chunk c of row r inside a swizzled tile with 256-byte rows.
__device__ __forceinline__ uint32_t swz(int r, int c) {
  return static_cast<uint32_t>(r * kRowBytes + ((c ^ (r & 7)) << 4));
}

// ------------------------------------------------------------------------------------------
// Decode
// ------------------------------------------------------------------------------------------
constexpr int kDecWarps = 4;
constexpr int kDecStages = 3;
constexpr int kDecSmem = kDecWarps * kDecStages * 2 * kTileBytes;   // 96 KiB

struct DecodeParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* block_tables;
  const int* kv_lens;
  __nv_bfloat16* out;
  float* ws_o;      // [seq, hq, split, 128]
  float* ws_lse;    // [seq, hq, split]
  int hq, hkv, block_size, max_blocks, splits;
  float scale_log2;
};

__global__ void __launch_bounds__(kDecWarps * 32, 2) attn_decode_kernel(const DecodeParams p) {
  grid_dep_launch();
  grid_dep_wait();
  extern __shared__ __align__(128) uint8_t smem[];
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int G = p.hq / p.hkv;
  const int kv_len = p.kv_lens[b];
  const int tiles_total = (kv_len + kTile - 1) / kTile;
  const int tiles_per_split = (tiles_total + p.splits - 1) / p.splits;
  const int tile0 = split * tiles_per_split;
  int tile1 = tile0 + tiles_per_split;
  if (tile1 > tiles_total) tile1 = tiles_total;
  const int n_tiles = tile1 > tile0 ? tile1 - tile0 : 0;
  const int tiles_per_block = p.block_size / kTile;

  // Q fragments: rows = query heads of this KV group (zero beyond G).
  uint32_t qf[8][4];
  {
    const __nv_bfloat16* qb = p.q + static_cast<size_t>(b) * p.hq * kD + static_cast<size_t>(h) * G * kD;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const int d0 = kk * 16 + t * 2;
      qf[kk][0] = g < G ? *reinterpret_cast<const uint32_t*>(qb + g * kD + d0) : 0u;
      qf[kk][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + (g + 8) * kD + d0) : 0u;
      qf[kk][2] = g < G ? *reinterpret_cast<const uint32_t*>(qb + g * kD + d0 + 8) : 0u;
      qf[kk][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + (g + 8) * kD + d0 + 8) : 0u;
    }
  }

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;

  uint8_t* ring = smem + static_cast<size_t>(warp) * kDecStages * 2 * kTileBytes;
  const int my_tiles = n_tiles > warp ? (n_tiles - warp + kDecWarps - 1) / kDecWarps : 0;

  auto issue = [&](int i) {   // i-th tile of this warp
    if (i < my_tiles) {
      const int tt = tile0 + warp + i * kDecWarps;
      const int blk = p.block_tables[static_cast<size_t>(b) * p.max_blocks + tt / tiles_per_block];
      const size_t base = ((static_cast<size_t>(blk) * p.hkv + h) * p.block_size +
                           static_cast<size_t>(tt % tiles_per_block) * kTile) * kD;
      const uint8_t* ks = reinterpret_cast<const uint8_t*>(p.k_cache + base);
      const uint8_t* vs = reinterpret_cast<const uint8_t*>(p.v_cache + base);
      uint8_t* kd = ring + static_cast<size_t>(i % kDecStages) * 2 * kTileBytes;
      uint8_t* vd = kd + kTileBytes;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = lane + 32 * j;          // chunk id in the page: row c/16, chunk c%16
        cp_async16(kd + swz(c >> 4, c & 15), ks + c * 16);
        // V rows past the end of the sequence are zero-filled: their probabilities are zero, but whatever an
        // earlier owner of the page left there (possibly NaN) must not reach the product. K rows only feed
        // scores that are masked afterwards.
        cp_async16_zfill(vd + swz(c >> 4, c & 15), vs + c * 16, tt * kTile + (c >> 4) < kv_len);
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int i = 0; i < kDecStages - 1; ++i) issue(i);

  for (int i = 0; i < my_tiles; ++i) {
    issue(i + kDecStages - 1);
    cp_async_wait<kDecStages - 1>();
    __syncwarp();
    const uint32_t kb = smem_u32(ring + static_cast<size_t>(i % kDecStages) * 2 * kTileBytes);
    const uint32_t vb = kb + kTileBytes;
    const int tok0 = (tile0 + warp + i * kDecWarps) * kTile;

    // S = Q K^T for 16 tokens: two 8-token column tiles
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const int mi = lane >> 3;
      const int r = ((mi >> 1) << 3) + (lane & 7);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        uint32_t kf[4];
        ldmatrix_x4(kf, kb + swz(r, 2 * kk + (mi & 1)));
        mma_bf16_16816(s0, qf[kk], kf[0], kf[1]);
        mma_bf16_16816(s1, qf[kk], kf[2], kf[3]);
      }
    }
    // scale, mask tokens past the end, online softmax for rows g and g+8
    const int c0 = tok0 + 2 * t;
    float v[8] = {s0[0], s0[1], s1[0], s1[1], s0[2], s0[3], s1[2], s1[3]};   // row g: 0..3, row g+8: 4..7
    const int col[4] = {c0, c0 + 1, c0 + 8, c0 + 9};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool ok = col[j] < kv_len;
      v[j] = ok ? v[j] * p.scale_log2 : -CUDART_INF_F;
      v[4 + j] = ok ? v[4 + j] * p.scale_log2 : -CUDART_INF_F;
    }
    float mx0 = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
    float mx1 = fmaxf(fmaxf(v[4], v[5]), fmaxf(v[6], v[7]));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float base0 = mn0 == -CUDART_INF_F ? 0.f : mn0, base1 = mn1 == -CUDART_INF_F ? 0.f : mn1;
    const float cr0 = exp2f(m0 - base0), cr1 = exp2f(m1 - base1);   // m == -inf gives 0
    m0 = mn0;
    m1 = mn1;
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[j] = exp2f(v[j] - base0);
      v[4 + j] = exp2f(v[4 + j] - base1);
      ps0 += v[j];
      ps1 += v[4 + j];
    }
    l0 = l0 * cr0 + ps0;
    l1 = l1 * cr1 + ps1;
#pragma unroll
    for (int i2 = 0; i2 < 16; ++i2) {
      o[i2][0] *= cr0; o[i2][1] *= cr0; o[i2][2] *= cr1; o[i2][3] *= cr1;
    }
    uint32_t pf[4];
    pf[0] = pack_bf16(v[0], v[1]);   // row g,   tokens 2t, 2t+1
    pf[1] = pack_bf16(v[4], v[5]);   // row g+8
    pf[2] = pack_bf16(v[2], v[3]);   // row g,   tokens 8+2t, 9+2t
    pf[3] = pack_bf16(v[6], v[7]);   // row g+8
    // O += P V
    {
      const int mi = lane >> 3;
      const int r = ((mi & 1) << 3) + (lane & 7);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t vf[4];
        ldmatrix_x4_trans(vf, vb + swz(r, 2 * j + (mi >> 1)));
        mma_bf16_16816(o[2 * j], pf, vf[0], vf[1]);
        mma_bf16_16816(o[2 * j + 1], pf, vf[2], vf[3]);
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();

  // quad-reduce the row sums
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

  // merge the warps through shared memory (the rings are idle now)
  __syncthreads();
  float* mo = reinterpret_cast<float*>(smem);                 // [warp][16][128]
  float* mm = mo + kDecWarps * 16 * kD;                       // [warp][16]
  float* ml = mm + kDecWarps * 16;                            // [warp][16]
  {
    float* wo = mo + warp * 16 * kD;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      const int d0 = nt * 8 + 2 * t;
      *reinterpret_cast<float2*>(wo + g * kD + d0) = make_float2(o[nt][0], o[nt][1]);
      *reinterpret_cast<float2*>(wo + (g + 8) * kD + d0) = make_float2(o[nt][2], o[nt][3]);
    }
    if (t == 0) {
      mm[warp * 16 + g] = m0;
      mm[warp * 16 + g + 8] = m1;
      ml[warp * 16 + g] = l0;
      ml[warp * 16 + g + 8] = l1;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * kD; idx += blockDim.x) {
    const int r = idx / kD, d = idx - r * kD;
    float M = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, mm[w * 16 + r]);
    float L = 0.f, acc = 0.f;
    if (M != -CUDART_INF_F) {
#pragma unroll
      for (int w = 0; w < kDecWarps; ++w) {
        const float sc = exp2f(mm[w * 16 + r] - M);
        L += ml[w * 16 + r] * sc;
        acc += mo[(w * 16 + r) * kD + d] * sc;
      }
    }
    const float val = L > 0.f ? acc / L : 0.f;
    const int head = h * G + r;
    if (p.splits == 1) {
      p.out[(static_cast<size_t>(b) * p.hq + head) * kD + d] = __float2bfloat16(val);
    } else {
      const size_t wi = (static_cast<size_t>(b) * p.hq + head) * p.splits + split;
      p.ws_o[wi * kD + d] = val;
      if (d == 0) p.ws_lse[wi] = L > 0.f ? M + log2f(L) : -CUDART_INF_F;
    }
  }
}

// out[seq, head, :] = sum_s w_s * O_s with w_s = 2^(lse_s - max) / sum.
__global__ void attn_combine_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_lse,
                                    __nv_bfloat16* __restrict__ out, int splits) {
  grid_dep_launch();
  grid_dep_wait();
  const size_t row = blockIdx.x;      // seq * hq + head
  const int d = threadIdx.x;
  float M = -CUDART_INF_F;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, ws_lse[row * splits + s]);
  float L = 0.f, acc = 0.f;
  if (M != -CUDART_INF_F) {
    for (int s = 0; s < splits; ++s) {
      const float w = exp2f(ws_lse[row * splits + s] - M);
      L += w;
      acc += w * ws_o[(row * splits + s) * kD + d];
    }
  }
  out[row * kD + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
}

// ------------------------------------------------------------------------------------------
// Prefill
// ------------------------------------------------------------------------------------------
constexpr int kPfBM = 64, kPfBN = 64, kPfWarps = 4;
constexpr int kPfTileBytes = kPfBN * kRowBytes;                     // 16 KiB
constexpr int kPfSmem = kPfBM * kRowBytes + 4 * kPfTileBytes;       // Q + 2 x (K, V) = 80 KiB

struct PrefillParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* block_tables;
  const int* cu_q;
  const int* kv_lens;
  __nv_bfloat16* out;
  int seq_begin, hq, hkv, block_size, max_blocks;
  float scale_log2;
};

__global__ void __launch_bounds__(kPfWarps * 32, 2) attn_prefill_kernel(const PrefillParams p) {
  grid_dep_launch();
  grid_dep_wait();
  extern __shared__ __align__(128) uint8_t smem[];
  const int qt = blockIdx.x, head = blockIdx.y, b = p.seq_begin + blockIdx.z;
  const int q_begin = p.cu_q[b];
  const int q_len = p.cu_q[b + 1] - q_begin;
  const int row0 = qt * kPfBM;
  if (row0 >= q_len) return;
  const int kv_len = p.kv_lens[b];
  const int pos0 = kv_len - q_len;                    // absolute position of query row 0
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int hk = head / (p.hq / p.hkv);
  const int rows_here = min(kPfBM, q_len - row0);
  const int last_pos = pos0 + row0 + rows_here - 1;
  const int n_kv = min(kv_len, last_pos + 1);
  const int n_tiles = (n_kv + kPfBN - 1) / kPfBN;
  const int tiles_per_block = p.block_size / kTile;

  uint8_t* sq = smem;
  uint8_t* skv = smem + kPfBM * kRowBytes;

  // Q tile -> shared (rows past the sequence end are zero-filled)
  {
    const size_t ld = static_cast<size_t>(p.hq) * kD;
    const __nv_bfloat16* qb = p.q + (static_cast<size_t>(q_begin) + row0) * ld + static_cast<size_t>(head) * kD;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = threadIdx.x + 128 * j;     // 1024 chunks: row c/16, chunk c%16
      const int r = c >> 4, ch = c & 15;
      const bool ok = r < rows_here;
      cp_async16_zfill(sq + swz(r, ch), qb + (ok ? static_cast<size_t>(r) * ld + ch * 8 : 0), ok);
    }
  }
  auto issue_kv = [&](int j) {
    if (j < n_tiles) {
      uint8_t* kd = skv + static_cast<size_t>(j & 1) * 2 * kPfTileBytes;
      uint8_t* vd = kd + kPfTileBytes;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = threadIdx.x + 128 * i;   // row c/16 of the 64-token tile
        const int r = c >> 4, ch = c & 15;
        const int tok = j * kPfBN + r;
        const bool ok = tok < n_kv;
        const int tt = (ok ? tok : 0) / kTile;
        const int blk = p.block_tables[static_cast<size_t>(b) * p.max_blocks + tt / tiles_per_block];
        const size_t off = ((static_cast<size_t>(blk) * p.hkv + hk) * p.block_size +
                            static_cast<size_t>(tt % tiles_per_block) * kTile + (tok & (kTile - 1))) * kD + ch * 8;
        cp_async16_zfill(kd + swz(r, ch), p.k_cache + (ok ? off : 0), ok);
        cp_async16_zfill(vd + swz(r, ch), p.v_cache + (ok ? off : 0), ok);
      }
    }
    cp_async_commit();
  };
  issue_kv(0);          // group 0 also carries the Q loads

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
  uint32_t qf[8][4];
  const int my_pos0 = pos0 + row0 + warp * 16 + g;     // position of row g; row g+8 is +8

  for (int j = 0; j < n_tiles; ++j) {
    issue_kv(j + 1);
    cp_async_wait<1>();
    __syncthreads();
    if (j == 0) {
      const int mi = lane >> 3;
      const int r = warp * 16 + ((mi & 1) << 3) + (lane & 7);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) ldmatrix_x4(qf[kk], smem_u32(sq) + swz(r, 2 * kk + (mi >> 1)));
    }
    const uint32_t kb = smem_u32(skv + static_cast<size_t>(j & 1) * 2 * kPfTileBytes);
    const uint32_t vb = kb + kPfTileBytes;
    // warps whose rows all sit before this tile's first key still run it (keys <= position);
    // tiles entirely after a warp's last row are skipped
    const int tile_k0 = j * kPfBN;
    const bool warp_active = tile_k0 <= my_pos0 - g + 15;
    if (warp_active) {
      float s[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      {
        const int mi = lane >> 3;
        const int r = ((mi >> 1) << 3) + (lane & 7);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
          for (int jp = 0; jp < 4; ++jp) {
            uint32_t kf[4];
            ldmatrix_x4(kf, kb + swz(jp * 16 + r, 2 * kk + (mi & 1)));
            mma_bf16_16816(s[2 * jp], qf[kk], kf[0], kf[1]);
            mma_bf16_16816(s[2 * jp + 1], qf[kk], kf[2], kf[3]);
          }
        }
      }
      float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = tile_k0 + nt * 8 + 2 * t + e;
          const bool in = key < n_kv;
          s[nt][e] = (in && key <= my_pos0) ? s[nt][e] * p.scale_log2 : -CUDART_INF_F;
          s[nt][2 + e] = (in && key <= my_pos0 + 8) ? s[nt][2 + e] * p.scale_log2 : -CUDART_INF_F;
          mx0 = fmaxf(mx0, s[nt][e]);
          mx1 = fmaxf(mx1, s[nt][2 + e]);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float base0 = mn0 == -CUDART_INF_F ? 0.f : mn0, base1 = mn1 == -CUDART_INF_F ? 0.f : mn1;
      const float cr0 = exp2f(m0 - base0), cr1 = exp2f(m1 - base1);
      m0 = mn0;
      m1 = mn1;
      float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        s[nt][0] = exp2f(s[nt][0] - base0);
        s[nt][1] = exp2f(s[nt][1] - base0);
        s[nt][2] = exp2f(s[nt][2] - base1);
        s[nt][3] = exp2f(s[nt][3] - base1);
        ps0 += s[nt][0] + s[nt][1];
        ps1 += s[nt][2] + s[nt][3];
      }
      l0 = l0 * cr0 + ps0;
      l1 = l1 * cr1 + ps1;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        o[i][0] *= cr0; o[i][1] *= cr0; o[i][2] *= cr1; o[i][3] *= cr1;
      }
      {
        const int mi = lane >> 3;
        const int r = ((mi & 1) << 3) + (lane & 7);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          uint32_t pf[4];
          pf[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
          pf[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
          pf[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
          pf[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
          for (int jd = 0; jd < 8; ++jd) {
            uint32_t vf[4];
            ldmatrix_x4_trans(vf, vb + swz(ks * 16 + r, 2 * jd + (mi >> 1)));
            mma_bf16_16816(o[2 * jd], pf, vf[0], vf[1]);
            mma_bf16_16816(o[2 * jd + 1], pf, vf[2], vf[3]);
          }
        }
      }
    }
    __syncthreads();    // everyone is done with buffer j&1 before tile j+2 overwrites it
  }
  cp_async_wait<0>();

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int r0 = row0 + warp * 16 + g, r1 = r0 + 8;
  const size_t ld = static_cast<size_t>(p.hq) * kD;
  __nv_bfloat16* ob = p.out + static_cast<size_t>(q_begin) * ld + static_cast<size_t>(head) * kD;
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
    const int d0 = nt * 8 + 2 * t;
    if (r0 < q_len)
      *reinterpret_cast<uint32_t*>(ob + static_cast<size_t>(r0) * ld + d0) = pack_bf16(o[nt][0] * inv0, o[nt][1] * inv0);
    if (r1 < q_len)
      *reinterpret_cast<uint32_t*>(ob + static_cast<size_t>(r1) * ld + d0) = pack_bf16(o[nt][2] * inv1, o[nt][3] * inv1);
  }
}

}  // namespace xv

using namespace xv;

extern "C" {

long long xv_attn_decode_workspace_bytes(int num_seqs, int hq, int d, int splits) {
  if (splits <= 1) return 0;
  return static_cast<long long>(num_seqs) * hq * splits * (d + 1) * 4;
}

int xv_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                   const int* kv_lens, void* out, int num_seqs, int hq, int hkv, int d, int block_size,
                   int max_blocks, float scale, int splits, void* workspace, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (d != kD) return XV_ERR_UNSUPPORTED;
  if (block_size % kTile || hq % hkv || hq / hkv > 16 || splits < 1) return XV_ERR_SHAPE;
  if (splits > 1 && !workspace) return XV_ERR_WORKSPACE;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmem) != cudaSuccess)
      return XV_ERR_LAUNCH;
    attr = true;
  }
  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.block_tables = block_tables;
  p.kv_lens = kv_lens;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ws_o = static_cast<float*>(workspace);
  p.ws_lse = p.ws_o ? p.ws_o + static_cast<size_t>(num_seqs) * hq * splits * kD : nullptr;
  p.hq = hq; p.hkv = hkv; p.block_size = block_size; p.max_blocks = max_blocks; p.splits = splits;
  p.scale_log2 = scale * kLog2e;
  dim3 grid(splits, hkv, num_seqs);
  launch_pdl(attn_decode_kernel, dim3(grid), dim3(kDecWarps * 32), kDecSmem, stream, p);
  if (cudaGetLastError() != cudaSuccess) return XV_ERR_LAUNCH;
  if (splits > 1) {
    launch_pdl(attn_combine_kernel, dim3(num_seqs * hq), dim3(kD), 0, stream, p.ws_o, p.ws_lse, p.out, splits);
    if (cudaGetLastError() != cudaSuccess) return XV_ERR_LAUNCH;
  }
  return 0;
}

int xv_attn_prefill(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                    const int* cu_q, const int* kv_lens, void* out, int seq_begin, int num_seqs, int max_q_len,
                    int hq, int hkv, int d, int block_size, int max_blocks, float scale, cudaStream_t stream) {
  if (num_seqs <= 0 || max_q_len <= 0) return 0;
  if (d != kD) return XV_ERR_UNSUPPORTED;
  if (block_size % kTile || hq % hkv) return XV_ERR_SHAPE;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmem) != cudaSuccess)
      return XV_ERR_LAUNCH;
    attr = true;
  }
  PrefillParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.block_tables = block_tables;
  p.cu_q = cu_q;
  p.kv_lens = kv_lens;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.seq_begin = seq_begin; p.hq = hq; p.hkv = hkv; p.block_size = block_size; p.max_blocks = max_blocks;
  p.scale_log2 = scale * kLog2e;
  dim3 grid((max_q_len + kPfBM - 1) / kPfBM, hq, num_seqs);
  launch_pdl(attn_prefill_kernel, dim3(grid), dim3(kPfWarps * 32), kPfSmem, stream, p);
  return cudaGetLastError() == cudaSuccess ? 0 : XV_ERR_LAUNCH;
}

}  // extern "C"
