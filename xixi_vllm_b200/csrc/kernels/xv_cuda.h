// C ABI of the sm_100a kernel library (loaded from Python through ctypes). Every function
// enqueues work on the given stream and returns 0, or a negative XV_ERR_* code without
// launching. Pointers are device pointers unless stated otherwise; bf16 activations/weights.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XV_ERR_SHAPE (-1)
#define XV_ERR_ALIGN (-2)
#define XV_ERR_WORKSPACE (-3)
#define XV_ERR_DRIVER (-4)
#define XV_ERR_TENSORMAP (-5)
#define XV_ERR_LAUNCH (-6)
#define XV_ERR_UNSUPPORTED (-7)

typedef struct XvGemmPlan {
  int swapped;             // 1: weights on the MMA M axis (few tokens)
  int bn;                  // MMA N
  int tiles_a, tiles_b;
  int splits;              // split-K factor (grid.z)
  int k_blocks_per_split;
  int stages;
  int smem_bytes;
  int ctas_per_sm;         // resident CTAs per SM the persistent grid is sized for
  int cluster;             // 1: the K splits of a tile are one thread-block cluster and sum their accumulators
                           //    through distributed shared memory (the output is final: no planes, no workspace)
  int pair;                // 1: CTA-pair kernel (cta_group::2, 256 x bn tiles, stream-K)
  int sk_tiles;            // pair kernel: tiles of the last wave that are cut into K parts (stream-K tail) ...
  int sk_parts;            // ... this many each (2 or 3), one part per SM pair ...
  int units_per_pair;      // ... of this many K blocks
  long long workspace_bytes;
} XvGemmPlan;

int xv_gemm_plan(int m, int n, int k, int num_sms, XvGemmPlan* plan);
// The plan of xv_gemm_bf16_noalloc: K splits are always fp32 planes in a workspace (never summed inside a cluster).
int xv_gemm_plan_planes(int m, int n, int k, int num_sms, XvGemmPlan* plan);
void xv_gemm_disable_pair(int disable);   // test hook: force the single-CTA kernel
// Test and tuning hook: fixed kernel (0 single CTA, 1 single CTA normal orientation, 2 CTA pairs, 3 CTA pairs
// in the swapped orientation for at most 256 rows), tile width, split-K and stage count instead of the planner's
// choice; values <= 0 keep the default, kind < 0 clears.
void xv_gemm_plan_override(int kind, int bn, int splits, int stages);
// `workspace`: fp32 partial planes of a split-K plan (plan.workspace_bytes). A workspace of 40 MiB or more also
// serves the CTA-pair kernel's K-part tail: its last 20 MiB then hold partial tiles and, in the final 4 KiB,
// counters; those must be zero before the first call that uses the buffer and are left zero by every call
// (the tiles need no initial value); planes use the part in front.
// With a smaller workspace the pair kernel deals whole tiles. Calls that overlap on the GPU must not share a
// workspace.
int xv_gemm_bf16(const void* x, const void* w, void* y, int m, int n, int k, long long ldx, long long ldw,
                 long long ldy, void* workspace, long long workspace_bytes, int num_sms, int* status,
                 cudaStream_t stream);

// As xv_gemm_bf16, but a split-K plan leaves its fp32 partial planes [splits][m][n] in `workspace`
// (y untouched) for a consumer kernel that sums them; *splits_out reports the split count.
int xv_gemm_bf16_defer(const void* x, const void* w, void* y, int m, int n, int k, long long ldx, long long ldw,
                       long long ldy, void* workspace, long long workspace_bytes, int num_sms, int* status,
                       cudaStream_t stream, int* splits_out);

// GEMM with a fused SiLU-mul epilogue: W's rows are interleaved in groups of 16 = [8 gate | 8 up],
// Y is [m, n/2]. Only for plans that do not split K into planes. `workspace` (may be null) is the same buffer
// the other GEMM entry points get: the CTA-pair kernel cuts a thin last wave along K through its tail.
int xv_gemm_bf16_silu_mul(const void* x, const void* w, void* y, int m, int n, int k, long long ldx, long long ldw,
                          long long ldy, void* workspace, long long workspace_bytes, int num_sms, int* status,
                          cudaStream_t stream);
// SiLU-mul over activations in that interleaved layout: bf16 x [rows, 2*inter], or `splits` fp32
// partial planes of a split-K GEMM when `partials` is non-null.
int xv_silu_mul_interleaved(const void* x, const float* partials, int splits, long long split_stride, void* y,
                            int rows, int inter, cudaStream_t stream);

// Same GEMM for callers that must not allocate GPU memory. This entry point has no counterpart
// in the reference project. Who needs it: code that runs where a device allocation is not
// allowed or would stall the GPU, for example a plug-in invoked from another runtime's execution
// callback, a latency-critical serving loop whose memory pool is frozen after start-up, or a
// host that only hands this library pre-existing buffers. xv_gemm_bf16 needs a caller-allocated
// split-K workspace for small-M problems; this variant keeps that scratch in a fixed buffer
// inside the library image instead (xv_gemm_noalloc_max_scratch_bytes() bytes, 16 MiB, resident
// on every GPU that loads the library until the process exits). It calls no cudaMalloc,
// cudaFree or allocating library routine; inputs and the output are still the caller's.
//   * Problems whose split-K partials exceed the built-in buffer are rejected with
//     XV_ERR_WORKSPACE and a message on stderr; nothing is launched.
//   * The first call on each device looks up the buffer's device address; make that first
//     call on a device before starting any stream capture on it.
//   * All calls on a device share the one buffer, which keeps the previous call's bytes.
//     Nothing in it has to start at zero: every element the reduction reads is rewritten by
//     the same call first. Two calls that overlap on the GPU (different streams, or graphs
//     replayed concurrently) race on it; serialise them.
long long xv_gemm_noalloc_max_scratch_bytes(void);
int xv_gemm_bf16_noalloc(const void* x, const void* w, void* y, int m, int n, int k, long long ldx, long long ldw,
                         long long ldy, int* status, cudaStream_t stream);

// ---- elementwise / normalisation ----
int xv_rmsnorm(const void* x, const void* w, void* y, int rows, int hidden, float eps, cudaStream_t stream);
// residual += x (in place), y = rmsnorm(residual) * w
int xv_add_rmsnorm(const void* x, void* residual, const void* w, void* y, int rows, int hidden, float eps,
                   cudaStream_t stream);
// x given as `splits` fp32 partial planes (stride split_stride elements) of a split-K GEMM.
int xv_add_rmsnorm_partials(const float* partials, int splits, long long split_stride, void* residual, const void* w,
                            void* y, int rows, int hidden, float eps, cudaStream_t stream);
int xv_silu_mul(const void* x, void* y, int rows, int inter, cudaStream_t stream);
int xv_embedding(const int* ids, const void* w, void* y, int tokens, int hidden, int vocab_start, int vocab_rows,
                 cudaStream_t stream);
int xv_gather_rows(const void* x, const int* rows, void* y, int n, int hidden, cudaStream_t stream);
// Per-head RMSNorm of q and k, NeoX RoPE, q written to q_out [T, hq*d], k/v appended to the
// paged cache [blocks, hkv, block_size, d] at `slots` (negative slot = skip).
// When `partials` is non-null the QKV activations are read as the sum of `splits` fp32 planes.
// Tokens from index `prefill_begin` on are prefill rows: after the last row such a chunk writes into a
// page, the remaining V rows of that page are cleared (the tcgen05 prefill kernel reads whole tiles).
int xv_qk_norm_rope_cache_partials(const float* partials, int splits, long long split_stride, const void* q_w,
                                   const void* k_w, float eps, const float* cos_sin, const int* positions,
                                   const int* slots, void* q_out, void* k_cache, void* v_cache, int tokens, int hq,
                                   int hkv, int d, int block_size, int prefill_begin, cudaStream_t stream);
int xv_qk_norm_rope_cache(const void* qkv, const void* q_w, const void* k_w, float eps, const float* cos_sin,
                          const int* positions, const int* slots, void* q_out, void* k_cache, void* v_cache,
                          int tokens, int hq, int hkv, int d, int block_size, int prefill_begin, cudaStream_t stream);

// ---- attention ----
// Decode: one query row per sequence (rows 0..num_seqs-1 of q) against the paged cache.
// `workspace` holds split partials: xv_attn_decode_workspace_bytes(...) bytes.
long long xv_attn_decode_workspace_bytes(int num_seqs, int hq, int d, int splits);
int xv_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                   const int* kv_lens, void* out, int num_seqs, int hq, int hkv, int d, int block_size,
                   int max_blocks, float scale, int splits, void* workspace, cudaStream_t stream);
// Prefill: packed varlen causal attention; sequence b owns query rows cu_q[b]..cu_q[b+1] which
// are the last rows of its kv_lens[b] cached tokens. `q_row0` offsets the first query row.
int xv_attn_prefill(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                    const int* cu_q, const int* kv_lens, void* out, int seq_begin, int num_seqs, int max_q_len,
                    int hq, int hkv, int d, int block_size, int max_blocks, float scale, cudaStream_t stream);
// The same operation on tcgen05 tensor cores (attn_prefill_sm100.cu): 128-row query tiles, K/V pages
// fetched by TMA. `total_tokens` is the row count of q/out, `num_blocks` the page count of the caches.
// Supported for head_dim 128 and page sizes that divide 64 or are multiples of 64.
int xv_attn_prefill_tc_supported(int d, int block_size);
void xv_attn_prefill_tc_single_unit(int on);   // 1: one head per CTA even when heads of a KV group could pair up
int xv_attn_prefill_tc(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                       const int* cu_q, const int* kv_lens, void* out, int seq_begin, int num_seqs, int max_q_len,
                       int total_tokens, int num_blocks, int hq, int hkv, int d, int block_size, int max_blocks,
                       float scale, int* status, cudaStream_t stream);
// Instrumented build of the same kernel: adds per-phase cycle totals to `prof` (xv_attn_prefill_tc_profile_slots()
// zero-initialised 64-bit device counters). For finding where the warps of a CTA wait; slower than the plain kernel.
int xv_attn_prefill_tc_profile_slots(void);
int xv_attn_prefill_tc_profile(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                               const int* cu_q, const int* kv_lens, void* out, int seq_begin, int num_seqs,
                               int max_q_len, int total_tokens, int num_blocks, int hq, int hkv, int d, int block_size,
                               int max_blocks, float scale, int* status, unsigned long long* prof,
                               cudaStream_t stream);

// Input ids < 0 are references into the previous step's samples: ids[i] = prev[-ids[i] - 1] (elementwise.cu).
int xv_resolve_token_refs(int* ids, int n, const long long* prev, int n_prev, cudaStream_t stream);

// ---- sampling ----
int xv_argmax(const void* logits, long long* out, int rows, int vocab, long long ld, cudaStream_t stream);
// rng: device int32[2] = {seed, step}. Rows with temperature <= 1e-5 are greedy.
int xv_sample(const void* logits, long long* out, int rows, int vocab, long long ld, const float* temperature,
              const int* top_k, const float* top_p, const float* min_p, const int* rng, cudaStream_t stream);

// ---- tensor-parallel fused reductions over peer memory (see tp_fused.cu) ----
int xv_tp_reduce_norm(const void* const* peer_bufs, void* const* peer_flags, const void* mc_buf, void* epoch,
                      int rank, int world, long long buf_offset, const void* residual_in, void* residual_out,
                      const void* w, void* y, int rows, int hidden, float eps, int mode, unsigned spin_limit,
                      int* status, cudaStream_t stream);
int xv_tp_reduce_norm_sharded(const void* const* peer_bufs, void* const* peer_flags, const void* mc_buf, void* epoch,
                              int rank, int world, long long buf_offset, long long h_offset, int has_residual,
                              void* residual, const void* w, int rows, int hidden, float eps, unsigned spin_limit,
                              int* status, cudaStream_t stream);
int xv_tp_reduce_norm_sharded_nowait(const void* const* peer_bufs, void* const* peer_flags, const void* mc_buf,
                                     void* epoch, int rank, int world, long long buf_offset, long long h_offset,
                                     int has_residual, void* residual, const void* w, int rows, int hidden,
                                     float eps, unsigned spin_limit, int* status, cudaStream_t stream);
int xv_tp_argmax(const void* const* peer_bufs, void* const* peer_flags, void* epoch, int rank, int world,
                 long long slots_offset, const void* logits, long long ld, int local_vocab, int valid_vocab,
                 int vocab_start, long long* out, int rows, unsigned spin_limit, int* status, cudaStream_t stream);

// Sampling over a vocabulary sharded across ranks without gathering the logits (sampler.cu): `logits` is this
// rank's [rows, >= valid_vocab] shard holding tokens vocab_start .. vocab_start + valid_vocab of total_vocab. The
// ranks exchange per-row maxima, 256-bin histograms and their best candidate through a zero-initialised region of
// xv_tp_sample_region_bytes(max_rows, world) bytes at `region_offset` of every rank's symmetric buffer; `epoch`
// words 24 and 25 count the launches. All ranks write the same tokens to `out`.
long long xv_tp_sample_region_bytes(int max_rows, int world);
int xv_tp_sample(const void* const* peer_bufs, void* const* peer_flags, void* epoch, int rank, int world,
                 long long region_offset, int max_rows, const void* logits, long long ld, int valid_vocab,
                 int vocab_start, int total_vocab, long long* out, int rows, const float* temperature,
                 const int* top_k, const float* top_p, const float* min_p, const int* rng, unsigned spin_us,
                 int* status, cudaStream_t stream);

int xv_tp_allgather_cols(const void* const* peer_bufs, void* const* peer_flags, const void* mc_buf, void* epoch,
                         int rank, int world, const void* src, long long ld, int local_cols, long long total_cols,
                         int rows, unsigned spin_limit, int* status, cudaStream_t stream);

// RowParallel GEMM + cross-rank sum + residual add + RMSNorm in ONE kernel (gemm_sm100.cu, tp_device.cuh):
// the GEMM epilogue pushes its tiles into the slot array (`slot_offset`, `slot_bytes`, inside the
// symmetric buffer) of the ranks that reduce them. two_shot = 1: rows are dealt to the ranks, the
// finished rows are broadcast to byte offset `h_offset` of every rank's symmetric buffer and the
// residual buffers hold only this rank's rows; two_shot = 0: every rank reduces all rows into its own
// y_out. `epoch`: 32 zero-initialised uint32 words of local device memory kept across calls.
int xv_gemm_bf16_tp(const void* x, const void* w, int m, int n, int k, long long ldx, long long ldw, void* workspace,
                    long long workspace_bytes, int num_sms, const void* const* peer_bufs, void* const* peer_flags,
                    const void* mc_buf, void* epoch, int rank,
                    int world, long long slot_offset, long long slot_bytes, int two_shot, long long h_offset,
                    const void* residual_in, void* residual_out, const void* norm_w, void* y_out, float eps, int mode,
                    int defer_row_wait, unsigned spin_us, int* status, cudaStream_t stream);
// All-gather -> GEMM. With defer_row_wait = 1 (two-shot form) xv_gemm_bf16_tp ends without waiting for the rows
// the other ranks broadcast; the GEMM that reads the activation waits for them in its loader instead: call
// xv_gemm_wait_for_rows right before launching that GEMM from the same thread. flags: this rank's flag array
// at word xv_tp_bcast_word(); targets: the `epoch` words from xv_tp_bcast_base_word() on; n: ranks.
void xv_gemm_wait_for_rows(const void* flags, const void* targets, int n, unsigned spin_us);
// The same hand-over for the row-sharded reduction kernel (xv_tp_reduce_norm_sharded_nowait): flags = this rank's
// flag array at word xv_tp_pull_done_word(), target = the `epoch` word xv_tp_pull_target_word(); all n flags must
// reach that one value.
void xv_gemm_wait_for_epoch(const void* flags, const void* target, int n, unsigned spin_us);
int xv_tp_pull_done_word(void);
int xv_tp_pull_target_word(void);
int xv_tp_bcast_word(void);
int xv_tp_bcast_base_word(void);

// Diagnostics for xv_gemm_bf16_tp: 8 global-timer stamps per CTA (kernel entry, GEMM roles done, tiles arrived,
// rows done, broadcast raised, all rows arrived (CTA 0), exit, unused) into `buf`; null switches it off.
void xv_tp_profile_buffer(void* buf);
// The single-CTA GEMM kernel's own phases (entry, barriers + TMEM ready, first load issued, first stage landed,
// first tile's MMAs issued, its accumulator complete, last epilogue done, exit), same buffer format.
void xv_gemm_profile_buffer(void* buf);

// ---- native forward executor (forward.cu): one call launches a whole Qwen3 forward ----
typedef struct XvLayerWeights {
  const void* input_norm;
  const void* qkv;
  const void* q_norm;
  const void* k_norm;
  const void* o;
  const void* post_norm;
  const void* gate_up;
  const void* down;
  void* k_cache;
  void* v_cache;
} XvLayerWeights;

typedef struct XvModelDesc {
  int num_layers, hidden, hq, hkv, head_dim, inter_local, qkv_rows, block_size;
  float eps, attn_scale;
  int gate_up_interleaved;
  int vocab_start, vocab_rows;        // this rank's embedding / LM-head shard
  int lm_head_rows, lm_valid;         // rows of the shard, and how many of them are real vocabulary
  const void* embed;
  const void* final_norm;
  const void* lm_head;
  const float* cos_sin;
  const XvLayerWeights* layers;       // host array of num_layers entries
  int tp_rank, tp_world;              // tensor parallel; with tp_world == 1 the fields below are unused
  const void* const* peer_bufs;       // host arrays of tp_world device pointers
  void* const* peer_flags;
  const void* mc_buf;
  void* epoch;
  long long h_offset;                 // byte offset of the activation buffer h inside the symmetric buffer: the
                                      // two-shot reductions broadcast the normalised rows there (< 0: none)
  long long buf_bytes;                // size of each of the three symmetric partial buffers
  long long slots_offset;             // byte offset of the argmax slots in the symmetric buffer
  unsigned spin_us;
  int num_kv_blocks;                  // pages in each layer's k_cache / v_cache
  int prefill_tc;                     // 1: prefill attention on the tcgen05 kernel when the shape allows
  int tp_push;                        // 1: row-parallel GEMM + reduction + norm as one kernel (xv_gemm_bf16_tp) ...
  int tp_push_max;                    // ... for forwards of at most this many tokens
  int tp_one_shot_max;                // of those, forwards of at most this many tokens reduce every row on every rank
  int tp_pull_two_shot;               // two-kernel form (GEMM, then a reduction kernel that pulls): 1 = row-sharded
  int tp_defer_row_wait;              // the GEMM that reads h waits for the other ranks' rows instead of the kernel that
                                      // caused them: bit 0 after the one-kernel two-shot projection, bit 1 after the
                                      // row-sharded reduction kernel
  int is_first, is_last;              // pipeline stage: the first owns the embedding, the last the LM head; on
                                      // other stages `final_norm` is the next stage's first input norm and the
                                      // arena's h / residual are received from / sent to the neighbours
} XvModelDesc;

typedef struct XvBatchDesc {
  int num_tokens, num_seqs, num_decode, max_q_len, max_blocks, num_samples, all_greedy;
  const int* input_ids;
  const int* positions;
  const int* slots;
  const int* cu_q;
  const int* kv_lens;
  const int* block_tables;
  const int* sample_rows;
} XvBatchDesc;

typedef struct XvArena {              // device scratch sized for the largest step; nothing is allocated per call
  void* h;                            // [T, hidden] normalised activations
  void* qkv;                          // [T, qkv_rows]
  void* q;                            // [T, hq * head_dim]
  void* attn;                         // [T, hq * head_dim]
  void* act;                          // [T, inter_local]
  void* gu;                           // [T, 2 * inter_local] (only without the fused SiLU-mul epilogue)
  void* residual;                     // [T, hidden]
  void* partial;                      // [T, hidden] row-parallel output when tp_world == 1
  void* hidden_out;                   // [S, hidden]
  void* logits;                       // [S, lm_head_rows]
  long long* tokens;                  // [S]
  void* gemm_ws;
  long long gemm_ws_bytes;
  void* attn_ws;
  long long attn_ws_bytes;
  int* status;
  int num_sms;
} XvArena;

// Returns 0 or the first failing launch's XV_ERR_* code (xv_forward_failed_op() names the step).
int xv_qwen3_forward(const XvModelDesc* model, const XvBatchDesc* batch, const XvArena* arena, cudaStream_t stream);
// Both are kept per calling thread: they describe the forwards that this thread issued.
int xv_forward_failed_op(void);
long long xv_forward_launch_calls(void);   // launch calls issued by forwards so far (each is at least one kernel)
int xv_forward_decode_splits(int num_seqs, int hkv, int num_sms, int max_tokens_per_seq);

// ---- diagnostics ----
// Waits (bounded) on a flag nobody sets and reports kHostFlagTimeout through `status`;
// proves the timeout path returns instead of hanging. `limit` polls.
int xv_selftest_bounded_wait(int* flag, int* status, unsigned limit, cudaStream_t stream);
int xv_num_sms(void);

#ifdef __cplusplus
}
#endif
