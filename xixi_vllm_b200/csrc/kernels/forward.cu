// Native forward executor: launches every kernel of one Qwen3 forward pass (embedding, all
// decoder layers, final norm, LM head, greedy sampling) from a single C call.
//
// Driving ~10 launches per layer from Python costs more host time than a tensor-parallel rank
// needs GPU time for the step, so eager (prefill-carrying) steps were bound by the interpreter.
// Here the host side of a step is one call that walks plain structs: weights and caches per
// layer, the packed batch metadata, and a preallocated activation arena (nothing is allocated).
// The same call is what gets captured into the decode CUDA graphs.
//
// The reference drives its forward from Python module by module
// (reference: src/compute/models/qwen3.py:149-208, src/compute/model_runner.py:145-262).

#include <cuda_runtime.h>

#include <cstdint>

#include "xv_cuda.h"

namespace {

// Per calling thread: a process that drives several devices runs one forward per thread, and the step that
// failed (or the launch count) a thread reads back is the one of its own forwards.
thread_local int g_failed_op = 0;
thread_local long long g_launch_calls = 0;     // launch calls issued by this thread's forwards (each is >= 1 kernel)

struct Ctx {
  const XvModelDesc* m;
  const XvBatchDesc* b;
  const XvArena* a;
  cudaStream_t s;
  int call_idx;      // reduction points issued so far in this forward (symmetric-buffer rotation)
  bool two_shot;     // this forward's reductions deal the rows to the ranks (residual stream sharded by rows)
  bool push;         // row-parallel GEMM and its reduction run as one kernel
  bool rows_pending; // the last reduction did not wait for the broadcast rows: the next GEMM on h does
};

// all-gather -> GEMM: the column-parallel GEMM that reads h waits for the rows itself
inline void await_rows_in_next_gemm(Ctx& c) {
  if (!c.rows_pending) return;
  c.rows_pending = false;
  const XvModelDesc* m = c.m;
  if (!c.push) {
    // the row-sharded reduction kernel left its "every rank's rows are here" wait to this GEMM
    xv_gemm_wait_for_epoch(static_cast<const uint32_t*>(m->peer_flags[m->tp_rank]) + xv_tp_pull_done_word(),
                           static_cast<const uint32_t*>(m->epoch) + xv_tp_pull_target_word(), m->tp_world, m->spin_us);
    return;
  }
  xv_gemm_wait_for_rows(static_cast<const uint32_t*>(m->peer_flags[m->tp_rank]) + xv_tp_bcast_word(),
                        static_cast<const uint32_t*>(m->epoch) + xv_tp_bcast_base_word(), m->tp_world, m->spin_us);
}

#define XV_TRY(opid, expr)      \
  do {                          \
    int rc_ = (expr);           \
    if (rc_ != 0) {             \
      g_failed_op = (opid);     \
      return rc_;               \
    }                           \
    ++g_launch_calls;           \
  } while (0)

inline char* symm_local(const Ctx& c, int which) {
  return const_cast<char*>(static_cast<const char*>(c.m->peer_bufs[c.m->tp_rank])) + which * c.m->buf_bytes;
}

// Row-parallel projection followed by the reduction point that consumes it:
//   residual += sum_over_ranks(x W^T);  h = rmsnorm(residual) * norm_w
// Under tensor parallelism this is the GEMM into the symmetric buffer followed by a reduction kernel that
// pulls the partial sums, or, when the model description asks for it (tp_push), ONE kernel
// (xv_gemm_bf16_tp: tiles pushed from the GEMM epilogue to the ranks that reduce them).
int row_linear_reduce_norm(Ctx& c, const void* x, const void* w, int k, const void* norm_w, bool final_call) {
  const XvModelDesc* m = c.m;
  const int T = c.b->num_tokens, H = m->hidden;
  if (m->tp_world > 1) {
    const int which = final_call ? 2 : (c.call_idx & 1);
    ++c.call_idx;
    const long long slot_off = static_cast<long long>(which) * m->buf_bytes;
    if (c.push) {
      // the consumer of h is a GEMM on every call but the forward's last (LM head via a row gather)
      const bool defer = c.two_shot && !final_call && (m->tp_defer_row_wait & 1) != 0;
      XV_TRY(16, xv_gemm_bf16_tp(x, w, T, H, k, k, k, c.a->gemm_ws, c.a->gemm_ws_bytes, c.a->num_sms, m->peer_bufs, m->peer_flags, m->mc_buf, m->epoch,
                                 m->tp_rank, m->tp_world, slot_off, m->buf_bytes, c.two_shot ? 1 : 0, m->h_offset,
                                 c.a->residual, c.a->residual, norm_w, c.a->h, m->eps, 0, defer ? 1 : 0, m->spin_us,
                                 c.a->status, c.s));
      c.rows_pending = defer;
      return 0;
    }
    XV_TRY(10, xv_gemm_bf16(x, w, symm_local(c, which), T, H, k, k, k, H, c.a->gemm_ws, c.a->gemm_ws_bytes,
                            c.a->num_sms, c.a->status, c.s));
    if (c.two_shot) {
      // the consumer of h is a GEMM on every call but the forward's last: it waits for the other ranks' rows
      if (!final_call && (m->tp_defer_row_wait & 2) != 0) {
        XV_TRY(15, xv_tp_reduce_norm_sharded_nowait(m->peer_bufs, m->peer_flags, m->mc_buf, m->epoch, m->tp_rank,
                                                    m->tp_world, slot_off, m->h_offset, 1, c.a->residual, norm_w, T,
                                                    H, m->eps, m->spin_us, c.a->status, c.s));
        c.rows_pending = true;
        return 0;
      }
      XV_TRY(15, xv_tp_reduce_norm_sharded(m->peer_bufs, m->peer_flags, m->mc_buf, m->epoch, m->tp_rank, m->tp_world,
                                           slot_off, m->h_offset, 1, c.a->residual, norm_w, T, H, m->eps, m->spin_us,
                                           c.a->status, c.s));
      return 0;
    }
    XV_TRY(11, xv_tp_reduce_norm(m->peer_bufs, m->peer_flags, m->mc_buf, m->epoch, m->tp_rank, m->tp_world, slot_off,
                                 c.a->residual, c.a->residual, norm_w, c.a->h, T, H, m->eps, 0, m->spin_us,
                                 c.a->status, c.s));
    return 0;
  }
  int splits = 1;
  XV_TRY(12, xv_gemm_bf16_defer(x, w, c.a->partial, T, H, k, k, k, H, c.a->gemm_ws, c.a->gemm_ws_bytes, c.a->num_sms,
                                c.a->status, c.s, &splits));
  if (splits > 1) {
    XV_TRY(13, xv_add_rmsnorm_partials(static_cast<const float*>(c.a->gemm_ws), splits,
                                       static_cast<long long>(T) * H, c.a->residual, norm_w, c.a->h, T, H, m->eps,
                                       c.s));
  } else {
    XV_TRY(14, xv_add_rmsnorm(c.a->partial, c.a->residual, norm_w, c.a->h, T, H, m->eps, c.s));
  }
  return 0;
}

int decode_splits(int num_seqs, int hkv, int num_sms, int max_tokens_per_seq) {
  int ctas = num_seqs * hkv;
  if (ctas < 1) ctas = 1;
  int want = (2 * num_sms + ctas - 1) / ctas;
  int by_len = max_tokens_per_seq / 256;
  if (by_len < 1) by_len = 1;
  int s = want < by_len ? want : by_len;
  if (s > 16) s = 16;
  if (s < 1) s = 1;
  return s;
}

}  // namespace

extern "C" {

int xv_forward_failed_op(void) { return g_failed_op; }
long long xv_forward_launch_calls(void) { return g_launch_calls; }

int xv_forward_decode_splits(int num_seqs, int hkv, int num_sms, int max_tokens_per_seq) {
  return decode_splits(num_seqs, hkv, num_sms, max_tokens_per_seq);
}

int xv_qwen3_forward(const XvModelDesc* m, const XvBatchDesc* b, const XvArena* a, cudaStream_t stream) {
  Ctx c{m, b, a, stream, 0, false, false, false};
  const int T = b->num_tokens, H = m->hidden, D = m->head_dim;
  if (T <= 0) return 0;
  const int q_cols = m->hq * D;
  const int L = m->num_layers;
  if (m->tp_world > 1) {
    // One kernel per row-parallel projection (tiles pushed to the reducing ranks) up to tp_push_max tokens.
    // Few rows: every rank reduces every row (one wait per reduction point). More rows: the rows are dealt
    // to the ranks (traffic per GPU independent of the rank count, a second wait for the broadcast).
    // The form fixes the layout of the residual stream, so it is chosen once per forward, and identically
    // on both sides of a pipeline hand-off (same token count, same settings).
    if (m->tp_push != 0 && m->h_offset >= 0 && T <= m->tp_push_max && H <= 6144) {     // 6144: the fused tail's row width
      c.two_shot = T > m->tp_one_shot_max;
      const long long cap = c.two_shot ? (T + m->tp_world - 1) / m->tp_world : T;
      c.push = static_cast<long long>(m->tp_world) * cap * H * 2 <= m->buf_bytes;
    }
    if (!c.push) c.two_shot = m->h_offset >= 0 && m->tp_pull_two_shot != 0;
  }

  // ---- embedding and the first normalisation point (first pipeline stage) ----
  if (!m->is_first) {
    // h (normalised by the sender with this stage's first input norm) and the residual stream were received
    // into the arena; after a two-shot reduction each rank holds only its rows of the residual.
  } else if (m->tp_world > 1) {
    const int which = (L == 0) ? 2 : (c.call_idx & 1);
    ++c.call_idx;
    XV_TRY(1, xv_embedding(b->input_ids, m->embed, symm_local(c, which), T, H, m->vocab_start, m->vocab_rows, stream));
    const void* w0 = L > 0 ? m->layers[0].input_norm : m->final_norm;
    if (c.two_shot) {
      XV_TRY(5, xv_tp_reduce_norm_sharded(m->peer_bufs, m->peer_flags, m->mc_buf, m->epoch, m->tp_rank, m->tp_world,
                                          static_cast<long long>(which) * m->buf_bytes, m->h_offset, 0, a->residual, w0,
                                          T, H, m->eps, m->spin_us, a->status, stream));
    } else
    XV_TRY(2, xv_tp_reduce_norm(m->peer_bufs, m->peer_flags, m->mc_buf, m->epoch, m->tp_rank, m->tp_world,
                                static_cast<long long>(which) * m->buf_bytes, nullptr, a->residual, w0, a->h, T, H,
                                m->eps, 0, m->spin_us, a->status, stream));
  } else {
    XV_TRY(3, xv_embedding(b->input_ids, m->embed, a->residual, T, H, m->vocab_start, m->vocab_rows, stream));
    const void* w0 = L > 0 ? m->layers[0].input_norm : m->final_norm;
    XV_TRY(4, xv_rmsnorm(a->residual, w0, a->h, T, H, m->eps, stream));
  }

  const int n_dec = b->num_decode, n_pre = b->num_seqs - b->num_decode;
  const int splits_attn = n_dec > 0 ? decode_splits(n_dec, m->hkv, a->num_sms, b->max_blocks * m->block_size) : 1;
  if (n_dec > 0 && xv_attn_decode_workspace_bytes(n_dec, m->hq, D, splits_attn) > a->attn_ws_bytes) {
    g_failed_op = 20;
    return XV_ERR_WORKSPACE;
  }

  // Short chunks do not fill a 128-row tile; they stay on the 64-row warp-MMA kernel.
  const bool prefill_tc = m->prefill_tc && m->num_kv_blocks > 0 && b->max_q_len > 64 &&
                          xv_attn_prefill_tc_supported(D, m->block_size);

  for (int l = 0; l < L; ++l) {
    const XvLayerWeights& w = m->layers[l];
    // ---- attention block ----
    int splits = 1;
    await_rows_in_next_gemm(c);
    XV_TRY(30, xv_gemm_bf16_defer(a->h, w.qkv, a->qkv, T, m->qkv_rows, H, H, H, m->qkv_rows, a->gemm_ws,
                                  a->gemm_ws_bytes, a->num_sms, a->status, stream, &splits));
    if (splits > 1) {
      XV_TRY(31, xv_qk_norm_rope_cache_partials(static_cast<const float*>(a->gemm_ws), splits,
                                                static_cast<long long>(T) * m->qkv_rows, w.q_norm, w.k_norm, m->eps,
                                                m->cos_sin, b->positions, b->slots, a->q, w.k_cache, w.v_cache, T,
                                                m->hq, m->hkv, D, m->block_size, n_dec, stream));
    } else {
      XV_TRY(32, xv_qk_norm_rope_cache(a->qkv, w.q_norm, w.k_norm, m->eps, m->cos_sin, b->positions, b->slots, a->q,
                                       w.k_cache, w.v_cache, T, m->hq, m->hkv, D, m->block_size, n_dec, stream));
    }
    if (n_dec > 0)
      XV_TRY(33, xv_attn_decode(a->q, w.k_cache, w.v_cache, b->block_tables, b->kv_lens, a->attn, n_dec, m->hq, m->hkv,
                                D, m->block_size, b->max_blocks, m->attn_scale, splits_attn, a->attn_ws, stream));
    if (n_pre > 0 && prefill_tc)
      XV_TRY(35, xv_attn_prefill_tc(a->q, w.k_cache, w.v_cache, b->block_tables, b->cu_q, b->kv_lens, a->attn, n_dec,
                                    n_pre, b->max_q_len, T, m->num_kv_blocks, m->hq, m->hkv, D, m->block_size,
                                    b->max_blocks, m->attn_scale, a->status, stream));
    else if (n_pre > 0)
      XV_TRY(34, xv_attn_prefill(a->q, w.k_cache, w.v_cache, b->block_tables, b->cu_q, b->kv_lens, a->attn, n_dec,
                                 n_pre, b->max_q_len, m->hq, m->hkv, D, m->block_size, b->max_blocks, m->attn_scale,
                                 stream));
    {
      int rc = row_linear_reduce_norm(c, a->attn, w.o, q_cols, w.post_norm, false);
      if (rc) return rc;
    }
    // ---- MLP block ----
    const int I = m->inter_local;
    await_rows_in_next_gemm(c);
    if (m->gate_up_interleaved) {
      XvGemmPlan pl;
      if (int rc = xv_gemm_plan(T, 2 * I, H, a->num_sms, &pl)) {   // host arithmetic only, not a launch
        g_failed_op = 40;
        return rc;
      }
      if (pl.splits == 1 || pl.cluster) {
        XV_TRY(41, xv_gemm_bf16_silu_mul(a->h, w.gate_up, a->act, T, 2 * I, H, H, H, I, a->gemm_ws, a->gemm_ws_bytes,
                                         a->num_sms, a->status, stream));
      } else {
        int sp = 1;
        XV_TRY(42, xv_gemm_bf16_defer(a->h, w.gate_up, nullptr, T, 2 * I, H, H, H, 2 * I, a->gemm_ws, a->gemm_ws_bytes,
                                      a->num_sms, a->status, stream, &sp));
        XV_TRY(43, xv_silu_mul_interleaved(nullptr, static_cast<const float*>(a->gemm_ws), sp,
                                           static_cast<long long>(T) * 2 * I, a->act, T, I, stream));
      }
    } else {
      XV_TRY(44, xv_gemm_bf16(a->h, w.gate_up, a->gu, T, 2 * I, H, H, H, 2 * I, a->gemm_ws, a->gemm_ws_bytes,
                              a->num_sms, a->status, stream));
      XV_TRY(45, xv_silu_mul(a->gu, a->act, T, I, stream));
    }
    // the stage's last point normalises with the next stage's first input norm (a copy of it is loaded here)
    const void* next_norm = (l + 1 < L) ? m->layers[l + 1].input_norm : m->final_norm;
    {
      int rc = row_linear_reduce_norm(c, a->act, w.down, I, next_norm, l + 1 == L);
      if (rc) return rc;
    }
  }

  // ---- sampling rows -> LM head (last pipeline stage) ----
  const int S = b->num_samples;
  if (S <= 0 || !m->is_last) return 0;
  XV_TRY(50, xv_gather_rows(a->h, b->sample_rows, a->hidden_out, S, H, stream));
  XV_TRY(51, xv_gemm_bf16(a->hidden_out, m->lm_head, a->logits, S, m->lm_head_rows, H, H, H, m->lm_head_rows,
                          a->gemm_ws, a->gemm_ws_bytes, a->num_sms, a->status, stream));
  if (b->all_greedy) {
    if (m->tp_world > 1) {
      XV_TRY(52, xv_tp_argmax(m->peer_bufs, m->peer_flags, m->epoch, m->tp_rank, m->tp_world, m->slots_offset, a->logits,
                              m->lm_head_rows, m->lm_head_rows, m->lm_valid, m->vocab_start, a->tokens, S, m->spin_us,
                              a->status, stream));
    } else {
      XV_TRY(53, xv_argmax(a->logits, a->tokens, S, m->lm_valid, m->lm_head_rows, stream));
    }
  }
  return 0;
}

}  // extern "C"
