// Host-side executor of one continuous-batching step over a hybrid decoder stack: gated-delta-rule
// linear-attention layers (fp32 recurrent state per sequence in a slot pool) interleaved with gated
// full-attention layers (paged KV cache, block 16, head_dim 128 or 256), SwiGLU MLPs, int4 group-32
// weights. The reference has no decoder model (crates/decoders/src/lib.rs:1-15); the recurrence is
// gated_delta_rule_recurrent_fwd (crates/kernels/src/gated_delta_rule/cpu.rs:92-182), the gate
// formulas are those of research/14-gdn-aiter-preflight.md:190-198, :209-219, and the contract is
// "a packed step equals running every sequence alone".
//
// A step packs decode tokens (one per sequence) first and prefill chunks after them (a chunk may start its
// sequence or continue it: positions, cache slots and the recurrent state carry on from the cached length):
//   embed -> per layer [ rms_norm -> mixer -> residual -> rms_norm -> gate/up + SwiGLU -> down +
//   residual ] -> last token rows -> final norm -> lm_head (int4 GEMV) -> greedy argmax
//   full-attention mixer: one GEMM to q | k | v | gate columns; RoPE on q and k; K/V rows scattered
//     into the paged cache; paged decode kernel for the decode rows, ragged causal attention for the
//     prefill rows (over the chunk's own rows when every chunk starts its sequence, else over keys and
//     values gathered from the cache through the block tables); out *= sigmoid(gate); o_proj
//     accumulates into the fp32 residual
//   linear-attention mixer: one GEMM to q | k | v | z columns, one to fp32 a | b columns; L2 norm of
//     q, k and the fp32 gates; the recurrence over every sequence's new tokens against its state
//     slot (a decode token is a sequence of one token); out *= silu(z); out_proj accumulates into
//     the residual
#include <cuda_runtime.h>

#include <cmath>
#include <mutex>
#include <string>
#include <vector>

#include "logismos_kernels.h"
#include "logismos_model.h"
#include "model_util.h"

namespace {

using namespace lgm;

struct HLayer {
  bool full = false;
  Buf norm1, norm2, kpool, vpool, state, A_log, dt_bias;
  QMat w_in, w_ab, w_out, wgu, wdown;
};

constexpr int kChunkTokens = 512;
constexpr int kBlock = 16;
constexpr int kGdnDim = 128;

struct Hybrid {
  lg_hybrid_config_t cfg{};
  int device = 0;
  int qw = 0, kvw = 0, attn_n = 0;  // full attention: q width, kv width, projection width (2 qw + 2 kvw)
  int gw = 0, gdn_n = 0;            // linear attention: heads * 128, projection width (4 gw)
  int mix_w = 0;                    // widest mixer output fed to the output projection
  Buf tok_embed, final_norm, cos, sin;
  QMat lm_head;
  std::vector<HLayer> layers;
  Buf delta;  // partial sum of an output projection when a cross-rank reduction is installed
  lg_allreduce_f32_fn allreduce = nullptr;
  void* allreduce_user = nullptr;
  lg_reduce_add_f32_fn reduce_add = nullptr;  // reduction fused with the residual add (takes precedence)
  void* reduce_add_user = nullptr;
  Buf x, h, proj, mix, qdec, ab, g, beta, act, wscratch, accws, last, last_bf16, logits, tokens, status;
  Buf gdn_scratch;  // per (chunk, head) intermediates of the chunk-parallel recurrence (two-launch form)
  Buf gdn_pairs;    // arrival counters of the fused decode kernel's CTA pairs, all zero between launches
  Buf ids, pos, slots, cu_all, cu_prefill, last_idx, dec_ctx, dec_tables, dec_chunks, dec_scratch, attn_ws, state_slots, fresh, pre_kv;
  uint8_t* pinned = nullptr;
  size_t pinned_bytes = 0;
  cudaStream_t stream = nullptr;
  std::mutex mu;
  int T = 0, n_dec = 0, n_pre = 0, n_seqs = 0, max_pre_len = 0, total_chunks = 0, chunk_tokens = kChunkTokens, launches = 0, logits_f32 = 0;
  std::vector<int> order;
  size_t max_chunks = 0;
  // the fused int4 linears rely on `accws` being all zero between calls, which their finishing kernels
  // restore; a step that failed part-way may have left partial sums there, so the next one clears it
  bool acc_dirty = false;
  size_t accws_bytes = 0;
  // prefill chunks that continue cached sequences: runs of prefill sequences whose keys fit the gather
  // workspace together (one gather + attention launch pair per run)
  struct PrefixRun { int s0, s1, total_kv, max_q, max_kv; };
  std::vector<PrefixRun> prefix_runs;
  bool pre_has_prefix = false;
  size_t prefix_cap_tokens = 0;
};

uint32_t qlinear(Hybrid* m, const void* a, const QMat& w, void* out, int T, int lda, int ldc, int epi, cudaStream_t s) {
  LG_TRY(qlinear_any(a, w, nullptr, out, T, lda, ldc, epi, m->wscratch.p, m->accws.p, m->status.p, &m->launches, s), "int4 linear");
  return 0;
}

// x += A W^T for an output projection; with a cross-rank reduction installed the local partial sum
// is reduced over the ranks before it joins the residual stream
uint32_t out_proj(Hybrid* m, const void* a, const QMat& w, int T, int lda, cudaStream_t s) {
  const int H = m->cfg.hidden;
  if (!m->allreduce && !m->reduce_add) return qlinear(m, a, w, m->x.p, T, lda, H, LG_EPI_RESID_F32, s);
  LG_TRY(cudaMemsetAsync(m->delta.p, 0, (size_t)T * H * 4, s), "memset partial sum");
  if (uint32_t rc = qlinear(m, a, w, m->delta.p, T, lda, H, LG_EPI_RESID_F32, s)) return rc;
  if (m->reduce_add) {
    if (m->reduce_add(m->reduce_add_user, m->x.p, m->delta.p, (uint64_t)T * H, m->status.p, (void*)s) != 0) {
      set_error("the installed reduce-add reported a failure");
      return LG_EMB_COMPUTE;
    }
    m->launches += 1;
    return 0;
  }
  if (m->allreduce(m->allreduce_user, m->delta.p, (uint64_t)T * H, (void*)s) != 0) {
    set_error("the installed all-reduce reported a failure");
    return LG_EMB_COMPUTE;
  }
  LG_TRY(logismos_launch_add_f32(m->x.p, m->delta.p, (int64_t)T * H, s), "add partial sum");
  m->launches += 1;
  return 0;
}

uint32_t run_device(Hybrid* m, cudaStream_t s) {
  const lg_hybrid_config_t& c = m->cfg;
  const int H = c.hidden, I = c.intermediate, D = c.attn_head_dim, T = m->T, QW = m->qw, KW = m->kvw, AN = m->attn_n;
  const int GW = m->gw, GN = m->gdn_n, GH = c.gdn_heads;
  void* st = m->status.p;
  m->launches = 0;
  if (m->acc_dirty) {
    LG_TRY(cudaMemsetAsync(m->accws.p, 0, m->accws_bytes, s), "clear accumulation workspace");
    LG_TRY(cudaMemsetAsync(m->gdn_pairs.p, 0, (size_t)m->cfg.max_step_seqs * m->cfg.gdn_heads * 4, s), "clear pair counters");
    m->acc_dirty = false;
  }
  LG_TRY(logismos_launch_embed_lookup_bf16(m->tok_embed.p, m->ids.p, m->x.p, T, H, c.vocab, s), "embed_lookup");
  m->launches += 1;
  for (int l = 0; l < c.n_layers; ++l) {
    HLayer& L = m->layers[l];
    LG_TRY(logismos_launch_rms_norm_f32(m->x.p, L.norm1.p, m->h.p, T, H, c.rms_eps, 0, s), "rms_norm");
    m->launches += 1;
    uint16_t* p16 = (uint16_t*)m->proj.p;
    if (L.full) {
      // columns: q [QW] | k [KW] | v [KW] | gate [QW]
      if (uint32_t rc = qlinear(m, m->h.p, L.w_in, m->proj.p, T, H, AN, LG_EPI_BF16, s)) return rc;
      LG_TRY(logismos_launch_rope_halves_bf16(m->proj.p, m->cos.p, m->sin.p, m->pos.p, T, c.n_heads + c.n_kv_heads, D, AN,
                                              c.max_pos, st, s), "rope");
      LG_TRY(logismos_launch_paged_kv_store_bf16(p16 + QW, p16 + QW + KW, AN, L.kpool.p, L.vpool.p, m->slots.p, T, KW,
                                                 (int64_t)c.n_pool_blocks * kBlock, st, s), "paged_kv_store");
      m->launches += 2;
      if (m->n_dec > 0) {
        LG_TRY(cudaMemcpy2DAsync(m->qdec.p, (size_t)QW * 2, m->proj.p, (size_t)AN * 2, (size_t)QW * 2, m->n_dec,
                                 cudaMemcpyDeviceToDevice, s), "q gather");
        LG_TRY(logismos_launch_paged_attention_decode_bf16(m->qdec.p, L.kpool.p, L.vpool.p, nullptr, nullptr, m->dec_tables.p,
                                                           m->dec_ctx.p, m->dec_chunks.p, m->mix.p, m->dec_scratch.p, st, m->n_dec,
                                                           m->total_chunks, m->chunk_tokens, c.max_blocks_per_seq, c.n_pool_blocks,
                                                           c.n_heads, c.n_kv_heads, D, s), "paged_attention_decode");
        m->launches += 2;
      }
      if (m->n_pre > 0 && m->pre_has_prefix) {
        // some chunk continues a cached sequence: keys and values come from the cache (the chunk's own rows
        // were stored above), gathered per run of sequences into attn_ws
        const int32_t* tabs = (const int32_t*)m->dec_tables.p + (size_t)m->n_dec * c.max_blocks_per_seq;
        for (const Hybrid::PrefixRun& r : m->prefix_runs) {
          LG_TRY(logismos_launch_paged_prefix_attention_tc_bf16(
                     p16 + (size_t)m->n_dec * AN, AN, (const int32_t*)m->cu_prefill.p + r.s0, (const int32_t*)m->pre_kv.p + r.s0,
                     L.kpool.p, L.vpool.p, tabs + (size_t)r.s0 * c.max_blocks_per_seq, c.max_blocks_per_seq, c.n_pool_blocks,
                     (uint16_t*)m->mix.p + (size_t)m->n_dec * QW, m->attn_ws.p, T - m->n_dec, r.total_kv, r.s1 - r.s0, r.max_q,
                     r.max_kv, c.n_heads, c.n_kv_heads, D, st, s),
                 "paged_prefix_attention");
          m->launches += 2;
        }
      } else if (m->n_pre > 0) {
        // tcgen05 kernel; V transposed into attn_ws first
        LG_TRY(logismos_launch_varlen_attention_tc_bf16(p16 + (size_t)m->n_dec * AN, m->cu_prefill.p,
                                                        (uint16_t*)m->mix.p + (size_t)m->n_dec * QW, m->attn_ws.p, T - m->n_dec,
                                                        m->n_pre, m->max_pre_len, c.n_heads, c.n_kv_heads, D, AN, QW, QW + KW, 1,
                                                        st, s), "varlen_attention");
        m->launches += 2;
      }
      LG_TRY(logismos_launch_gated_mul_bf16(m->mix.p, QW, p16 + QW + 2 * KW, AN, T, QW, 0, s), "attention gate");
      m->launches += 1;
      if (uint32_t rc = out_proj(m, m->mix.p, L.w_out, T, QW, s)) return rc;
    } else {
      // columns: q [GW] | k [GW] | v [GW] | z [GW] | a [GH] | b [GH] of one weight matrix
      // fused up to 64 rows (the 64-token tile of the fused-dequant kernel) even when the dense route has
      // a bf16 copy to work on. Measured per decode step, fused against dense (GEMM + memset + a|b GEMM +
      // prepare + recurrence): 56 rows 4.60 against 4.79 ms, 72 rows 4.95 against 4.95, 88 rows 5.61 against
      // 5.38, 96 rows 5.81 against 5.50, 128 rows 6.44 against 6.10: above 64 rows the fused kernel is on its
      // 128-token configuration (two issuing threads) and loses
      bool recurrence_done = false;
      if (T <= (L.w_in.dense.p ? 64 : kFusedDequantMaxRows)) {
        // one fused-dequant accumulation of all six blocks, finished by the kernel that also normalises
        // q, k and computes the gates from the fp32 sums
        const int ld = GN + 2 * GH;
        LG_TRY(logismos_launch_qlinear_int4_g32_acc_f32_static(m->h.p, L.w_in.codes.p, L.w_in.scales.p, m->accws.p, T, ld, H, H, ld, st, s),
               "int4 linear");
        if (m->n_pre == 0) {
          // a pure decode step: normalisation, gates and the recurrence in one launch from the fp32 sums
          LG_TRY(logismos_launch_gdn_decode_from_acc(L.state.p, m->accws.p, ld, L.A_log.p, L.dt_bias.p, m->mix.p, m->state_slots.p,
                                                     m->fresh.p, m->gdn_pairs.p, m->n_dec, GH, 1.0f / std::sqrt((float)kGdnDim), s),
                 "gdn decode from the accumulation workspace");
          m->launches += 2;
          recurrence_done = true;
        } else {
          LG_TRY(logismos_launch_gdn_finish(m->accws.p, ld, L.A_log.p, L.dt_bias.p, m->proj.p, GN, m->g.p, m->beta.p, T, GH, s), "gdn_finish");
          m->launches += 2;
        }
      } else {
        // dense path: q | k | v | z to bf16, a | b as fp32 through the accumulate epilogue
        QMat main_rows = L.w_in, ab_rows = L.w_in;  // views of the row blocks (no ownership)
        main_rows.n = GN;
        ab_rows.n = 2 * GH;
        ab_rows.codes.p = (uint8_t*)L.w_in.codes.p + (size_t)GN * (H / 2);
        ab_rows.scales.p = (uint8_t*)L.w_in.scales.p + (size_t)GN * (H / 32) * 2;
        if (L.w_in.dense.p) ab_rows.dense.p = (uint8_t*)L.w_in.dense.p + (size_t)GN * H * 2;
        if (uint32_t rc = qlinear(m, m->h.p, main_rows, m->proj.p, T, H, GN, LG_EPI_BF16, s)) return rc;
        LG_TRY(cudaMemsetAsync(m->ab.p, 0, (size_t)T * 2 * GH * 4, s), "memset a|b");
        if (uint32_t rc = qlinear(m, m->h.p, ab_rows, m->ab.p, T, H, 2 * GH, LG_EPI_RESID_F32, s)) return rc;
        LG_TRY(logismos_launch_gdn_prepare(p16, p16 + GW, m->ab.p, (const float*)m->ab.p + GH, L.A_log.p, L.dt_bias.p, m->g.p,
                                           m->beta.p, T, GH, GN, 2 * GH, s), "gdn_prepare");
        m->launches += 1;
      }
      // decode sequences (one token each, bound by the state traffic) run the token-serial kernel,
      // prefill sequences the chunk-parallel one; they are disjoint runs of the packed batch
      const float gscale = 1.0f / std::sqrt((float)kGdnDim);
      if (m->n_dec > 0 && !recurrence_done) {
        LG_TRY(logismos_launch_gdn_prefill(L.state.p, p16, p16 + GW, p16 + 2 * GW, m->g.p, m->beta.p, m->mix.p, p16 + 3 * GW,
                                           m->cu_all.p, m->state_slots.p, m->fresh.p, m->n_dec, GH, GN, gscale,
                                           1 | LG_GDN_STATIC_STATE /* states and index arrays date from before this step's first kernel */, s),
               "gdn recurrence (decode rows)");
        m->launches += 1;
      }
      if (m->n_pre > 0) {
        LG_TRY(logismos_launch_gdn_chunked(L.state.p, p16, p16 + GW, p16 + 2 * GW, m->g.p, m->beta.p, m->mix.p, p16 + 3 * GW,
                                           (const int32_t*)m->cu_all.p + m->n_dec, (const int32_t*)m->state_slots.p + m->n_dec,
                                           (const uint8_t*)m->fresh.p + m->n_dec, m->n_pre, GH, GN, gscale, m->gdn_scratch.p, T, s),
               "gdn chunk-parallel (prefill rows)");
        m->launches += 2;
      }
      if (uint32_t rc = out_proj(m, m->mix.p, L.w_out, T, GW, s)) return rc;
    }
    LG_TRY(logismos_launch_rms_norm_f32(m->x.p, L.norm2.p, m->h.p, T, H, c.rms_eps, 0, s), "rms_norm");
    m->launches += 1;
    if (uint32_t rc = qlinear(m, m->h.p, L.wgu, m->act.p, T, H, I, LG_EPI_SWIGLU, s)) return rc;
    if (uint32_t rc = out_proj(m, m->act.p, L.wdown, T, I, s)) return rc;
  }
  LG_TRY(logismos_launch_gather_rows_f32(m->x.p, m->last_idx.p, m->last.p, m->n_seqs, H, T, st, s), "gather_rows");
  LG_TRY(logismos_launch_rms_norm_f32(m->last.p, m->final_norm.p, m->last_bf16.p, m->n_seqs, H, c.rms_eps, 0, s), "final_norm");
  m->launches += 2;
  if (uint32_t rc = lm_head_and_greedy(m->lm_head, m->last_bf16.p, m->logits.p, m->tokens.p, m->n_seqs, H, st, &m->logits_f32,
                                       &m->launches, s)) {
    char buf[96];
    std::snprintf(buf, sizeof(buf), "lm_head / greedy failed: %s (code %u)", cudaGetErrorString((cudaError_t)rc), rc);
    set_error(buf);
    return LG_EMB_COMPUTE;
  }
  return 0;
}

uint32_t read_rows_bf16(Hybrid* m, const Buf& src, int n_seqs, size_t width, float* host_out, const char* what) {
  if (n_seqs != m->n_seqs) { set_error(std::string(what) + ": n_seqs differs from the last step"); return LG_EMB_COMPUTE; }
  cudaSetDevice(m->device);
  std::vector<uint16_t> tmp((size_t)n_seqs * width);
  LG_TRY(cudaDeviceSynchronize(), "device synchronize");
  LG_TRY(cudaMemcpy(tmp.data(), src.p, tmp.size() * 2, cudaMemcpyDeviceToHost), "D2H rows");
  for (int k = 0; k < n_seqs; ++k)
    for (size_t j = 0; j < width; ++j) {
      const uint32_t u = (uint32_t)tmp[(size_t)k * width + j] << 16;
      std::memcpy(&host_out[(size_t)m->order[k] * width + j], &u, 4);
    }
  return LG_EMB_OK;
}

}  // namespace

extern "C" {

uint32_t lg_hybrid_create(int32_t device, const lg_hybrid_config_t* cfg, const lg_hybrid_weights_t* w, void** model) {
  if (!cfg || !w || !model) { set_error("null argument"); return LG_EMB_COMPUTE; }
  *model = nullptr;
  const lg_hybrid_config_t& c = *cfg;
  if (c.hidden <= 0 || c.hidden % 128 || c.intermediate <= 0 || c.intermediate % 128 || c.n_layers < 0 || c.n_heads <= 0 ||
      c.n_kv_heads <= 0 || c.n_heads % c.n_kv_heads || c.n_heads / c.n_kv_heads > 16 ||
      (c.attn_head_dim != 128 && c.attn_head_dim != 256) || c.gdn_heads <= 0 || c.gdn_heads % 8 || c.full_attn_interval <= 0 ||
      c.n_pool_blocks <= 0 || c.max_blocks_per_seq <= 0 || c.max_step_tokens <= 0 || c.max_step_seqs <= 0 || c.max_pos <= 0 ||
      c.vocab <= 0 || c.n_state_slots <= 0) {
    set_error("unsupported hybrid config (attn_head_dim 128 or 256; gdn_heads a multiple of 8; hidden, intermediate multiples of 128)");
    return LG_EMB_COMPUTE;
  }
  if (cudaSetDevice(device) != cudaSuccess) { set_error("cudaSetDevice failed"); return LG_EMB_COMPUTE; }
  Hybrid* m = new Hybrid();
  m->cfg = c;
  m->device = device;
  m->qw = c.n_heads * c.attn_head_dim;
  m->kvw = c.n_kv_heads * c.attn_head_dim;
  m->attn_n = 2 * m->qw + 2 * m->kvw;
  m->gw = c.gdn_heads * kGdnDim;
  m->gdn_n = 4 * m->gw;
  m->mix_w = m->qw > m->gw ? m->qw : m->gw;
  const int H = c.hidden, I = c.intermediate, QW = m->qw, KW = m->kvw, GW = m->gw, GH = c.gdn_heads;
  bool ok = true;
  {
    std::vector<uint16_t> tmp((size_t)c.vocab * H);
    for (size_t i = 0; i < tmp.size(); ++i) tmp[i] = f32_to_bf16(w->tok_embed[i]);
    ok = ok && m->tok_embed.upload(tmp.data(), tmp.size() * 2);
  }
  ok = ok && m->final_norm.upload(w->final_norm, (size_t)H * 4);
  ok = ok && upload_q(m->lm_head, {&w->lm_head}, {c.vocab}, H);
  m->layers.resize(c.n_layers);
  const size_t pool_bytes = (size_t)c.n_pool_blocks * kBlock * KW * 2;
  const size_t state_bytes = (size_t)c.n_state_slots * GH * kGdnDim * kGdnDim * 4;
  for (int l = 0; l < c.n_layers && ok; ++l) {
    const lg_hybrid_layer_weights_t& lw = w->layers[l];
    HLayer& L = m->layers[l];
    L.full = (l + 1) % c.full_attn_interval == 0;
    ok = ok && L.norm1.upload(lw.norm1, (size_t)H * 4) && L.norm2.upload(lw.norm2, (size_t)H * 4);
    if (L.full) {
      ok = ok && upload_q(L.w_in, {&lw.wq, &lw.wk, &lw.wv, &lw.wgate}, {QW, KW, KW, QW}, H);
      ok = ok && upload_q(L.w_out, {&lw.wo}, {H}, QW);
      ok = ok && L.kpool.alloc(pool_bytes) && L.vpool.alloc(pool_bytes);
      ok = ok && cudaMemset(L.kpool.p, 0, pool_bytes) == cudaSuccess && cudaMemset(L.vpool.p, 0, pool_bytes) == cudaSuccess;
    } else {
      if (!lw.A_log || !lw.dt_bias) { ok = false; break; }
      ok = ok && upload_q(L.w_in, {&lw.wq, &lw.wk, &lw.wv, &lw.wgate, &lw.wa, &lw.wb}, {GW, GW, GW, GW, GH, GH}, H);
      ok = ok && upload_q(L.w_out, {&lw.wo}, {H}, GW);
      ok = ok && L.A_log.upload(lw.A_log, (size_t)GH * 4) && L.dt_bias.upload(lw.dt_bias, (size_t)GH * 4);
      ok = ok && L.state.alloc(state_bytes) && cudaMemset(L.state.p, 0, state_bytes) == cudaSuccess;
    }
    ok = ok && upload_q_gate_up(L.wgu, lw.w_gate, lw.w_up, I, H);
    ok = ok && upload_q(L.wdown, {&lw.w_down}, {H}, I);
    if (c.keep_bf16_copy) ok = ok && make_dense_copy(L.w_in) && make_dense_copy(L.w_out) && make_dense_copy(L.wgu) && make_dense_copy(L.wdown);
  }
  if (ok) {  // RoPE table in f64 then f32 (cpu_f32/mod.rs:599-619)
    const size_t half = c.attn_head_dim / 2;
    std::vector<float> cs((size_t)c.max_pos * half), sn((size_t)c.max_pos * half);
    for (int p = 0; p < c.max_pos; ++p)
      for (size_t i = 0; i < half; ++i) {
        const double ang = (double)p * std::pow(c.rope_theta, -(2.0 * (double)i) / (double)c.attn_head_dim);
        cs[p * half + i] = (float)std::cos(ang);
        sn[p * half + i] = (float)std::sin(ang);
      }
    ok = ok && m->cos.upload(cs.data(), cs.size() * 4) && m->sin.upload(sn.data(), sn.size() * 4);
  }
  const size_t T = c.max_step_tokens, S = c.max_step_seqs, MB = c.max_blocks_per_seq;
  const size_t pn = (size_t)(m->attn_n > m->gdn_n ? m->attn_n : m->gdn_n);
  size_t wmax = pn * H;
  if ((size_t)2 * I * H > wmax) wmax = (size_t)2 * I * H;
  if ((size_t)m->mix_w * H > wmax) wmax = (size_t)m->mix_w * H;
  m->max_chunks = S * ((MB * kBlock + kChunkTokens - 1) / kChunkTokens);
  const size_t acc_n = pn + 2 * GH > (size_t)2 * I ? pn + 2 * GH : (size_t)2 * I;
  ok = ok && m->x.alloc(T * H * 4) && m->delta.alloc(T * H * 4) && m->h.alloc(T * H * 2) && m->proj.alloc(T * pn * 2) && m->mix.alloc(T * m->mix_w * 2) &&
       m->qdec.alloc(S * QW * 2) && m->ab.alloc(T * 2 * GH * 4) && m->g.alloc(T * GH * 4) && m->beta.alloc(T * GH * 4) &&
       m->act.alloc(T * I * 2) && m->wscratch.alloc(wmax * 2) && m->last.alloc(S * H * 4) && m->last_bf16.alloc(S * H * 2) &&
       m->logits.alloc(S * (size_t)c.vocab * 4) && m->accws.alloc((size_t)kFusedDequantMaxRows * acc_n * 4) && m->tokens.alloc(S * 4) && m->status.alloc(4) && m->ids.alloc(T * 4) &&
       m->pos.alloc(T * 4) && m->slots.alloc(T * 8) && m->cu_all.alloc((S + 1) * 4) && m->cu_prefill.alloc((S + 1) * 4) &&
       m->last_idx.alloc(S * 4) && m->dec_ctx.alloc(S * 4) && m->dec_tables.alloc(S * MB * 4) && m->dec_chunks.alloc((S + 1) * 4) &&
       m->state_slots.alloc(S * 4) && m->fresh.alloc(S) && m->pre_kv.alloc(S * 4) &&
       m->gdn_scratch.alloc(logismos_gdn_chunked_scratch_bytes((int32_t)T, (int32_t)S, GH)) && m->gdn_pairs.alloc(S * GH * 4) &&
       m->dec_scratch.alloc(logismos_paged_decode_scratch_bytes((int32_t)m->max_chunks, c.n_heads, c.attn_head_dim));
  {
    // the attention workspace serves both prefill routes; the gather route holds one run of sequences at
    // a time, and any single sequence (at most a full block table) must fit
    m->prefix_cap_tokens = MB * kBlock > T ? MB * kBlock : T;
    size_t ws = logismos_varlen_attention_tc_scratch_bytes(c.max_step_tokens, c.max_step_seqs, c.n_kv_heads, c.attn_head_dim);
    const size_t ws2 = logismos_paged_prefix_attention_scratch_bytes((int32_t)m->prefix_cap_tokens, c.max_step_seqs, c.n_kv_heads, c.attn_head_dim);
    if (ws2 > ws) ws = ws2;
    ok = ok && m->attn_ws.alloc(ws);
  }
  ok = ok && cudaMemset(m->status.p, 0, 4) == cudaSuccess;
  m->accws_bytes = (size_t)kFusedDequantMaxRows * acc_n * 4;
  ok = ok && cudaMemset(m->accws.p, 0, m->accws_bytes) == cudaSuccess;
  ok = ok && cudaMemset(m->gdn_pairs.p, 0, S * GH * 4) == cudaSuccess;
  m->pinned_bytes = T * 16 + (S + 1) * 4 * 4 + S * MB * 4 + S * 4 + S * 4 + S * 4 + S + 64;
  ok = ok && cudaMallocHost((void**)&m->pinned, m->pinned_bytes) == cudaSuccess;
  ok = ok && cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking) == cudaSuccess;
  if (!ok) {
    set_error(std::string("lg_hybrid_create: missing weights, or allocation or upload failed: ") + cudaGetErrorString(cudaGetLastError()));
    lg_hybrid_destroy(m);
    return LG_EMB_COMPUTE;
  }
  *model = m;
  return LG_EMB_OK;
}

void lg_hybrid_destroy(void* model) {
  if (!model) return;
  Hybrid* m = static_cast<Hybrid*>(model);
  cudaSetDevice(m->device);
  Buf* bufs[] = {&m->delta, &m->tok_embed, &m->final_norm, &m->cos, &m->sin, &m->lm_head.codes, &m->lm_head.scales, &m->x, &m->h, &m->proj,
                 &m->mix, &m->qdec, &m->ab, &m->g, &m->beta, &m->act, &m->wscratch, &m->accws, &m->last, &m->last_bf16, &m->logits, &m->tokens,
                 &m->status, &m->ids, &m->pos, &m->slots, &m->cu_all, &m->cu_prefill, &m->last_idx, &m->dec_ctx, &m->dec_tables,
                 &m->dec_chunks, &m->dec_scratch, &m->attn_ws, &m->state_slots, &m->fresh, &m->pre_kv, &m->gdn_scratch, &m->gdn_pairs};
  for (Buf* b : bufs) b->release();
  for (auto& L : m->layers) {
    Buf* lb[] = {&L.norm1, &L.norm2, &L.kpool, &L.vpool, &L.state, &L.A_log, &L.dt_bias, &L.w_in.codes, &L.w_in.scales,
                 &L.w_ab.codes, &L.w_ab.scales, &L.w_out.codes, &L.w_out.scales, &L.wgu.codes, &L.wgu.scales, &L.wdown.codes,
                 &L.wdown.scales, &L.w_in.dense, &L.w_out.dense, &L.wgu.dense, &L.wdown.dense};
    for (Buf* b : lb) b->release();
  }
  if (m->pinned) cudaFreeHost(m->pinned);
  if (m->stream) cudaStreamDestroy(m->stream);
  delete m;
}

uint32_t lg_hybrid_step(void* model, const uint32_t* host_ids, const int32_t* cached, const int32_t* newl, int32_t n_seqs,
                        const int32_t* tables, const int32_t* state_slots, uint32_t* next_tokens) {
  Hybrid* m = static_cast<Hybrid*>(model);
  if (!m) { set_error("lg_hybrid_step: null model"); return LG_EMB_COMPUTE; }
  const lg_hybrid_config_t& c = m->cfg;
  if (n_seqs <= 0 || n_seqs > c.max_step_seqs || !host_ids || !cached || !newl || !tables || !state_slots || !next_tokens) {
    set_error("lg_hybrid_step: bad arguments or too many sequences for the workspace");
    return LG_EMB_COMPUTE;
  }
  std::lock_guard<std::mutex> lock(m->mu);
  if (cudaSetDevice(m->device) != cudaSuccess) { set_error("cudaSetDevice failed"); return LG_EMB_COMPUTE; }
  const int MB = c.max_blocks_per_seq;
  std::vector<int> order;
  std::vector<int64_t> src_off(n_seqs);
  std::vector<uint8_t> slot_used((size_t)c.n_state_slots, 0);
  int64_t off = 0, total = 0;
  for (int i = 0; i < n_seqs; ++i) {
    if (newl[i] <= 0 || cached[i] < 0) { set_error("lg_hybrid_step: every sequence needs >= 1 new token"); return LG_EMB_COMPUTE; }
    if ((int64_t)cached[i] + newl[i] > c.max_pos || (int64_t)cached[i] + newl[i] > (int64_t)MB * kBlock) {
      set_error("lg_hybrid_step: sequence exceeds max_pos or its block table");
      return LG_EMB_INPUT_TOO_LONG;
    }
    if (state_slots[i] < 0 || state_slots[i] >= c.n_state_slots || slot_used[state_slots[i]]) {
      set_error("lg_hybrid_step: state slot out of range or used twice in one step");
      return LG_EMB_COMPUTE;
    }
    slot_used[state_slots[i]] = 1;
    src_off[i] = off;
    off += newl[i];
    total += newl[i];
  }
  if (total > c.max_step_tokens) { set_error("lg_hybrid_step: step exceeds max_step_tokens"); return LG_EMB_COMPUTE; }
  for (int i = 0; i < n_seqs; ++i) if (newl[i] == 1) order.push_back(i);
  const int n_dec = (int)order.size();
  for (int i = 0; i < n_seqs; ++i) if (newl[i] > 1) order.push_back(i);
  const int n_pre = n_seqs - n_dec;
  uint8_t* pp = m->pinned;
  uint32_t* h_ids = (uint32_t*)pp; pp += (size_t)total * 4;
  int32_t* h_pos = (int32_t*)pp; pp += (size_t)total * 4;
  int64_t* h_slots = (int64_t*)pp; pp += (size_t)total * 8;
  int32_t* h_cu = (int32_t*)pp; pp += (size_t)(n_seqs + 1) * 4;
  int32_t* h_cu_pre = (int32_t*)pp; pp += (size_t)(n_seqs + 1) * 4;
  int32_t* h_last = (int32_t*)pp; pp += (size_t)(n_seqs + 1) * 4;
  int32_t* h_chunks = (int32_t*)pp; pp += (size_t)(n_seqs + 1) * 4;
  int32_t* h_tables = (int32_t*)pp; pp += (size_t)n_seqs * MB * 4;
  int32_t* h_ctx = (int32_t*)pp; pp += (size_t)n_seqs * 4;
  int32_t* h_state = (int32_t*)pp; pp += (size_t)n_seqs * 4;
  int32_t* h_prekv = (int32_t*)pp; pp += (size_t)n_seqs * 4;
  uint8_t* h_fresh = pp;
  std::vector<int32_t> o_cached(n_seqs), o_new(n_seqs), o_seqids((size_t)total);
  int64_t t = 0;
  for (int s = 0; s < n_seqs; ++s) {
    const int i = order[s];
    o_cached[s] = cached[i];
    o_new[s] = newl[i];
    h_state[s] = state_slots[i];
    h_fresh[s] = cached[i] == 0 ? 1 : 0;
    std::memcpy(h_tables + (size_t)s * MB, tables + (size_t)i * MB, (size_t)MB * 4);
    std::memcpy(h_ids + t, host_ids + src_off[i], (size_t)newl[i] * 4);
    t += newl[i];
  }
  const int64_t built = logismos_build_packing(o_cached.data(), o_new.data(), n_seqs, h_tables, MB, kBlock, c.n_pool_blocks, h_cu,
                                               h_pos, h_slots, o_seqids.data());
  if (built != total) { set_error("lg_hybrid_step: a block table entry is missing or outside the pool"); return LG_EMB_COMPUTE; }
  int max_pre = 0;
  bool has_prefix = false;
  h_cu_pre[0] = 0;
  for (int s = 0; s < n_seqs; ++s) {
    h_last[s] = h_cu[s + 1] - 1;
    if (s < n_dec) h_ctx[s] = o_cached[s] + 1;
    else {
      h_cu_pre[s - n_dec + 1] = h_cu[s + 1] - n_dec;
      h_prekv[s - n_dec] = o_cached[s] + o_new[s];
      if (o_cached[s] > 0) has_prefix = true;
      if (o_new[s] > max_pre) max_pre = o_new[s];
    }
  }
  std::vector<Hybrid::PrefixRun> runs;
  if (has_prefix) {
    Hybrid::PrefixRun r{0, 0, 0, 0, 0};
    for (int k = 0; k < n_pre; ++k) {
      const int kv = h_prekv[k], q = o_new[n_dec + k];
      if (r.s1 > r.s0 && (size_t)r.total_kv + kv > m->prefix_cap_tokens) { runs.push_back(r); r = Hybrid::PrefixRun{k, k, 0, 0, 0}; }
      r.s1 = k + 1; r.total_kv += kv;
      if (q > r.max_q) r.max_q = q;
      if (kv > r.max_kv) r.max_kv = kv;
    }
    runs.push_back(r);
  }
  m->chunk_tokens = n_dec > 0 ? logismos_pick_decode_chunk(h_ctx, n_dec, m->cfg.n_kv_heads, m->cfg.attn_head_dim) : kChunkTokens;
  const int total_chunks = n_dec > 0 ? logismos_build_decode_chunks(h_ctx, n_dec, m->chunk_tokens, h_chunks) : 0;
  if (total_chunks < 0 || (size_t)total_chunks > m->max_chunks) { set_error("lg_hybrid_step: decode chunk count exceeds the scratch"); return LG_EMB_COMPUTE; }
  m->T = (int)total; m->n_dec = n_dec; m->n_pre = n_pre; m->n_seqs = n_seqs; m->max_pre_len = max_pre; m->total_chunks = total_chunks;
  m->order = order;
  m->pre_has_prefix = has_prefix;
  m->prefix_runs = runs;
  cudaStream_t s = m->stream;
  LG_TRY(cudaMemsetAsync(m->status.p, 0, 4, s), "clear status");  // the status word describes this step only
  LG_TRY(cudaMemcpyAsync(m->ids.p, h_ids, (size_t)total * 4, cudaMemcpyHostToDevice, s), "H2D ids");
  LG_TRY(cudaMemcpyAsync(m->pos.p, h_pos, (size_t)total * 4, cudaMemcpyHostToDevice, s), "H2D positions");
  LG_TRY(cudaMemcpyAsync(m->slots.p, h_slots, (size_t)total * 8, cudaMemcpyHostToDevice, s), "H2D slots");
  LG_TRY(cudaMemcpyAsync(m->cu_all.p, h_cu, (size_t)(n_seqs + 1) * 4, cudaMemcpyHostToDevice, s), "H2D cu_seqlens");
  LG_TRY(cudaMemcpyAsync(m->cu_prefill.p, h_cu_pre, (size_t)(n_pre + 1) * 4, cudaMemcpyHostToDevice, s), "H2D prefill cu_seqlens");
  LG_TRY(cudaMemcpyAsync(m->last_idx.p, h_last, (size_t)n_seqs * 4, cudaMemcpyHostToDevice, s), "H2D last rows");
  LG_TRY(cudaMemcpyAsync(m->state_slots.p, h_state, (size_t)n_seqs * 4, cudaMemcpyHostToDevice, s), "H2D state slots");
  LG_TRY(cudaMemcpyAsync(m->fresh.p, h_fresh, (size_t)n_seqs, cudaMemcpyHostToDevice, s), "H2D fresh flags");
  if (n_dec > 0) {
    LG_TRY(cudaMemcpyAsync(m->dec_ctx.p, h_ctx, (size_t)n_dec * 4, cudaMemcpyHostToDevice, s), "H2D context lens");
    LG_TRY(cudaMemcpyAsync(m->dec_chunks.p, h_chunks, (size_t)(n_dec + 1) * 4, cudaMemcpyHostToDevice, s), "H2D chunk offsets");
  }
  if (n_dec > 0 || has_prefix)  // block tables in packed order: decode rows first, prefill rows after them
    LG_TRY(cudaMemcpyAsync(m->dec_tables.p, h_tables, (size_t)(has_prefix ? n_seqs : n_dec) * MB * 4, cudaMemcpyHostToDevice, s), "H2D block tables");
  if (has_prefix) LG_TRY(cudaMemcpyAsync(m->pre_kv.p, h_prekv, (size_t)n_pre * 4, cudaMemcpyHostToDevice, s), "H2D prefill key counts");
  if (uint32_t rc = run_device(m, s)) { m->acc_dirty = true; return rc; }
  std::vector<uint32_t> toks(n_seqs);
  LG_TRY(cudaMemcpyAsync(toks.data(), m->tokens.p, (size_t)n_seqs * 4, cudaMemcpyDeviceToHost, s), "D2H tokens");
  LG_TRY(cudaStreamSynchronize(s), "stream synchronize");
  for (int k = 0; k < n_seqs; ++k) next_tokens[order[k]] = toks[k];
  if (const int dev_status = lg_hybrid_device_status(m)) {
    m->acc_dirty = true;
    char buf[160];
    std::snprintf(buf, sizeof(buf), "device status 0x%x after a step of %d tokens in %d sequences (low byte 1: a range check failed, 2: a bounded wait expired in kernel family <next byte>, 3: a peer did not arrive)",
                  dev_status, (int)total, n_seqs);
    set_error(buf);
    return LG_EMB_COMPUTE;
  }
  return LG_EMB_OK;
}

uint32_t lg_hybrid_set_allreduce(void* model, lg_allreduce_f32_fn fn, void* user) {
  Hybrid* m = static_cast<Hybrid*>(model);
  if (!m) { set_error("lg_hybrid_set_allreduce: null model"); return LG_EMB_COMPUTE; }
  std::lock_guard<std::mutex> lock(m->mu);
  m->allreduce = fn;
  m->allreduce_user = user;
  m->reduce_add = nullptr;
  m->reduce_add_user = nullptr;
  return LG_EMB_OK;
}

uint32_t lg_hybrid_set_reduce_add(void* model, lg_reduce_add_f32_fn fn, void* user) {
  Hybrid* m = static_cast<Hybrid*>(model);
  if (!m) { set_error("lg_hybrid_set_reduce_add: null model"); return LG_EMB_COMPUTE; }
  std::lock_guard<std::mutex> lock(m->mu);
  m->reduce_add = fn;
  m->reduce_add_user = user;
  m->allreduce = nullptr;
  m->allreduce_user = nullptr;
  return LG_EMB_OK;
}

uint32_t lg_hybrid_replay_device(void* model, void* stream) {
  Hybrid* m = static_cast<Hybrid*>(model);
  if (!m || m->T <= 0) { set_error("lg_hybrid_replay_device: no step has run"); return LG_EMB_COMPUTE; }
  if (cudaSetDevice(m->device) != cudaSuccess) { set_error("cudaSetDevice failed"); return LG_EMB_COMPUTE; }
  return run_device(m, (cudaStream_t)stream);
}

uint32_t lg_hybrid_last_hidden(void* model, int32_t n_seqs, float* host_out) {
  Hybrid* m = static_cast<Hybrid*>(model);
  return read_rows_bf16(m, m->last_bf16, n_seqs, (size_t)m->cfg.hidden, host_out, "lg_hybrid_last_hidden");
}

uint32_t lg_hybrid_last_logits(void* model, int32_t n_seqs, float* host_out) {
  Hybrid* m = static_cast<Hybrid*>(model);
  if (!m->logits_f32) return read_rows_bf16(m, m->logits, n_seqs, (size_t)m->cfg.vocab, host_out, "lg_hybrid_last_logits");
  if (n_seqs != m->n_seqs) { set_error("lg_hybrid_last_logits: n_seqs differs from the last step"); return LG_EMB_COMPUTE; }
  cudaSetDevice(m->device);
  const size_t V = (size_t)m->cfg.vocab;
  std::vector<float> tmp((size_t)n_seqs * V);
  LG_TRY(cudaDeviceSynchronize(), "device synchronize");
  LG_TRY(cudaMemcpy(tmp.data(), m->logits.p, tmp.size() * 4, cudaMemcpyDeviceToHost), "D2H logits");
  for (int k = 0; k < n_seqs; ++k) std::memcpy(host_out + (size_t)m->order[k] * V, tmp.data() + (size_t)k * V, V * 4);
  return LG_EMB_OK;
}

int32_t lg_hybrid_launches_last_step(const void* model) { return static_cast<const Hybrid*>(model)->launches; }

int32_t lg_hybrid_device_status(void* model) {
  Hybrid* m = static_cast<Hybrid*>(model);
  int32_t v = -1;
  cudaSetDevice(m->device);
  if (cudaMemcpy(&v, m->status.p, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return v;
}

}  // extern "C"
