// Host-side executor of one continuous-batching step over a Qwen2-style decoder stack with int4
// group-32 weights and a paged KV cache (block 16). The reference has neither a decoder executor
// (crates/decoders/src/lib.rs:1-15) nor a scheduler (crates/sched/src/lib.rs:1-30); the contract
// kept is "a packed step equals running every sequence alone" through the causal variant of
// StellaLayer::forward (crates/encoders/src/stella.rs:190-206), lm_head and decode::greedy
// (crates/decode/src/lib.rs:73-83).
//
// A step packs decode tokens (one per sequence) first and prefill chunks after them:
//   embed -> per layer [ rms_norm -> QKV (int4 weights) + bias -> RoPE at each token's position ->
//   K/V rows scattered into the paged cache by slot mapping -> attention: paged decode kernel for
//   the decode rows, ragged causal attention for the prefill rows (over the chunk's own rows when every
//   chunk starts its sequence, else over keys and values gathered from the cache through the block
//   tables, so a chunk may continue a cached sequence) -> o_proj + residual ->
//   rms_norm -> gate/up with SwiGLU fused in the GEMM epilogue -> down + residual ] -> last token rows -> final norm ->
//   lm_head (int4 GEMV) -> greedy argmax.
// Contractions over the packed rows run on the tcgen05 GEMM over a per-layer bf16 expansion of the
// int4 codes; the lm_head, whose batch is the number of sequences, runs on the int4 GEMV kernel.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "logismos_kernels.h"
#include "logismos_model.h"

#include "model_util.h"

namespace {

using namespace lgm;

struct DLayer {
  Buf norm1, norm2, bqkv, kpool, vpool;
  QMat wqkv, wo, wgu, wdown;
};

constexpr int kChunkTokens = 512;
constexpr int kBlock = 16;

struct Decoder {
  lg_decoder_config_t cfg{};
  int device = 0, head_dim = 0, qkv_dim = 0, kv_dim = 0;
  Buf tok_embed, final_norm, cos, sin;
  QMat lm_head;
  std::vector<DLayer> layers;
  // workspace
  Buf x, h, qkv, attn, qdec, gu, act, wscratch, accws, last, last_bf16, logits, tokens, status;
  Buf ids, pos, slots, cu_prefill, last_idx, dec_ctx, dec_tables, dec_chunks, dec_scratch, attn_ws, pre_kv;
  // pinned staging (one block)
  uint8_t* pinned = nullptr;
  size_t pinned_bytes = 0;
  cudaStream_t stream = nullptr;
  std::mutex mu;
  // description of the last step (for replay and diagnostics)
  int T = 0, n_dec = 0, n_pre = 0, n_seqs = 0, pre_tokens = 0, max_pre_len = 0, total_chunks = 0, chunk_tokens = kChunkTokens, launches = 0, logits_f32 = 0;
  std::vector<int> order;  // internal slot -> caller's sequence index
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

uint32_t qlinear(Decoder* m, const void* a, const QMat& w, const void* bias, void* out, int T, int lda, int ldc,
                 int epi, cudaStream_t s) {
  LG_TRY(qlinear_any(a, w, bias, out, T, lda, ldc, epi, m->wscratch.p, m->accws.p, m->status.p, &m->launches, s), "int4 linear");
  return 0;
}

uint32_t run_device(Decoder* m, cudaStream_t s) {
  const lg_decoder_config_t& c = m->cfg;
  const int H = c.hidden, I = c.intermediate, D = m->head_dim, QKV = m->qkv_dim, KV = m->kv_dim, T = m->T;
  void* st = m->status.p;
  m->launches = 0;
  if (m->acc_dirty) {
    LG_TRY(cudaMemsetAsync(m->accws.p, 0, m->accws_bytes, s), "clear accumulation workspace");
    m->acc_dirty = false;
  }
  LG_TRY(logismos_launch_embed_lookup_bf16(m->tok_embed.p, m->ids.p, m->x.p, T, H, c.vocab, s), "embed_lookup");
  m->launches += 1;
  for (int l = 0; l < c.n_layers; ++l) {
    DLayer& L = m->layers[l];
    LG_TRY(logismos_launch_rms_norm_f32(m->x.p, L.norm1.p, m->h.p, T, H, c.rms_eps, 0, s), "rms_norm");
    if (uint32_t rc = qlinear(m, m->h.p, L.wqkv, L.bqkv.p, m->qkv.p, T, H, QKV, LG_EPI_BF16, s)) return rc;
    LG_TRY(logismos_launch_rope_halves_bf16(m->qkv.p, m->cos.p, m->sin.p, m->pos.p, T, c.n_heads + c.n_kv_heads, D, QKV,
                                            c.max_pos, st, s), "rope");
    const uint16_t* qkv16 = (const uint16_t*)m->qkv.p;
    if (c.kv_turbo3) {
      // TurboQuant 3-bit cache: rows are encoded on the way in and every sequence of the step (decode
      // tokens are chunks of one query) attends through the decoding gather, run by run
      LG_TRY(logismos_launch_paged_kv_store_turbo3(qkv16 + H, qkv16 + H + KV, QKV, L.kpool.p, L.vpool.p, m->slots.p, T, KV,
                                                   (int64_t)c.n_pool_blocks * kBlock, st, s), "paged_kv_store_turbo3");
      m->launches += 3;
      for (const Decoder::PrefixRun& r : m->prefix_runs) {
        LG_TRY(logismos_launch_paged_prefix_attention_turbo3_bf16(
                   qkv16, QKV, (const int32_t*)m->cu_prefill.p + r.s0, (const int32_t*)m->pre_kv.p + r.s0, L.kpool.p, L.vpool.p,
                   (const int32_t*)m->dec_tables.p + (size_t)r.s0 * c.max_blocks_per_seq, c.max_blocks_per_seq, c.n_pool_blocks, m->attn.p,
                   m->attn_ws.p, T, r.total_kv, r.s1 - r.s0, r.max_q, r.max_kv, c.n_heads, c.n_kv_heads, D, st, s),
               "paged_prefix_attention_turbo3");
        m->launches += 2;
      }
    } else {
    LG_TRY(logismos_launch_paged_kv_store_bf16(qkv16 + H, qkv16 + H + KV, QKV, L.kpool.p, L.vpool.p, m->slots.p, T, KV,
                                               (int64_t)c.n_pool_blocks * kBlock, st, s), "paged_kv_store");
    m->launches += 3;
    if (m->n_dec > 0) {
      // decode rows are the first n_dec rows of the packed batch: gather their q heads contiguously
      LG_TRY(cudaMemcpy2DAsync(m->qdec.p, (size_t)H * 2, m->qkv.p, (size_t)QKV * 2, (size_t)H * 2, m->n_dec,
                               cudaMemcpyDeviceToDevice, s), "q gather");
      LG_TRY(logismos_launch_paged_attention_decode_bf16(m->qdec.p, L.kpool.p, L.vpool.p, nullptr, nullptr, m->dec_tables.p,
                                                         m->dec_ctx.p, m->dec_chunks.p, m->attn.p, m->dec_scratch.p, st, m->n_dec,
                                                         m->total_chunks, m->chunk_tokens, c.max_blocks_per_seq, c.n_pool_blocks,
                                                         c.n_heads, c.n_kv_heads, D, s), "paged_attention_decode");
      m->launches += 2;
    }
    if (m->n_pre > 0 && m->pre_has_prefix) {
      // some chunk continues a cached sequence: keys and values come from the cache (the chunk's own rows
      // were stored above), gathered per run of sequences into attn_ws
      const int32_t* tabs = (const int32_t*)m->dec_tables.p + (size_t)m->n_dec * c.max_blocks_per_seq;
      for (const Decoder::PrefixRun& r : m->prefix_runs) {
        LG_TRY(logismos_launch_paged_prefix_attention_tc_bf16(
                   qkv16 + (size_t)m->n_dec * QKV, QKV, (const int32_t*)m->cu_prefill.p + r.s0, (const int32_t*)m->pre_kv.p + r.s0,
                   L.kpool.p, L.vpool.p, tabs + (size_t)r.s0 * c.max_blocks_per_seq, c.max_blocks_per_seq, c.n_pool_blocks,
                   (uint16_t*)m->attn.p + (size_t)m->n_dec * H, m->attn_ws.p, T - m->n_dec, r.total_kv, r.s1 - r.s0, r.max_q, r.max_kv,
                   c.n_heads, c.n_kv_heads, D, st, s),
               "paged_prefix_attention");
        m->launches += 2;
      }
    } else if (m->n_pre > 0) {  // tcgen05 kernel; V transposed into attn_ws first
      LG_TRY(logismos_launch_varlen_attention_tc_bf16(qkv16 + (size_t)m->n_dec * QKV, m->cu_prefill.p,
                                                      (uint16_t*)m->attn.p + (size_t)m->n_dec * H, m->attn_ws.p, T - m->n_dec,
                                                      m->n_pre, m->max_pre_len, c.n_heads, c.n_kv_heads, D, QKV, H, H + KV, 1, st, s),
             "varlen_attention");
      m->launches += 2;
    }
    }
    if (uint32_t rc = qlinear(m, m->attn.p, L.wo, nullptr, m->x.p, T, H, H, LG_EPI_RESID_F32, s)) return rc;
    LG_TRY(logismos_launch_rms_norm_f32(m->x.p, L.norm2.p, m->h.p, T, H, c.rms_eps, 0, s), "rms_norm");
    if (uint32_t rc = qlinear(m, m->h.p, L.wgu, nullptr, m->act.p, T, H, I, LG_EPI_SWIGLU, s)) return rc;
    if (uint32_t rc = qlinear(m, m->act.p, L.wdown, nullptr, m->x.p, T, I, H, LG_EPI_RESID_F32, s)) return rc;
    m->launches += 1;
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

}  // namespace

extern "C" {

uint32_t lg_decoder_create(int32_t device, const lg_decoder_config_t* cfg, const lg_decoder_weights_t* w, void** model) {
  if (!cfg || !w || !model) { set_error("null argument"); return LG_EMB_COMPUTE; }
  *model = nullptr;
  const lg_decoder_config_t& c = *cfg;
  if (c.hidden <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.hidden % c.n_heads || c.n_heads % c.n_kv_heads ||
      c.hidden / c.n_heads != 128 || c.hidden % 128 || c.intermediate % 128 || c.n_layers < 0 || c.n_pool_blocks <= 0 ||
      c.max_blocks_per_seq <= 0 || c.max_step_tokens <= 0 || c.max_step_seqs <= 0 || c.max_pos <= 0 || c.vocab <= 0 ||
      c.n_heads / c.n_kv_heads > 16) {
    set_error("unsupported decoder config (head_dim must be 128; hidden and intermediate multiples of 128)");
    return LG_EMB_COMPUTE;
  }
  if (cudaSetDevice(device) != cudaSuccess) { set_error("cudaSetDevice failed"); return LG_EMB_COMPUTE; }
  Decoder* m = new Decoder();
  m->cfg = c;
  m->device = device;
  m->head_dim = c.hidden / c.n_heads;
  m->kv_dim = c.n_kv_heads * m->head_dim;
  m->qkv_dim = c.hidden + 2 * m->kv_dim;
  const size_t H = c.hidden, I = c.intermediate, KV = m->kv_dim, QKV = m->qkv_dim;
  bool ok = true;
  {
    std::vector<uint16_t> tmp((size_t)c.vocab * H);
    for (size_t i = 0; i < tmp.size(); ++i) tmp[i] = f32_to_bf16(w->tok_embed[i]);
    ok = ok && m->tok_embed.upload(tmp.data(), tmp.size() * 2);
  }
  ok = ok && m->final_norm.upload(w->final_norm, H * 4);
  ok = ok && upload_q(m->lm_head, {&w->lm_head}, {c.vocab}, (int)H);
  m->layers.resize(c.n_layers);
  const size_t pool_bytes = (size_t)c.n_pool_blocks * kBlock * (c.kv_turbo3 ? logismos_turbo3_row_bytes((int32_t)KV) : KV * 2);
  for (int l = 0; l < c.n_layers && ok; ++l) {
    const lg_decoder_layer_weights_t& lw = w->layers[l];
    DLayer& L = m->layers[l];
    ok = ok && L.norm1.upload(lw.norm1, H * 4) && L.norm2.upload(lw.norm2, H * 4);
    std::vector<float> b(QKV);
    std::memcpy(b.data(), lw.bq, H * 4);
    std::memcpy(b.data() + H, lw.bk, KV * 4);
    std::memcpy(b.data() + H + KV, lw.bv, KV * 4);
    ok = ok && L.bqkv.upload(b.data(), QKV * 4);
    ok = ok && upload_q(L.wqkv, {&lw.wq, &lw.wk, &lw.wv}, {(int)H, (int)KV, (int)KV}, (int)H);
    ok = ok && upload_q(L.wo, {&lw.wo}, {(int)H}, (int)H);
    ok = ok && upload_q_gate_up(L.wgu, lw.w_gate, lw.w_up, (int)I, (int)H);
    ok = ok && upload_q(L.wdown, {&lw.w_down}, {(int)H}, (int)I);
    if (c.keep_bf16_copy) ok = ok && make_dense_copy(L.wqkv) && make_dense_copy(L.wo) && make_dense_copy(L.wgu) && make_dense_copy(L.wdown);
    ok = ok && L.kpool.alloc(pool_bytes) && L.vpool.alloc(pool_bytes);
    ok = ok && cudaMemset(L.kpool.p, 0, pool_bytes) == cudaSuccess && cudaMemset(L.vpool.p, 0, pool_bytes) == cudaSuccess;
  }
  if (ok) {  // RoPE table in f64 then f32 (cpu_f32/mod.rs:599-619)
    const size_t half = m->head_dim / 2;
    std::vector<float> cs((size_t)c.max_pos * half), sn((size_t)c.max_pos * half);
    for (int p = 0; p < c.max_pos; ++p)
      for (size_t i = 0; i < half; ++i) {
        const double ang = (double)p * std::pow(c.rope_theta, -(2.0 * (double)i) / (double)m->head_dim);
        cs[p * half + i] = (float)std::cos(ang);
        sn[p * half + i] = (float)std::sin(ang);
      }
    ok = ok && m->cos.upload(cs.data(), cs.size() * 4) && m->sin.upload(sn.data(), sn.size() * 4);
  }
  const size_t T = c.max_step_tokens, S = c.max_step_seqs, MB = c.max_blocks_per_seq;
  size_t wmax = QKV * H;
  if (2 * I * H > wmax) wmax = 2 * I * H;
  // every sequence of a step may be a decode sequence of up to max_blocks_per_seq blocks
  m->max_chunks = S * ((MB * kBlock + kChunkTokens - 1) / kChunkTokens);
  const size_t acc_n = QKV > 2 * I ? QKV : 2 * I;
  ok = ok && m->x.alloc(T * H * 4) && m->h.alloc(T * H * 2) && m->qkv.alloc(T * QKV * 2) && m->attn.alloc(T * H * 2) &&
       m->qdec.alloc(S * H * 2) && m->gu.alloc(16) && m->act.alloc(T * I * 2) && m->wscratch.alloc(wmax * 2) &&
       m->last.alloc(S * H * 4) && m->last_bf16.alloc(S * H * 2) && m->logits.alloc(S * (size_t)c.vocab * 4) && m->accws.alloc((size_t)kFusedDequantMaxRows * acc_n * 4) &&
       m->tokens.alloc(S * 4) && m->status.alloc(4) && m->ids.alloc(T * 4) && m->pos.alloc(T * 4) && m->slots.alloc(T * 8) &&
       m->cu_prefill.alloc((S + 1) * 4) && m->last_idx.alloc(S * 4) && m->dec_ctx.alloc(S * 4) && m->dec_tables.alloc(S * MB * 4) &&
       m->dec_chunks.alloc((S + 1) * 4) && m->pre_kv.alloc(S * 4) &&
       m->dec_scratch.alloc(logismos_paged_decode_scratch_bytes((int32_t)m->max_chunks, c.n_heads, m->head_dim));
  {
    // the attention workspace serves both prefill routes; the gather route holds one run of sequences at
    // a time, and any single sequence (at most a full block table) must fit
    m->prefix_cap_tokens = MB * kBlock > T ? MB * kBlock : T;
    if (c.kv_turbo3) {  // every sequence of a step goes through the gather: room for many contexts at once
      const size_t all = S * MB * kBlock, cap = (size_t)512 * 1024;
      m->prefix_cap_tokens = all < cap ? all : cap;
      if (m->prefix_cap_tokens < MB * kBlock) m->prefix_cap_tokens = MB * kBlock;
    }
    size_t ws = logismos_varlen_attention_tc_scratch_bytes((int32_t)T, (int32_t)S, c.n_kv_heads, 128);
    const size_t ws2 = logismos_paged_prefix_attention_scratch_bytes((int32_t)m->prefix_cap_tokens, (int32_t)S, c.n_kv_heads, 128);
    if (ws2 > ws) ws = ws2;
    ok = ok && m->attn_ws.alloc(ws);
  }
  ok = ok && cudaMemset(m->status.p, 0, 4) == cudaSuccess;
  m->accws_bytes = (size_t)kFusedDequantMaxRows * acc_n * 4;
  ok = ok && cudaMemset(m->accws.p, 0, m->accws_bytes) == cudaSuccess;
  m->pinned_bytes = T * 16 + (S + 1) * 4 * 4 + S * MB * 4 + S * 4 + S * 4;
  ok = ok && cudaMallocHost((void**)&m->pinned, m->pinned_bytes) == cudaSuccess;
  ok = ok && cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking) == cudaSuccess;
  if (!ok) {
    set_error(std::string("lg_decoder_create: allocation or upload failed: ") + cudaGetErrorString(cudaGetLastError()));
    lg_decoder_destroy(m);
    return LG_EMB_COMPUTE;
  }
  *model = m;
  return LG_EMB_OK;
}

void lg_decoder_destroy(void* model) {
  if (!model) return;
  Decoder* m = static_cast<Decoder*>(model);
  cudaSetDevice(m->device);
  Buf* bufs[] = {&m->tok_embed, &m->final_norm, &m->cos, &m->sin, &m->lm_head.codes, &m->lm_head.scales, &m->x, &m->h, &m->qkv,
                 &m->attn, &m->qdec, &m->gu, &m->act, &m->wscratch, &m->accws, &m->last, &m->last_bf16, &m->logits, &m->tokens, &m->status,
                 &m->ids, &m->pos, &m->slots, &m->cu_prefill, &m->last_idx, &m->dec_ctx, &m->dec_tables, &m->dec_chunks, &m->dec_scratch, &m->attn_ws, &m->pre_kv};
  for (Buf* b : bufs) b->release();
  for (auto& L : m->layers) {
    Buf* lb[] = {&L.norm1, &L.norm2, &L.bqkv, &L.kpool, &L.vpool, &L.wqkv.codes, &L.wqkv.scales, &L.wo.codes, &L.wo.scales,
                 &L.wgu.codes, &L.wgu.scales, &L.wdown.codes, &L.wdown.scales, &L.wqkv.dense, &L.wo.dense, &L.wgu.dense, &L.wdown.dense};
    for (Buf* b : lb) b->release();
  }
  if (m->pinned) cudaFreeHost(m->pinned);
  if (m->stream) cudaStreamDestroy(m->stream);
  delete m;
}

uint32_t lg_decoder_step(void* model, const uint32_t* host_ids, const int32_t* cached, const int32_t* newl, int32_t n_seqs,
                         const int32_t* tables, uint32_t* next_tokens) {
  Decoder* m = static_cast<Decoder*>(model);
  const lg_decoder_config_t& c = m->cfg;
  if (n_seqs <= 0 || n_seqs > c.max_step_seqs || !host_ids || !cached || !newl || !tables || !next_tokens) {
    set_error("lg_decoder_step: bad arguments or too many sequences for the workspace");
    return LG_EMB_COMPUTE;
  }
  std::lock_guard<std::mutex> lock(m->mu);
  if (cudaSetDevice(m->device) != cudaSuccess) { set_error("cudaSetDevice failed"); return LG_EMB_COMPUTE; }
  const int MB = c.max_blocks_per_seq;
  // internal order: decode sequences first, then prefill chunks
  std::vector<int> order;
  std::vector<int64_t> src_off(n_seqs);
  int64_t off = 0, total = 0;
  for (int i = 0; i < n_seqs; ++i) {
    if (newl[i] <= 0 || cached[i] < 0) { set_error("lg_decoder_step: every sequence needs >= 1 new token"); return LG_EMB_COMPUTE; }
    if ((int64_t)cached[i] + newl[i] > c.max_pos || (int64_t)cached[i] + newl[i] > (int64_t)MB * kBlock) {
      set_error("lg_decoder_step: sequence exceeds max_pos or its block table");
      return LG_EMB_INPUT_TOO_LONG;
    }
    src_off[i] = off;
    off += newl[i];
    total += newl[i];
  }
  if (total > c.max_step_tokens) { set_error("lg_decoder_step: step exceeds max_step_tokens"); return LG_EMB_COMPUTE; }
  for (int i = 0; i < n_seqs; ++i) if (newl[i] == 1) order.push_back(i);
  const int n_dec = (int)order.size();
  for (int i = 0; i < n_seqs; ++i) if (newl[i] > 1) order.push_back(i);
  const int n_pre = n_seqs - n_dec;
  // carve the pinned block
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
  int32_t* h_prekv = (int32_t*)pp;
  std::vector<int32_t> o_cached(n_seqs), o_new(n_seqs), o_seqids((size_t)total);
  int64_t t = 0;
  for (int s = 0; s < n_seqs; ++s) {
    const int i = order[s];
    o_cached[s] = cached[i];
    o_new[s] = newl[i];
    std::memcpy(h_tables + (size_t)s * MB, tables + (size_t)i * MB, (size_t)MB * 4);
    std::memcpy(h_ids + t, host_ids + src_off[i], (size_t)newl[i] * 4);
    t += newl[i];
  }
  const int64_t built = logismos_build_packing(o_cached.data(), o_new.data(), n_seqs, h_tables, MB, kBlock, c.n_pool_blocks, h_cu,
                                               h_pos, h_slots, o_seqids.data());
  if (built != total) { set_error("lg_decoder_step: a block table entry is missing or outside the pool"); return LG_EMB_COMPUTE; }
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
  std::vector<Decoder::PrefixRun> runs;
  const bool t3 = c.kv_turbo3 != 0;
  if (t3) {  // all sequences, packed order: key counts and query offsets of the whole step
    has_prefix = true;
    for (int k = 0; k < n_seqs; ++k) h_prekv[k] = o_cached[k] + o_new[k];
    std::memcpy(h_cu_pre, h_cu, (size_t)(n_seqs + 1) * 4);
  }
  const int run_first = t3 ? 0 : n_dec, run_count = t3 ? n_seqs : n_pre;
  if (has_prefix) {
    Decoder::PrefixRun r{0, 0, 0, 0, 0};
    for (int k = 0; k < run_count; ++k) {
      const int kv = h_prekv[k], q = o_new[run_first + k];
      if (r.s1 > r.s0 && (size_t)r.total_kv + kv > m->prefix_cap_tokens) { runs.push_back(r); r = Decoder::PrefixRun{k, k, 0, 0, 0}; }
      r.s1 = k + 1; r.total_kv += kv;
      if (q > r.max_q) r.max_q = q;
      if (kv > r.max_kv) r.max_kv = kv;
    }
    runs.push_back(r);
  }
  m->chunk_tokens = n_dec > 0 ? logismos_pick_decode_chunk(h_ctx, n_dec, m->cfg.n_kv_heads, m->head_dim) : kChunkTokens;
  const int total_chunks = n_dec > 0 ? logismos_build_decode_chunks(h_ctx, n_dec, m->chunk_tokens, h_chunks) : 0;
  if (total_chunks < 0 || (size_t)total_chunks > m->max_chunks) { set_error("lg_decoder_step: decode chunk count exceeds the scratch"); return LG_EMB_COMPUTE; }
  m->T = (int)total; m->n_dec = n_dec; m->n_pre = n_pre; m->n_seqs = n_seqs; m->max_pre_len = max_pre; m->total_chunks = total_chunks;
  m->order = order;
  m->pre_has_prefix = has_prefix;
  m->prefix_runs = runs;
  cudaStream_t s = m->stream;
  LG_TRY(cudaMemsetAsync(m->status.p, 0, 4, s), "clear status");  // the status word describes this step only
  LG_TRY(cudaMemcpyAsync(m->ids.p, h_ids, (size_t)total * 4, cudaMemcpyHostToDevice, s), "H2D ids");
  LG_TRY(cudaMemcpyAsync(m->pos.p, h_pos, (size_t)total * 4, cudaMemcpyHostToDevice, s), "H2D positions");
  LG_TRY(cudaMemcpyAsync(m->slots.p, h_slots, (size_t)total * 8, cudaMemcpyHostToDevice, s), "H2D slots");
  LG_TRY(cudaMemcpyAsync(m->cu_prefill.p, h_cu_pre, (size_t)(run_count + 1) * 4, cudaMemcpyHostToDevice, s), "H2D cu_seqlens");
  LG_TRY(cudaMemcpyAsync(m->last_idx.p, h_last, (size_t)n_seqs * 4, cudaMemcpyHostToDevice, s), "H2D last rows");
  if (n_dec > 0) {
    LG_TRY(cudaMemcpyAsync(m->dec_ctx.p, h_ctx, (size_t)n_dec * 4, cudaMemcpyHostToDevice, s), "H2D context lens");
    LG_TRY(cudaMemcpyAsync(m->dec_chunks.p, h_chunks, (size_t)(n_dec + 1) * 4, cudaMemcpyHostToDevice, s), "H2D chunk offsets");
  }
  if (n_dec > 0 || has_prefix)  // block tables in packed order: decode rows first, prefill rows after them
    LG_TRY(cudaMemcpyAsync(m->dec_tables.p, h_tables, (size_t)(has_prefix ? n_seqs : n_dec) * MB * 4, cudaMemcpyHostToDevice, s), "H2D block tables");
  if (has_prefix) LG_TRY(cudaMemcpyAsync(m->pre_kv.p, h_prekv, (size_t)run_count * 4, cudaMemcpyHostToDevice, s), "H2D prefill key counts");
  if (uint32_t rc = run_device(m, s)) { m->acc_dirty = true; return rc; }
  std::vector<uint32_t> toks(n_seqs);
  LG_TRY(cudaMemcpyAsync(toks.data(), m->tokens.p, (size_t)n_seqs * 4, cudaMemcpyDeviceToHost, s), "D2H tokens");
  LG_TRY(cudaStreamSynchronize(s), "stream synchronize");
  for (int k = 0; k < n_seqs; ++k) next_tokens[order[k]] = toks[k];
  if (const int dev_status = lg_decoder_device_status(m)) {
    m->acc_dirty = true;
    char buf[160];
    std::snprintf(buf, sizeof(buf), "device status 0x%x after a step of %d tokens in %d sequences (low byte 1: a range check failed, 2: a bounded wait expired in kernel family <next byte>, 3: a peer did not arrive)",
                  dev_status, (int)total, n_seqs);
    set_error(buf);
    return LG_EMB_COMPUTE;
  }
  return LG_EMB_OK;
}

uint32_t lg_decoder_replay_device(void* model, void* stream) {
  Decoder* m = static_cast<Decoder*>(model);
  if (m->T <= 0) { set_error("lg_decoder_replay_device: no step has run"); return LG_EMB_COMPUTE; }
  if (cudaSetDevice(m->device) != cudaSuccess) { set_error("cudaSetDevice failed"); return LG_EMB_COMPUTE; }
  return run_device(m, (cudaStream_t)stream);
}

uint32_t lg_decoder_last_hidden(void* model, int32_t n_seqs, float* host_out) {
  Decoder* m = static_cast<Decoder*>(model);
  if (n_seqs != m->n_seqs) { set_error("lg_decoder_last_hidden: n_seqs differs from the last step"); return LG_EMB_COMPUTE; }
  cudaSetDevice(m->device);
  const size_t H = m->cfg.hidden;
  std::vector<uint16_t> tmp((size_t)n_seqs * H);
  LG_TRY(cudaDeviceSynchronize(), "device synchronize");
  LG_TRY(cudaMemcpy(tmp.data(), m->last_bf16.p, tmp.size() * 2, cudaMemcpyDeviceToHost), "D2H hidden");
  for (int k = 0; k < n_seqs; ++k)
    for (size_t j = 0; j < H; ++j) {
      const uint32_t u = (uint32_t)tmp[(size_t)k * H + j] << 16;
      std::memcpy(&host_out[(size_t)m->order[k] * H + j], &u, 4);
    }
  return LG_EMB_OK;
}

uint32_t lg_decoder_last_logits(void* model, int32_t n_seqs, float* host_out) {
  Decoder* m = static_cast<Decoder*>(model);
  if (n_seqs != m->n_seqs) { set_error("lg_decoder_last_logits: n_seqs differs from the last step"); return LG_EMB_COMPUTE; }
  cudaSetDevice(m->device);
  const size_t V = m->cfg.vocab;
  LG_TRY(cudaDeviceSynchronize(), "device synchronize");
  if (m->logits_f32) {
    std::vector<float> tmp((size_t)n_seqs * V);
    LG_TRY(cudaMemcpy(tmp.data(), m->logits.p, tmp.size() * 4, cudaMemcpyDeviceToHost), "D2H logits");
    for (int k = 0; k < n_seqs; ++k) std::memcpy(host_out + (size_t)m->order[k] * V, tmp.data() + (size_t)k * V, V * 4);
    return LG_EMB_OK;
  }
  std::vector<uint16_t> tmp((size_t)n_seqs * V);
  LG_TRY(cudaMemcpy(tmp.data(), m->logits.p, tmp.size() * 2, cudaMemcpyDeviceToHost), "D2H logits");
  for (int k = 0; k < n_seqs; ++k)
    for (size_t j = 0; j < V; ++j) {
      const uint32_t u = (uint32_t)tmp[(size_t)k * V + j] << 16;
      std::memcpy(&host_out[(size_t)m->order[k] * V + j], &u, 4);
    }
  return LG_EMB_OK;
}

int32_t lg_decoder_launches_last_step(const void* model) { return static_cast<const Decoder*>(model)->launches; }

int32_t lg_decoder_device_status(void* model) {
  Decoder* m = static_cast<Decoder*>(model);
  int32_t v = -1;
  cudaSetDevice(m->device);
  if (cudaMemcpy(&v, m->status.p, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return v;
}

}  // extern "C"
