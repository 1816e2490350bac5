/*
 * CPU oracle for the logismos inference hot path.
 *
 * TEST INFRASTRUCTURE ONLY. This library restates, in plain C++ fp32, the
 * arithmetic of the reference's CPU path so that the CUDA kernels can be
 * checked against it and so that a CPU baseline can be timed beside them.
 * Nothing in the shipped package links, loads or calls it; only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * Parity status, per group of functions:
 *   - cpu_f32 kernels, attention/MLP/encoder composition, TurboQuant nibble
 *     packing, flat KV cache rows, gated delta rule, greedy argmax, fp16 op
 *     references: restated from the reference sources cited beside each
 *     function and pinned against the known-answer vectors in the reference's
 *     own unit tests (see tests/test_oracle_*.py).
 *   - GEMM summation order: the reference delegates to the third-party crate
 *     `matrixmultiply` 0.3 (patch version unpinned, Cargo.lock is ignored in
 *     the reference tree); its fp32 summation order is unspecified, so GEMM
 *     bearing results are pinned to tolerance, not bit-exactly.
 *   - int4 group-32 GEMV, paged KV cache / paged decode attention, ragged
 *     packing indices, GDN gate preprocessing: the reference has no
 *     implementation. PARITY UNPINNED for those: the oracle is this build's
 *     own fp32 definition, constrained by equivalences with pinned functions
 *     (dequantise + linear_t, flat-cache gather + attention, per-sequence
 *     execution) that the tests check.
 */
#pragma once
#include <cstddef>
#include <cstdint>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- crates/kernels/src/cpu_f32/mod.rs ---------------------------------- */
void orc_embed_lookup(const float* weight, size_t hidden, size_t vocab,
                      const uint32_t* ids, size_t n_ids, float* out);
void orc_rms_norm(const float* x, const float* w, size_t rows, size_t n, float eps, float* y);
/* returns 0 on success, nonzero where the reference would panic */
int orc_linear(const float* a, size_t a_len, const float* b, size_t b_len,
               const float* bias, size_t bias_len, size_t m, size_t n, size_t k, float* c);
int orc_linear_t(const float* a, size_t a_len, const float* b, size_t b_len,
                 const float* bias, size_t bias_len, size_t m, size_t n, size_t k, float* c);
void orc_silu(const float* x, size_t n, float* y);
int orc_hadamard(const float* a, size_t a_len, const float* b, size_t b_len, float* c);
void orc_softmax_last_dim(const float* x, size_t rows, size_t n, float* y);
int orc_mask_additive_in_place(float* scores, size_t scores_len, const uint8_t* mask,
                               size_t mask_len, size_t rows, size_t n);
void orc_rope_halves_in_place(float* x, const float* cos, const float* sin, size_t rows,
                              size_t head_dim);
void orc_build_rope_table_f32(size_t seq, size_t head_dim, double theta, float* cos, float* sin);
void orc_mean_pool_masked(const float* h, const uint8_t* mask, size_t seq, size_t hidden,
                          float* out);
void orc_l2_normalize_in_place(float* v, size_t n);

/* ---- crates/transformers: attention, MLP, RoPE gather -------------------- */
typedef struct {
  size_t hidden, n_heads, n_kv_heads, head_dim;
  const float *wq, *bq, *wk, *bk, *wv, *bv, *wo;
} orc_attn_t;
/* causal = 0 is the reference behaviour; causal = 1 is this build's decoder variant */
int orc_rope_gather(const float* cos_tab, const float* sin_tab, size_t max_seq, size_t head_dim,
                    const size_t* positions, size_t n_pos, float* cos_rows, float* sin_rows);
int orc_attention_forward(const orc_attn_t* a, const float* x, const uint8_t* mask, size_t seq,
                          const float* cos_tab, const float* sin_tab, size_t rope_max_seq,
                          int causal, float* out);
int orc_sdpa(const float* q, const float* k, const float* v, const uint8_t* mask, size_t seq,
             size_t n_h, size_t n_kv, size_t d, int causal, float* merged_out);
void orc_transpose_seq_heads(const float* x, size_t seq, size_t heads, size_t d, float* out);
void orc_merge_heads(const float* x, size_t heads, size_t seq, size_t d, float* out);
void orc_repeat_kv(const float* kv, size_t n_kv, size_t groups, size_t seq, size_t d, float* out);
int orc_swiglu_forward(const float* w_gate, const float* w_up, const float* w_down, size_t hidden,
                       size_t inter, const float* x, size_t seq, float* out);

/* ---- crates/encoders/src/stella.rs + crates/embed/src/stella.rs ---------- */
typedef struct {
  const float *norm1, *norm2;
  const float *wq, *bq, *wk, *bk, *wv, *bv, *wo;
  const float *w_gate, *w_up, *w_down;
} orc_layer_weights_t;
typedef struct {
  size_t vocab, hidden, n_layers, n_heads, n_kv_heads, intermediate, max_pos, head_out_dim;
  float rms_eps;
  double rope_theta;
  const float* tok_embed;
  const float* final_norm;
  const orc_layer_weights_t* layers;
  const float* head_w; /* [head_out_dim, hidden] */
  const float* head_b; /* [head_out_dim] */
} orc_stella_t;
void* orc_stella_create(const orc_stella_t* desc); /* copies the descriptor, builds the RoPE table */
void orc_stella_destroy(void* model);
/* -1: ids/mask length mismatch (n/a here), -2: seq > max_pos */
int orc_stella_forward(void* model, const uint32_t* ids, const uint8_t* mask, size_t seq,
                       int causal, float* hidden_out);
int orc_stella_encode_raw(void* model, const uint32_t* ids, const uint8_t* mask, size_t seq,
                          float* emb_out);
/* one worker per sequence, at most n_threads running, single-threaded GEMM inside each */
int orc_stella_encode_batch(void* model, const uint32_t* ids, const int32_t* cu_seqlens,
                            size_t n_seq, size_t n_threads, float* emb_out);
size_t orc_physical_cores(void);
size_t orc_count_physical_cores_text(const char* cpuinfo_text);

/* ---- [NEW] hybrid decoder stack (no reference model; see hybrid.cpp) --------- */
typedef struct {
  int kind; /* 0 = gated full attention, 1 = gated delta rule linear attention */
  const float *norm1, *norm2;
  const float* w_mix_in;  /* kind 0: [2*nq*ad + 2*nkv*ad, hidden] rows q|gate|k|v; kind 1: [4*gh*128, hidden] rows q|k|v|z */
  const float* w_mix_out; /* [hidden, nq*ad] or [hidden, gh*128] */
  const float *w_ab, *A_log, *dt_bias; /* kind 1: [2*gh, hidden], [gh], [gh] */
  const float *w_gate, *w_up, *w_down;
} orc_hybrid_layer_t;
typedef struct {
  size_t vocab, hidden, n_layers, n_heads, n_kv_heads, attn_head_dim, gdn_heads, intermediate, max_pos;
  float rms_eps;
  double rope_theta;
  const float *tok_embed, *final_norm, *lm_head;
  const orc_hybrid_layer_t* layers;
} orc_hybrid_t;
void* orc_hybrid_create(const orc_hybrid_t* desc);
void orc_hybrid_destroy(void* model);
int orc_hybrid_forward(void* model, const uint32_t* ids, size_t seq, float* hidden_out, float* logits_last);

/* ---- crates/kernels/src/gated_delta_rule/cpu.rs -------------------------- */
void orc_l2_norm_rows(float* x, size_t len, size_t k);
void orc_cumsum(const float* g, size_t n, float* out);
void orc_gdn_recurrent_fwd(const float* q, const float* k, const float* v, const float* beta,
                           const float* g, size_t t, float scale, const float* state_in,
                           size_t k_dim, size_t v_dim, float* o, float* state_out);
void orc_gdn_chunk_fwd(const float* q, const float* k, const float* v, const float* beta,
                       const float* g, size_t t, float scale, const float* state_in, size_t k_dim,
                       size_t v_dim, size_t bt, float* o, float* chunk_states);
/* [NEW] gate preprocessing: g = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b) */
void orc_gdn_gates(const float* a, const float* b, const float* A_log, const float* dt_bias,
                   size_t t, size_t heads, float* g, float* beta);

/* ---- crates/quant/src/lib.rs (nibble order) + [NEW] int4 group-32 -------- */
int orc_pack_turbo4(const uint8_t idx[32], uint8_t out[16]);
void orc_unpack_turbo4(const uint8_t packed[16], uint8_t idx[32]);
int orc_pack_turbo3(const uint8_t idx[32], uint8_t out[12]);
void orc_unpack_turbo3(const uint8_t packed[12], uint8_t idx[32]);
/* TurboQuant 3-bit head codec (crates/quant/src/lib.rs:90-114, :316-413): 128 values <-> 4 x 14 bytes */
void orc_fwht_128(float* data128);
void orc_turbo3_encode_head(const float* values128, uint8_t* out56);
void orc_turbo3_decode_head(const uint8_t* in56, float* out128);
/* codes: int8 in [-8,7], [n,k] -> packed [n,k/2] two's-complement nibbles */
int orc_int4_pack(const int8_t* codes, size_t n, size_t k, uint8_t* packed);
void orc_int4_unpack(const uint8_t* packed, size_t n, size_t k, int8_t* codes);
/* absmax symmetric quantiser: scale = fp16(absmax/7), code = clamp(rne(w/scale),-8,7) */
void orc_int4_quantize(const float* w, size_t n, size_t k, uint8_t* packed, uint16_t* scales_f16);
void orc_int4_dequant(const uint8_t* packed, const uint16_t* scales_f16, size_t n, size_t k,
                      float* w);
/* y[b,n] = sum_g s[n,g] * sum_{k in g} code[n,k] * x[b,k]  (== linear_t on the dequantised W) */
void orc_int4_gemv(const uint8_t* packed, const uint16_t* scales_f16, size_t n, size_t k,
                   const float* x, size_t batch, float* y);

/* ---- crates/cache/src/flat.rs + [NEW] paged cache ------------------------ */
void* orc_flatkv_create(size_t num_layers, size_t row_bytes, size_t max_seq_len);
void orc_flatkv_destroy(void* c);
/* 0 ok, 1 LayerOutOfRange, 2 LenOverflow, 3 ReadBeyondWritten, 4 ShapeMismatch */
int orc_flatkv_put(void* c, size_t layer, const uint8_t* k, const uint8_t* v, size_t n_tokens);
int orc_flatkv_get(void* c, size_t layer, size_t len, uint8_t* k_out, uint8_t* v_out);
long orc_flatkv_len_of(void* c, size_t layer);
void orc_flatkv_reset(void* c);
/* paged: pool [n_blocks, block_size, row_bytes] per K and V; logical token t of a sequence lives
   in physical block table[t / block_size], slot t % block_size */
int orc_paged_append(uint8_t* k_pool, uint8_t* v_pool, size_t n_blocks, size_t block_size,
                     size_t row_bytes, const int32_t* table, size_t table_len, size_t pos,
                     const uint8_t* k_row, const uint8_t* v_row);
int orc_paged_gather(const uint8_t* k_pool, const uint8_t* v_pool, size_t n_blocks,
                     size_t block_size, size_t row_bytes, const int32_t* table, size_t table_len,
                     size_t len, uint8_t* k_out, uint8_t* v_out);
/* decode attention for ONE sequence, fp32 rows: q [n_heads, d]; k,v [len, n_kv*d] -> out [n_heads*d] */
void orc_decode_attention(const float* q, const float* k, const float* v, size_t len,
                          size_t n_heads, size_t n_kv, size_t d, float* out);

/* ---- [NEW] ragged packing (crates/sched is an empty scaffold) ------------ */
/* seq i contributes new_lens[i] tokens whose positions continue from cached_lens[i].
   Outputs: cu_seqlens [n+1], positions [total], slot_mapping [total] (physical slot =
   block*block_size + offset through tables[i*max_blocks + ..]), seq_ids [total].
   returns total tokens, or -1 when a table entry is missing (<0) or out of range. */
long orc_build_packing(const int32_t* cached_lens, const int32_t* new_lens, size_t n_seq,
                       const int32_t* tables, size_t max_blocks, size_t block_size,
                       size_t n_pool_blocks, int32_t* cu_seqlens, int32_t* positions,
                       int64_t* slot_mapping, int32_t* seq_ids);

/* ---- crates/decode/src/lib.rs -------------------------------------------- */
uint32_t orc_greedy(const float* logits, size_t n);

/* ---- crates/kernels/src/{matmul,rms_norm,softmax,rope}/cpu.rs (fp16) ----- */
void orc_matmul_fp16_ref(const uint16_t* a, const uint16_t* b, size_t m, size_t n, size_t k,
                         uint16_t* d);
void orc_rms_norm_fp16_ref(const uint16_t* x, const uint16_t* w, size_t m, size_t n, float eps,
                           uint16_t* y);
int orc_softmax_fp16_ref(const uint16_t* x, size_t x_len, size_t m, size_t n, uint16_t* y);
void orc_build_cos_sin_table(size_t seq, size_t head_dim, float theta, float* table);
int orc_rope_apply_fp16_ref(uint16_t* qk, size_t qk_len, const float* cos_sin, size_t cs_len,
                            size_t batch, size_t seq, size_t heads, size_t head_dim);

/* helpers */
void orc_f32_to_bf16(const float* x, size_t n, uint16_t* y);
void orc_bf16_to_f32(const uint16_t* x, size_t n, float* y);
void orc_f32_to_f16(const float* x, size_t n, uint16_t* y);
void orc_f16_to_f32(const uint16_t* x, size_t n, float* y);

/* ---- crates/decode: logit processors and samplers (processors.rs:15-199, sampler.rs:31-58),
 * one row of logits in place; orc_multinomial takes the uniform draw the reference takes from its RNG */
void orc_temperature(float* logits, size_t n, float temperature);
void orc_top_k(float* logits, size_t n, size_t k);
void orc_top_p(float* logits, size_t n, float p);
void orc_min_p(float* logits, size_t n, float p);
void orc_repetition_penalty(float* logits, size_t n, const uint32_t* tokens, size_t n_tokens, float penalty);
uint32_t orc_multinomial(const float* logits, size_t n, float u);

#ifdef __cplusplus
}
#endif
