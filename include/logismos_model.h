/*
 * logismos_model.h - C ABI of the host-side executors above the kernel launchers.
 *
 * lg_stella_* is the GPU form of the reference's Stella embedding model:
 *   StellaEncoder::forward        crates/encoders/src/stella.rs:278-313 (layer body :190-206)
 *   StellaModel::encode_raw       crates/embed/src/stella.rs:221-248
 *   StellaModel::encode_batch     crates/embed/src/stella.rs:264-294
 * behind the consumer contract core::EmbeddingModel (crates/core/src/lib.rs:139-163). Text
 * handling (prompt, tokenizer) stays on the caller's side of this boundary: the entry points
 * take token ids, which is what `encode_raw(ids, mask, dim)` takes in the reference. There is no
 * padding in this path (the reference builds an all-ones mask, crates/embed/src/stella.rs:318),
 * so a batch is a ragged concatenation of id runs delimited by cu_seqlens.
 *
 * Results are EmbeddingError-shaped status codes; 0 is success.
 */
#ifndef LOGISMOS_MODEL_H
#define LOGISMOS_MODEL_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* EmbeddingError (crates/core/src/lib.rs:75-133) as status codes */
enum lg_embedding_status {
  LG_EMB_OK = 0,
  LG_EMB_INPUT_TOO_LONG = 1,   /* InputTooLong { got, limit }: never truncates (:63-66) */
  LG_EMB_UNSUPPORTED_DIM = 2,  /* UnsupportedDim { dim } */
  LG_EMB_TOKENIZE = 3,         /* unused at id level */
  LG_EMB_COMPUTE = 4,          /* Compute { message }: shape errors, CUDA failures */
  LG_EMB_IO = 5,
  LG_EMB_UNSUPPORTED_PROMPT = 6
};

/* StellaConfig (crates/encoders/src/stella.rs:45-80). head_dim = hidden / n_heads must be 128. */
typedef struct lg_stella_config {
  int32_t vocab, hidden, n_layers, n_heads, n_kv_heads, intermediate, max_pos;
  float rms_eps;
  double rope_theta;
  int32_t max_tokens;        /* default per-input limit (EncodeOpts::max_tokens None -> 512) */
  int32_t n_dims;            /* number of dense heads loaded (supported_dims) */
  int32_t dims[8];           /* output dims, dims[0] is default_dim */
  int32_t max_batch_tokens;  /* workspace capacity in tokens; larger batches are run in pieces */
  int32_t max_batch_seqs;
  int32_t fuse_swiglu;       /* 1: SwiGLU fused into the gate/up GEMM epilogue */
} lg_stella_config_t;

/* The 12 tensors of one layer (crates/encoders/src/stella.rs:326-349), HOST fp32, HF [out, in]. */
typedef struct lg_stella_layer_weights {
  const float *norm1, *norm2;
  const float *wq, *bq, *wk, *bk, *wv, *bv, *wo;
  const float *w_gate, *w_up, *w_down;
} lg_stella_layer_weights_t;

typedef struct lg_stella_weights {
  const float* tok_embed;   /* [vocab, hidden] */
  const float* final_norm;  /* [hidden] */
  const lg_stella_layer_weights_t* layers;
  const float* head_w[8];   /* [dims[i], hidden]  (2_Dense_{dim}/linear.weight) */
  const float* head_b[8];   /* [dims[i]] */
} lg_stella_weights_t;

/* StellaModel::load counterpart for in-memory weights: casts to bf16, uploads, sizes the
 * workspace. All device allocation happens here. Returns LG_EMB_COMPUTE on failure with the
 * reason available from lg_last_error(). */
uint32_t lg_stella_create(int32_t device, const lg_stella_config_t* cfg, const lg_stella_weights_t* w,
                          void** model);
void lg_stella_destroy(void* model);

/* StellaModel::load (crates/embed/src/stella.rs:138-201) from a checkpoint directory: `root`/
 * model.safetensors must hold exactly 2 + 12 n_layers fp32 tensors under the names and shapes of
 * crates/encoders/src/stella.rs:126-127, :326-349 (anything else is LG_EMB_COMPUTE with the reason in
 * lg_last_error(); a missing or malformed file is LG_EMB_IO), and `root`/2_Dense_<dim>/model.safetensors
 * one dense head (linear.weight [dim, hidden], linear.bias [dim]) for every cfg->dims entry. The
 * supported dims are sorted and the default is 1024 when that head is loaded, else the smallest. The
 * files are mapped, not copied; the mapping is released before returning. */
uint32_t lg_stella_load(int32_t device, const char* root, const lg_stella_config_t* cfg, void** model);

/* EmbeddingModel::{default_dim, supported_dims, max_tokens} */
int32_t lg_stella_default_dim(const void* model);
int32_t lg_stella_supported_dims(const void* model, int32_t* out, int32_t cap);
int32_t lg_stella_max_tokens(const void* model);

/* EmbeddingModel::encode_batch at id level. host_ids u32 [cu_seqlens[n_seqs]], host_cu_seqlens
 * i32 [n_seqs + 1], host_out f32 [n_seqs, dim], unit-norm rows. dim == 0 selects default_dim;
 * max_tokens == 0 selects the model default. Copies ids to the device, runs the forward, copies
 * the embeddings back and synchronises. Thread-safe (calls are serialised per model). */
uint32_t lg_stella_encode_ids_batch(void* model, const uint32_t* host_ids, const int32_t* host_cu_seqlens,
                                    int32_t n_seqs, int32_t dim, int32_t max_tokens, float* host_out);

/* The same forward with everything already resident: dev_ids u32 [n_tokens], dev_cu_seqlens i32
 * [n_seqs+1], dev_positions i32 [n_tokens] (position of each token inside its sequence),
 * dev_out f32 [n_seqs, dim]. Enqueues on `stream` and returns without synchronising.
 * n_tokens <= max_batch_tokens and n_seqs <= max_batch_seqs (LG_EMB_COMPUTE otherwise); max_seqlen
 * must be >= the longest sequence of the batch (it sizes the attention grid: queries beyond it are
 * not computed) and <= max_pos. causal != 0 runs the decoder-style (causal) variant. */
uint32_t lg_stella_forward_device(void* model, const void* dev_ids, const void* dev_cu_seqlens,
                                  const void* dev_positions, int32_t n_tokens, int32_t n_seqs,
                                  int32_t max_seqlen, int32_t dim, int32_t causal, void* dev_out, void* stream);

/* StellaEncoder::forward output of the last forward: f32 [n_tokens, hidden] copied to host. */
uint32_t lg_stella_last_hidden(void* model, int32_t n_tokens, float* host_out);
/* Number of kernel launches one forward of n_layers issues (for launch accounting). */
int32_t lg_stella_launches_per_forward(const void* model);
/* Status word written by kernels with bounded waits / range checks during the last forward. */
int32_t lg_stella_device_status(void* model);

/* ====================================================================================
 * Continuous-batching decoder step over a Qwen2-style layer stack with int4 group-32 weights and
 * a paged KV cache. The reference has no decoder executor (crates/decoders is an empty scaffold,
 * src/lib.rs:1-15) and no scheduler (crates/sched/src/lib.rs:1-30); the contract kept is the
 * reference's only execution semantics, one sequence per call
 * (crates/transformers/src/attention.rs:13-14): a packed step must equal running every sequence
 * alone through the causal variant of StellaEncoder::forward, followed by lm_head + decode::greedy
 * (crates/decode/src/lib.rs:73-83) on its last token.
 * ==================================================================================== */
typedef struct lg_decoder_config {
  int32_t vocab, hidden, n_layers, n_heads, n_kv_heads, intermediate, max_pos;
  float rms_eps;
  double rope_theta;
  int32_t n_pool_blocks;       /* KV blocks of 16 tokens per layer */
  int32_t max_blocks_per_seq;  /* width of a block-table row */
  int32_t max_step_tokens;     /* capacity of one packed step */
  int32_t max_step_seqs;
  int32_t keep_bf16_copy;      /* != 0: also keep a bf16 expansion of every layer matrix (2 B per weight) for
                                  steps of more than 128 rows, instead of expanding per layer per step */
  int32_t kv_turbo3;           /* != 0: the paged cache holds TurboQuant 3-bit rows (56 bytes per 128-value head
                                  chunk instead of 256: crates/quant/src/lib.rs:316-413); every sequence of a step,
                                  decode tokens included, then attends through the decoding gather of
                                  logismos_launch_paged_prefix_attention_turbo3_bf16. A capacity mode: 4.57 times
                                  more context per byte of pool, at the codec's accuracy */
} lg_decoder_config_t;

/* int4 group-32 matrix on the HOST: codes u8 [n, k/2], scales fp16 bits [n, k/32]
 * (storage contract of logismos_launch_gemv_int4_g32_bf16). */
typedef struct lg_int4_matrix { const uint8_t* codes; const uint16_t* scales; } lg_int4_matrix_t;
typedef struct lg_decoder_layer_weights {
  const float *norm1, *norm2, *bq, *bk, *bv;            /* fp32 */
  lg_int4_matrix_t wq, wk, wv, wo, w_gate, w_up, w_down;  /* HF [out, in] */
} lg_decoder_layer_weights_t;
typedef struct lg_decoder_weights {
  const float* tok_embed;  /* fp32 [vocab, hidden], stored bf16 on the device */
  const float* final_norm;
  const lg_decoder_layer_weights_t* layers;
  lg_int4_matrix_t lm_head;  /* [vocab, hidden] */
} lg_decoder_weights_t;

uint32_t lg_decoder_create(int32_t device, const lg_decoder_config_t* cfg, const lg_decoder_weights_t* w, void** model);
/* The decoder from a Qwen2-style fp32 safetensors file (the tensor names of crates/encoders/src/
 * stella.rs:326-349, plus lm_head.weight [vocab, hidden]; without it the head is tied to the
 * embedding): exact tensor accounting as lg_stella_load, every matrix quantised to int4 group-32 on
 * the device (logismos_launch_quantize_int4_g32). */
uint32_t lg_decoder_load(int32_t device, const char* path, const lg_decoder_config_t* cfg, void** model);
void lg_decoder_destroy(void* model);

/* One packed step. Sequence i brings new_lens[i] new tokens (ids packed in sequence order in
 * host_ids) on top of cached_lens[i] tokens already in the paged cache; its block-table row
 * host_block_tables[i, :] must cover cached + new tokens. new_lens[i] == 1 is a decode token,
 * > 1 a prefill chunk, which may start its sequence (cached_lens[i] == 0) or continue it: positions
 * and cache slots carry on from the cached length and the chunk attends to the cached prefix through
 * the block table, so a prompt fed in chunks gives the result of the whole prompt fed at once. All
 * K/V rows of the new tokens are written to the cache; host_next_tokens[i] receives the greedy token after the last
 * new token of sequence i. Synchronises before returning. Status codes as lg_embedding_status. */
uint32_t lg_decoder_step(void* model, const uint32_t* host_ids, const int32_t* host_cached_lens,
                         const int32_t* host_new_lens, int32_t n_seqs, const int32_t* host_block_tables,
                         uint32_t* host_next_tokens);
/* Re-runs the device work of the last lg_decoder_step (same indices, same ids; the cache rows are
 * rewritten with the same values) on `stream` without host transfers or synchronisation: for
 * kernel-only timing. */
uint32_t lg_decoder_replay_device(void* model, void* stream);
/* fp32 [n_seqs, hidden]: final-norm output of each sequence's last new token in the last step. */
uint32_t lg_decoder_last_hidden(void* model, int32_t n_seqs, float* host_out);
/* fp32 logits of the last step [n_seqs, vocab] (the values decode::greedy ran on). */
uint32_t lg_decoder_last_logits(void* model, int32_t n_seqs, float* host_out);
int32_t lg_decoder_launches_last_step(const void* model);
int32_t lg_decoder_device_status(void* model);

/* ====================================================================================
 * Hybrid decoder step: a stack that mixes gated-delta-rule linear-attention layers (fp32 recurrent
 * state per sequence, crates/kernels/src/gated_delta_rule/cpu.rs:92-182) with gated full-attention
 * layers (paged KV cache, head_dim 128 or 256), SwiGLU MLPs, int4 group-32 weights. No reference
 * counterpart (crates/decoders/src/lib.rs:1-15 is an empty scaffold); the layer formulas are those
 * of research/14-gdn-aiter-preflight.md:190-198, :209-219 and the contract is the same as
 * lg_decoder_step: a packed step equals running every sequence alone.
 *   block:  x += mixer(rms_norm(x, norm1));  x += swiglu(rms_norm(x, norm2))
 *   full attention (layer l with (l + 1) % full_attn_interval == 0), no biases:
 *     q, gate [n_heads * d], k, v [n_kv_heads * d] = h W^T; RoPE(halves) on q, k; causal attention;
 *     out *= sigmoid(gate); o_proj
 *   linear attention (all other layers), gdn_heads heads of key = value dim 128:
 *     q, k, v, z [gdn_heads * 128] = h W^T; a, b [gdn_heads] = h W^T (fp32 outputs);
 *     q, k L2-normalised per head; g = -exp(A_log) softplus(a + dt_bias); beta = sigmoid(b);
 *     o = gated delta rule (scale 1/sqrt(128)); o *= silu(z); out_proj
 * ==================================================================================== */
typedef struct lg_hybrid_config {
  int32_t vocab, hidden, n_layers, n_heads, n_kv_heads, attn_head_dim, gdn_heads, intermediate, max_pos;
  int32_t full_attn_interval;  /* 4 = three linear-attention layers, then one full-attention layer */
  float rms_eps;
  double rope_theta;
  int32_t n_pool_blocks;       /* KV blocks of 16 tokens per full-attention layer */
  int32_t max_blocks_per_seq;
  int32_t max_step_tokens;
  int32_t max_step_seqs;
  int32_t n_state_slots;       /* recurrent-state slots per linear-attention layer */
  int32_t keep_bf16_copy;      /* as in lg_decoder_config_t */
} lg_hybrid_config_t;

typedef struct lg_hybrid_layer_weights {
  const float *norm1, *norm2;
  /* full attention: wq, wgate [n_heads*d, hidden], wk, wv [n_kv_heads*d, hidden], wo [hidden, n_heads*d]
   * linear attention: wq, wk, wv, wgate(= z) [gdn_heads*128, hidden], wo [hidden, gdn_heads*128],
   *                   wa, wb [gdn_heads, hidden], A_log, dt_bias fp32 [gdn_heads] */
  lg_int4_matrix_t wq, wk, wv, wgate, wo, wa, wb;
  const float *A_log, *dt_bias;
  lg_int4_matrix_t w_gate, w_up, w_down;
} lg_hybrid_layer_weights_t;
typedef struct lg_hybrid_weights {
  const float* tok_embed;
  const float* final_norm;
  const lg_hybrid_layer_weights_t* layers;
  lg_int4_matrix_t lm_head;
} lg_hybrid_weights_t;

uint32_t lg_hybrid_create(int32_t device, const lg_hybrid_config_t* cfg, const lg_hybrid_weights_t* w, void** model);
void lg_hybrid_destroy(void* model);
/* As lg_decoder_step, plus host_state_slots i32 [n_seqs]: the recurrent-state slot of each
 * sequence (distinct within a step, < n_state_slots). A sequence with cached_lens[i] == 0 starts
 * from the zero state; otherwise its slot must hold the state its previous step left (decode tokens
 * and continuing prefill chunks alike). */
uint32_t lg_hybrid_step(void* model, const uint32_t* host_ids, const int32_t* host_cached_lens,
                        const int32_t* host_new_lens, int32_t n_seqs, const int32_t* host_block_tables,
                        const int32_t* host_state_slots, uint32_t* host_next_tokens);
/* Tensor-parallel form. A model created from a 1/tp slice of the heads and of the MLP (n_heads,
 * n_kv_heads, gdn_heads, intermediate divided by tp; input projections sliced by rows, output
 * projections by columns; embeddings, norms and lm_head replicated) produces partial sums in its
 * output projections. With a reduction installed, each partial sum [tokens, hidden] is computed into
 * a zeroed fp32 buffer, handed to `fn`, which must leave the sum over all ranks in place, ordered on
 * `stream` (an NCCL all-reduce enqueued on it; it need not synchronise), and is then added to the
 * residual stream. fn returns 0 on success. fn == NULL removes the reduction. No reference
 * counterpart (the reference has no tensor parallelism). */
typedef uint32_t (*lg_allreduce_f32_fn)(void* user, void* dev_buf_f32, uint64_t count, void* stream);
uint32_t lg_hybrid_set_allreduce(void* model, lg_allreduce_f32_fn fn, void* user);
/* The same slot for a reduction fused with the residual add: each partial sum is computed into a zeroed
 * fp32 buffer `delta` and fn(user, x, delta, count, status, stream) must leave x += sum over all ranks
 * of delta, ordered on `stream`, without synchronising; status_i32 is the model's device status word
 * (a bounded wait that expires raises it). lg_tp_reduce_add_f32 below has this signature. Installing
 * one kind of reduction removes the other. */
typedef uint32_t (*lg_reduce_add_f32_fn)(void* user, void* x_f32, void* delta_f32, uint64_t count, void* status_i32, void* stream);
uint32_t lg_hybrid_set_reduce_add(void* model, lg_reduce_add_f32_fn fn, void* user);
uint32_t lg_hybrid_replay_device(void* model, void* stream);
uint32_t lg_hybrid_last_hidden(void* model, int32_t n_seqs, float* host_out);
uint32_t lg_hybrid_last_logits(void* model, int32_t n_seqs, float* host_out);
int32_t lg_hybrid_launches_last_step(const void* model);
int32_t lg_hybrid_device_status(void* model);

/* ====================================================================================
 * Tensor-parallel exchange over NVLink peer memory (ranks = processes on different GPUs of one node).
 * No reference counterpart (the reference is single-device, README.md:19-21). One kernel per rank
 * writes the local partial sum into every peer's receive buffer with plain peer stores, raises a
 * flag there, waits (bounded: status 3 on expiry, the add is then skipped) for the peers' flags and adds all partial
 * sums, in rank order, into the residual stream.
 *   lg_tp_comm_alloc   allocates this rank's region (flags + two receive sets of tp * max_elems floats,
 *                      zeroed) on `device` and returns its 64-byte cudaIpc handle
 *   lg_tp_comm_open    given the handles of all ranks [tp][64] (exchanged by the host, e.g. an
 *                      all-gather over the process group), maps the peers' regions
 *   lg_tp_reduce_add_f32  x += sum over ranks of delta for count floats (count % 4 == 0, count <=
 *                      max_elems); every rank makes the same sequence of calls; signature of
 *                      lg_reduce_add_f32_fn with user = the communicator
 * ==================================================================================== */
size_t lg_tp_comm_region_bytes(int32_t tp, uint64_t max_elems);
uint32_t lg_tp_comm_alloc(int32_t device, int32_t tp, uint64_t max_elems, void** region, uint8_t* handle_out64);
uint32_t lg_tp_comm_open(int32_t device, void* region, int32_t rank, int32_t tp, uint64_t max_elems,
                         const uint8_t* all_handles, void** comm);
void lg_tp_comm_destroy(void* comm, int32_t free_region);
uint32_t lg_tp_reduce_add_f32(void* comm, void* x_f32, void* delta_f32, uint64_t count, void* status_i32, void* stream);

/* ====================================================================================
 * safetensors reader: crates/loader/src/safetensors.rs:44-197 (Reader::open / get / names / len) with
 * the dtype map of :199-217 and the truncation guard of crates/loader/src/lib.rs:229-246 (every get
 * re-stats the file and fails if its length changed since it was mapped). Status codes as
 * lg_embedding_status: LG_EMB_IO for I/O and format errors, with the reason in lg_last_error().
 * ==================================================================================== */
enum lg_dtype { LG_DT_F32 = 0, LG_DT_F16 = 1, LG_DT_BF16 = 2, LG_DT_F8E4M3 = 3, LG_DT_F8E5M2 = 4, LG_DT_I32 = 5, LG_DT_I8 = 6,
                LG_DT_I4 = 7, LG_DT_U8 = 8 };  /* order of taxis::DType, crates/taxis/src/dtype.rs:16-26 */
typedef struct lg_tensor_view {
  int32_t dtype;       /* lg_dtype */
  int32_t rank;
  int64_t shape[8];
  const void* data;    /* into the mapping; valid until lg_safetensors_close */
  uint64_t nbytes;
} lg_tensor_view_t;
uint32_t lg_safetensors_open(const char* path, void** reader);
void lg_safetensors_close(void* reader);
int32_t lg_safetensors_len(const void* reader);
/* name of tensor i in archive order (by on-disk offset); NULL when i is out of range */
const char* lg_safetensors_name(const void* reader, int32_t i);
uint64_t lg_safetensors_data_region_start(const void* reader);
uint32_t lg_safetensors_get(const void* reader, const char* name, lg_tensor_view_t* out);

/* Message of the last failure on the calling thread ("" if none). */
const char* lg_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
