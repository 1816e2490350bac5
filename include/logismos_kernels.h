/*
 * logismos_kernels.h - C ABI of the sm_100a kernel launchers.
 *
 * Convention of the reference's launchers (crates/kernels/src/<op>/mod.rs `unsafe extern "C"`
 * blocks; e.g. matmul/mod.rs:36-56 and matmul/hip/matmul_launchers.cpp:14-52), kept for every
 * entry point here:
 *   - the caller owns every buffer; all pointers are DEVICE pointers unless a parameter is
 *     named host_*; a launcher never allocates and never synchronises;
 *   - dims are int32; `stream` is a cudaStream_t passed as void* (NULL = the null stream);
 *   - the return value is the raw runtime status read right after the launch (0 = success); a
 *     shape the kernel cannot address is rejected before launching with cudaErrorInvalidValue
 *     (1), the counterpart of the Rust-side guards check_matmul_shape / check_rope_shape
 *     (matmul/mod.rs:89-117, rope/mod.rs:79-132).
 * The library is built as liblogismos_kernels.so (and .a, the archive name the reference's
 * build script links, crates/kernels/build.rs:117-122).
 */
#ifndef LOGISMOS_KERNELS_H
#define LOGISMOS_KERNELS_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Process-wide switch for bit-reproducible results. By default two GEMM paths split the reduction over
 * k across CTAs when few output tiles would leave SMs idle (the accumulating epilogue of
 * logismos_launch_linear_t_bf16 and the spans of logismos_launch_qlinear_int4_g32_acc_f32); the
 * slices meet in fp32 reductions whose order is not fixed, so the last bits of a result can differ
 * between runs and between a row computed alone and inside a batch (within the 2e-2 parity bar, but
 * not bit-identical). With the switch on, those splits are not used: every output element is summed in
 * one fixed order, at some cost in speed for small steps. The environment variable
 * LOGISMOS_DETERMINISTIC=1 sets the initial value. No reference counterpart (its CPU path is
 * deterministic by construction). */
void logismos_set_deterministic(int32_t on);
int32_t logismos_get_deterministic(void);

/* Process-wide switch, on by default (LOGISMOS_DEPENDENT_LAUNCH=0 sets the initial value to off): the
 * kernels of the model steps are launched with programmatic stream serialisation, i.e. the next kernel
 * of the same stream is scheduled while the current one drains and waits on the device for its
 * completion before touching memory. Results do not change; the gaps between dependent launches
 * shrink. Off, every launch is an ordinary stream-ordered launch. No reference counterpart. */
void logismos_set_dependent_launch(int32_t on);
int32_t logismos_get_dependent_launch(void);

/* ====================================================================================
 * The reference's four fp16 launchers, same symbols and argument lists.
 * ==================================================================================== */

/* crates/kernels/src/matmul/mod.rs:37-45 -> matmul_naive.hip. D[M,N] = A[M,K] B[K,N], row-major
 * fp16, fp32 accumulate. */
uint32_t logismos_launch_matmul_naive_fp16(const void* a_fp16, const void* b_fp16, void* d_fp16,
                                           int32_t m, int32_t n, int32_t k, void* stream);
/* crates/kernels/src/matmul/mod.rs:47-55 -> matmul_wmma.hip. Same contract on tensor cores; M, N,
 * K must be multiples of 16 (the only case crates/praxis/src/matmul.rs:113-117 selects it). */
uint32_t logismos_launch_matmul_wmma_fp16(const void* a_fp16, const void* b_fp16, void* d_fp16,
                                          int32_t m, int32_t n, int32_t k, void* stream);
/* crates/kernels/src/rms_norm/mod.rs:33-43 -> rms_norm.hip */
uint32_t logismos_launch_rms_norm_fp16(const void* x_fp16, const void* w_fp16, void* y_fp16,
                                       int32_t m, int32_t n, float eps, void* stream);
/* crates/kernels/src/softmax/mod.rs:28-36 -> softmax.hip. An all -inf row yields 1/n. */
uint32_t logismos_launch_softmax_fp16(const void* x_fp16, void* y_fp16, int32_t m, int32_t n,
                                      void* stream);
/* crates/kernels/src/rope/mod.rs:44-54 -> rope.hip. In-place interleaved-pair rotation of
 * (batch, seq, heads, head_dim) fp16 with an fp32 (seq, head_dim) table of (cos, sin) pairs. */
uint32_t logismos_launch_rope_fp16(void* qk_fp16, const void* cos_sin_f32, int32_t batch,
                                   int32_t seq, int32_t heads, int32_t head_dim, void* stream);

/* ====================================================================================
 * Encoder / prefill path (bf16 storage, fp32 accumulation). Each entry replaces the CPU
 * function of crates/kernels/src/cpu_f32/mod.rs named beside it.
 * ==================================================================================== */

/* cpu_f32::embed_lookup (mod.rs:106-127): out[i,:] = table[ids[i],:]; an id >= vocab yields a
 * zero row. table bf16 [vocab, hidden]; out f32 [n_ids, hidden] (the fp32 residual stream). */
uint32_t logismos_launch_embed_lookup_bf16(const void* table_bf16, const void* ids_u32,
                                           void* out_f32, int32_t n_ids, int32_t hidden,
                                           int32_t vocab, void* stream);

/* cpu_f32::rms_norm (mod.rs:137-159) over the fp32 residual stream: y = x * rsqrt(mean(x^2)+eps)
 * * w. x f32 [rows, n], w f32 [n]; y bf16 [rows, n] (out_f32 == 0) or f32 (out_f32 != 0). */
uint32_t logismos_launch_rms_norm_f32(const void* x_f32, const void* w_f32, void* y, int32_t rows,
                                      int32_t n, float eps, int32_t out_f32, void* stream);

/* cpu_f32::linear_t (mod.rs:271-345) on the tcgen05 tensor cores:  C = A W^T (+ bias).
 * A bf16 [m, k] row-major (row stride lda elements), W bf16 [n, k] row-major (the HF [out, in]
 * layout, untransposed). k % 64 == 0, n % 16 == 0, lda % 8 == 0, pointers 16-byte aligned.
 * epilogue selects what is stored:
 *   LG_EPI_BF16      out bf16 [m, n]      = acc + bias
 *   LG_EPI_RESID_F32 out f32  [m, n]     += acc + bias       (residual add, in place)
 *   LG_EPI_SWIGLU    out bf16 [m, n / 2]  = silu(gate) * up, W holding gate and up rows
 *                    interleaved in blocks of 32 rows (32 gate rows, then the 32 matching up
 *                    rows); n % 64 == 0; fuses cpu_f32::silu + hadamard (mod.rs:349-374)
 * bias_f32 may be NULL. ldc is the row stride of out in elements. status_i32 (may be NULL)
 * receives a value whose low byte is 2 if a bounded wait inside the kernel expired (the output is
 * then invalid); the next byte names the kernel family (1 dense GEMM, 2 fused-dequant linear, 3
 * tensor-core attention).
 * With few output tiles and a long reduction the accumulating epilogue splits k over CTAs; the
 * slices meet in the fp32 reduce-add, so the last bits of the sum can differ between runs.
 *
 * LG_EPI_STATIC_W, or-ed into `epilogue`, is the caller's promise that no work still in flight on the
 * stream writes `w_bf16` (model weights uploaded once). With dependent launch on, the kernel then
 * requests its first weight stages before the preceding kernel has finished. Without the flag the
 * weights are read only after everything before the launch has completed. */
enum { LG_EPI_BF16 = 0, LG_EPI_RESID_F32 = 1, LG_EPI_SWIGLU = 2, LG_EPI_STATIC_W = 0x100 };
uint32_t logismos_launch_linear_t_bf16(const void* a_bf16, const void* w_bf16,
                                       const void* bias_f32, void* out, int32_t m, int32_t n,
                                       int32_t k, int32_t lda, int32_t ldc, int32_t epilogue,
                                       void* status_i32, void* stream);
/* The same contract one thread per output, as the on-device correctness anchor (the role
 * matmul_naive.hip plays in the reference). LG_EPI_SWIGLU is not supported here. */
uint32_t logismos_launch_linear_t_naive_bf16(const void* a_bf16, const void* w_bf16,
                                             const void* bias_f32, void* out, int32_t m, int32_t n,
                                             int32_t k, int32_t lda, int32_t ldc, int32_t epilogue,
                                             void* stream);

/* cpu_f32::rope_halves_in_place (mod.rs:502-547) with RopeTable::gather (crates/transformers/
 * src/rope.rs:50-92) folded in: rotates, in place, the first n_rot_heads heads of every token row
 * of a packed bf16 [n_tokens, row_stride] buffer (q heads followed by k heads), head h at
 * column h * head_dim, using cos/sin f32 [max_pos, head_dim/2] rows selected by positions[token].
 * A position >= max_pos leaves the row untouched and sets *status (may be NULL) to 1. */
uint32_t logismos_launch_rope_halves_bf16(void* qk_bf16, const void* cos_f32, const void* sin_f32,
                                          const void* positions_i32, int32_t n_tokens,
                                          int32_t n_rot_heads, int32_t head_dim,
                                          int32_t row_stride, int32_t max_pos, void* status_i32,
                                          void* stream);

/* cpu_f32::silu + hadamard (mod.rs:349-374): out[t, j] = silu(gu[t, j]) * gu[t, inter + j].
 * gu bf16 [rows, 2*inter] (gate columns then up columns), out bf16 [rows, inter]. */
uint32_t logismos_launch_swiglu_bf16(const void* gu_bf16, void* out_bf16, int32_t rows,
                                     int32_t inter, void* stream);

/* QwenAttention::forward's score/softmax/PV stage (crates/transformers/src/attention.rs
 * :226-296) for a ragged batch, without materialising scores. qkv bf16 [n_tokens, row_stride]
 * with q heads at column 0, k heads at k_off, v heads at v_off (RoPE already applied); sequence
 * i owns token rows cu_seqlens[i] .. cu_seqlens[i+1]; q head j reads kv head j / (n_heads /
 * n_kv_heads) (attention.rs:366-382). causal = 0 is the reference's bidirectional encoder
 * attention, causal = 1 masks keys after the query. head_dim must be 128. out bf16
 * [n_tokens, n_heads * head_dim]. max_seqlen bounds the grid. */
uint32_t logismos_launch_varlen_attention_bf16(const void* qkv_bf16, const void* cu_seqlens_i32,
                                               void* out_bf16, int32_t n_seqs, int32_t max_seqlen,
                                               int32_t n_heads, int32_t n_kv_heads,
                                               int32_t head_dim, int32_t row_stride, int32_t k_off,
                                               int32_t v_off, int32_t causal, void* stream);

/* The same stage (attention.rs:226-296, head_dim 128 or 256) on the tcgen05 tensor cores: S = Q K^T and
 * O += P V as tcgen05.mma with the accumulators and P in tensor memory, operands moved by TMA. Same
 * layout contract as logismos_launch_varlen_attention_bf16; n_tokens = cu_seqlens[n_seqs]. scratch:
 * logismos_varlen_attention_tc_scratch_bytes(n_tokens, n_seqs, n_kv_heads, head_dim) bytes, 256-byte aligned
 * (receives V transposed per kv head with every sequence padded to a multiple of 8 keys). qkv and out
 * 16-byte aligned. Two launches. status (int32, may be NULL) is set to 2 (low byte; see logismos_launch_linear_t_bf16) if a bounded wait inside
 * the kernel expired. */
size_t logismos_varlen_attention_tc_scratch_bytes(int32_t n_tokens, int32_t n_seqs, int32_t n_kv_heads,
                                                  int32_t head_dim);
uint32_t logismos_launch_varlen_attention_tc_bf16(const void* qkv_bf16, const void* cu_seqlens_i32,
                                                  void* out_bf16, void* scratch, int32_t n_tokens,
                                                  int32_t n_seqs, int32_t max_seqlen, int32_t n_heads,
                                                  int32_t n_kv_heads, int32_t head_dim, int32_t row_stride,
                                                  int32_t k_off, int32_t v_off, int32_t causal,
                                                  void* status, void* stream);

/* The same with the halves-RoPE of the q and k heads (logismos_launch_rope_halves_bf16's contract:
 * the first n_rot_heads heads of every row are rotated in place by cos/sin f32 [max_pos, head_dim/2]
 * at positions[token]; a position outside [0, max_pos) sets status to 1) done by extra blocks of the
 * V-transposing launch, so the pair is still two launches. qkv is modified in place. */
uint32_t logismos_launch_rope_varlen_attention_tc_bf16(void* qkv_bf16, const void* cos_f32,
                                                       const void* sin_f32, const void* positions_i32,
                                                       int32_t n_rot_heads, int32_t max_pos,
                                                       const void* cu_seqlens_i32, void* out_bf16,
                                                       void* scratch, int32_t n_tokens, int32_t n_seqs,
                                                       int32_t max_seqlen, int32_t n_heads,
                                                       int32_t n_kv_heads, int32_t head_dim,
                                                       int32_t row_stride, int32_t k_off, int32_t v_off,
                                                       int32_t causal, void* status, void* stream);

/* A prefill chunk that continues a cached sequence (the reference has no scheduler, crates/sched/src/
 * lib.rs:1-30, and no paged cache; the anchors are QwenAttention::forward's score stage, crates/
 * transformers/src/attention.rs:226-296, made causal, and KvCache::get, crates/cache/src/flat.rs:254-304):
 * sequence s brings the query rows cu_seqlens_q[s] .. cu_seqlens_q[s+1] of q bf16 [n_q_tokens,
 * q_row_stride] (q heads at column 0, RoPE applied) and attends to its kv_lens[s] tokens in the paged
 * cache (k_pool / v_pool bf16 [n_pool_blocks, 16, n_kv_heads * head_dim], block_tables i32 [n_seqs,
 * max_blocks]); the K/V rows of the chunk's own tokens must already be stored there, so kv_lens[s] =
 * cached + new >= new, and query i sees keys 0 .. kv_lens[s] - new + i. out bf16 [n_q_tokens,
 * n_heads * head_dim]. total_kv_tokens >= sum(kv_lens), max_q_len / max_kv_len bound the grids (host
 * values). scratch: logismos_paged_prefix_attention_scratch_bytes(total_kv_tokens, n_seqs, n_kv_heads,
 * head_dim) bytes, 256-byte aligned: the first launch gathers each sequence's K rows and transposed V
 * through its block table into it, the second is the tcgen05 kernel of
 * logismos_launch_varlen_attention_tc_bf16. status (int32, may be NULL): 1 if a block id fell outside
 * the pool (zero rows are used) or kv_lens[s] is below the number of queries, 2 if a bounded wait
 * expired. head_dim 128 or 256. */
size_t logismos_paged_prefix_attention_scratch_bytes(int32_t total_kv_tokens, int32_t n_seqs,
                                                     int32_t n_kv_heads, int32_t head_dim);
uint32_t logismos_launch_paged_prefix_attention_tc_bf16(
    const void* q_bf16, int32_t q_row_stride, const void* cu_seqlens_q_i32, const void* kv_lens_i32,
    const void* k_pool_bf16, const void* v_pool_bf16, const void* block_tables_i32, int32_t max_blocks,
    int32_t n_pool_blocks, void* out_bf16, void* scratch, int32_t n_q_tokens, int32_t total_kv_tokens,
    int32_t n_seqs, int32_t max_q_len, int32_t max_kv_len, int32_t n_heads, int32_t n_kv_heads,
    int32_t head_dim, void* status, void* stream);

/* The same attention over a cache of TurboQuant 3-bit rows (logismos_launch_paged_kv_store_turbo3
 * below; pools u8 [n_pool_blocks, 16, n_kv_heads * head_dim / 128 * 56]): the gathering launch decodes
 * each head chunk (decode_turbo3_0_head, crates/quant/src/lib.rs:378-413) to bf16 on its way into the
 * scratch; everything else as above, a decode token included (one query per sequence). */
uint32_t logismos_launch_paged_prefix_attention_turbo3_bf16(
    const void* q_bf16, int32_t q_row_stride, const void* cu_seqlens_q_i32, const void* kv_lens_i32,
    const void* k_pool_t3, const void* v_pool_t3, const void* block_tables_i32, int32_t max_blocks,
    int32_t n_pool_blocks, void* out_bf16, void* scratch, int32_t n_q_tokens, int32_t total_kv_tokens,
    int32_t n_seqs, int32_t max_q_len, int32_t max_kv_len, int32_t n_heads, int32_t n_kv_heads,
    int32_t head_dim, void* status, void* stream);

/* mean_pool_masked -> l2_normalize -> linear_t(head) -> l2_normalize (cpu_f32 mod.rs:553-591 as
 * composed by StellaModel::encode_raw, crates/embed/src/stella.rs:231-246), mask all ones.
 * hidden f32 [n_tokens, hidden]; head_w bf16 [dim, hidden]; head_b f32 [dim]; out f32
 * [n_seqs, dim]; scratch_f32 [n_seqs, hidden] receives the pooled means. A sequence of length 0
 * pools to zeros. Three launches. */
uint32_t logismos_launch_pool_head_f32(const void* hidden_f32, const void* cu_seqlens_i32,
                                       const void* head_w_bf16, const void* head_b_f32,
                                       void* out_f32, void* scratch_f32, int32_t n_seqs,
                                       int32_t hidden, int32_t dim, void* stream);

/* ====================================================================================
 * Decode path. No reference GPU or CPU implementation exists for these; the anchors are the
 * contracts named beside each.
 * ==================================================================================== */

/* int4 group-32 dequant GEMV / skinny GEMM: y[b,n] = sum_g s[n,g] sum_{k in g} q[n,k] x[b,k].
 * codes u8 [n, k/2]: value k of a row in byte k/2, even k in the low nibble (the nibble order of
 * Turbo4Block, crates/quant/src/lib.rs:272-301), two's-complement 4-bit; scales fp16 [n, k/32];
 * x bf16 [batch, k]; y bf16 [batch, n]. 1 <= batch <= 64, k % 128 == 0. */
uint32_t logismos_launch_gemv_int4_g32_bf16(const void* codes_u8, const void* scales_f16,
                                            const void* x_bf16, void* y_bf16, int32_t batch,
                                            int32_t n, int32_t k, void* stream);
/* The same product with the fp32 accumulators stored unrounded, y f32 [batch, n]: the lm_head of a
 * decode step, whose logits go to decode::greedy (crates/decode/src/lib.rs:73-83), which takes the
 * first strict maximum of fp32 logits (a bf16 rounding would turn near-ties into ties). */
uint32_t logismos_launch_gemv_int4_g32_f32(const void* codes_u8, const void* scales_f16,
                                           const void* x_bf16, void* y_f32, int32_t batch, int32_t n,
                                           int32_t k, void* stream);

/* The same product, y bf16 [batch, n], with the kernel chosen by shape and batch
 * (logismos_skinny_int4_route: 0 = the streaming GEMV, 1 = the fused-dequant tensor-core linear below,
 * taken above 16 rows, for k >= 3 n, and from 8 rows up to n = 16384; needs k % 256 == 0, n % 4 == 0).
 * Route 1 accumulates in workspace_f32 [batch, n] (16-byte aligned, ALL ZERO on entry, left all zero
 * on return) and rounds once to bf16: two launches. workspace_f32 == NULL keeps the GEMV at every
 * batch. status_i32 as for logismos_launch_qlinear_int4_g32_acc_f32. */
int32_t logismos_skinny_int4_route(int32_t batch, int32_t n, int32_t k);
uint32_t logismos_launch_skinny_int4_g32_bf16(const void* codes_u8, const void* scales_f16,
                                              const void* x_bf16, void* y_bf16, int32_t batch, int32_t n,
                                              int32_t k, void* workspace_f32, void* status_i32, void* stream);

/* Expands int4 group-32 weights (same storage as above) to bf16 [n, k]: w = bf16(scale * code).
 * The prefill side of a mixed step runs its contractions on the tcgen05 GEMM over this expansion.
 * k % 32 == 0. */
uint32_t logismos_launch_dequant_int4_g32_bf16(const void* codes_u8, const void* scales_f16,
                                               void* out_bf16, int32_t n, int32_t k, void* stream);

/* Quantises fp32 weights [n, k] to the int4 group-32 storage above, on the device: per group of 32
 * values along k, scale = fp16(max|w| / 7), code = clamp(round-half-even(w / scale), -8, 7) (0 for an
 * all-zero group), packed in the Turbo4Block nibble order (crates/quant/src/lib.rs:272-301). The
 * reference has no quantiser (turbo4 encode returns Unsupported, crates/quant/src/lib.rs:361-367);
 * the output is integer and is checked bit for bit against the CPU definition. k % 32 == 0. */
uint32_t logismos_launch_quantize_int4_g32(const void* w_f32, void* codes_u8, void* scales_f16,
                                           int32_t n, int32_t k, void* stream);

/* acc[m, n] += A[m, k] * dequant(W)[n, k]^T for 1 <= m <= 256 tokens, int4 group-32 weights (storage
 * as above), dequantisation fused into the tensor-core operand pipeline. The linear of decode and
 * small mixed steps: linear_t (cpu_f32/mod.rs:271-345) on the dequantised matrix. a bf16 [m, k]
 * rows lda apart; acc fp32 [m, n] rows ldc apart (the fp32 residual stream itself for the output
 * projections, or a zeroed workspace finished by the call below). Weights enter the MMA as
 * bf16(code) * bf16(scale). k % 256 == 0. Slices of k meet in fp32 reductions: with several slices
 * the last bits of acc may differ between runs. status_i32 as for logismos_launch_linear_t_bf16. */
uint32_t logismos_launch_qlinear_int4_g32_acc_f32(const void* a_bf16, const void* codes_u8,
                                                  const void* scales_f16, void* acc_f32, int32_t m,
                                                  int32_t n, int32_t k, int32_t lda, int32_t ldc,
                                                  void* status_i32, void* stream);
/* The same launch with the caller's promise that no work still in flight on the stream writes the
 * codes or scales (model weights uploaded once): with dependent launch on, the kernel fills its weight
 * ring before the preceding kernel has finished. */
uint32_t logismos_launch_qlinear_int4_g32_acc_f32_static(const void* a_bf16, const void* codes_u8,
                                                         const void* scales_f16, void* acc_f32,
                                                         int32_t m, int32_t n, int32_t k, int32_t lda,
                                                         int32_t ldc, void* status_i32, void* stream);
/* Finishes an accumulation workspace: out bf16 [m, n] = acc (+ bias), or with swiglu != 0,
 * out bf16 [m, n/2] = silu(gate) * up over columns interleaved in blocks of 32 (the LG_EPI_SWIGLU
 * row order); acc is left zeroed for the next accumulation. n % 4 == 0 (n % 64 == 0 for swiglu). */
uint32_t logismos_launch_qlinear_finish_bf16(void* acc_f32, const void* bias_f32, void* out_bf16,
                                             int32_t m, int32_t n, int32_t ld_acc, int32_t ldc,
                                             int32_t swiglu, void* stream);

/* Paged-attention decode with fused KV append. The paged cache keeps the row layout of
 * FlatKvCache (crates/cache/src/flat.rs:36-69: one row = all kv heads of one token, contiguous):
 * k_pool / v_pool bf16 [n_pool_blocks, block_size = 16, n_kv_heads * head_dim]; logical token t
 * of sequence s lives in block block_tables[s * max_blocks + t / 16], slot t % 16.
 * For each sequence: the new token's k/v row (new_k / new_v bf16 [n_seqs, n_kv_heads*head_dim])
 * is written at position context_lens[s] - 1 (context_lens counts the new token), then
 * q bf16 [n_seqs, n_heads * head_dim] attends causally to positions 0 .. context_lens[s] - 1.
 * new_k == NULL skips the append. head_dim 128 or 256, n_heads / n_kv_heads <= 16. Every
 * context_lens[s] must be >= 1 (a sequence without a key would get no chunk and its output row
 * would stay unwritten; logismos_build_decode_chunks rejects such a batch).
 * Work is split along the context in chunks of `chunk_tokens` (a multiple of 64):
 * chunk_offsets i32 [n_seqs + 1] is the exclusive prefix sum of ceil(context_lens / chunk_tokens)
 * and total_chunks its last entry (host copy). scratch must hold
 * logismos_paged_decode_scratch_bytes(total_chunks, n_heads, head_dim) bytes. status_i32 (may be
 * NULL) receives 1 if a block id fell outside the pool (that block is then skipped). */
size_t logismos_paged_decode_scratch_bytes(int32_t total_chunks, int32_t n_heads, int32_t head_dim);
uint32_t logismos_launch_paged_attention_decode_bf16(
    const void* q_bf16, void* k_pool_bf16, void* v_pool_bf16, const void* new_k_bf16,
    const void* new_v_bf16, const void* block_tables_i32, const void* context_lens_i32,
    const void* chunk_offsets_i32, void* out_bf16, void* scratch, void* status_i32, int32_t n_seqs,
    int32_t total_chunks, int32_t chunk_tokens, int32_t max_blocks, int32_t n_pool_blocks,
    int32_t n_heads, int32_t n_kv_heads, int32_t head_dim, void* stream);

/* Paged-attention decode for callers that cannot allocate device memory where they decode (an
 * engine that has given all free HBM to its KV pool, a thread where an allocation's device-wide
 * synchronisation is unacceptable). It has no counterpart in the reference. Same arguments and
 * results as logismos_launch_paged_attention_decode_bf16 minus `scratch`: the per-chunk partials
 * go to a buffer of LOGISMOS_PAGED_DECODE_STATIC_SCRATCH_BYTES built into the library image (each
 * GPU that loads the library holds it until exit). The call allocates nothing.
 *   - Limit: logismos_paged_decode_scratch_bytes(total_chunks, n_heads, head_dim) must not exceed
 *     the constant (8 MiB: e.g. 1008 chunks at 16 heads x 128); beyond it the call returns
 *     cudaErrorMemoryAllocation (2) without launching and says why on stderr.
 *   - The first call on each device looks up the buffer's device address (that device must be
 *     current, as for any launch) and caches it; make that first call before starting any stream
 *     capture on the device. "Allocates nothing" holds from then on: the buffer belongs to the
 *     library's device code, which the CUDA runtime may load lazily at the first call into the
 *     library on a device, and loading takes device memory (the 8 MiB included). A host that then
 *     grabs all free HBM for its KV pool must therefore make one small valid call of this entry
 *     point on each device BEFORE that grab.
 *   - All calls share the one buffer and it keeps the previous call's contents; nothing in it needs
 *     clearing, since a launch only reads partials it wrote itself. For the same reason two calls
 *     whose kernels can overlap on the GPU (different streams, or threads) race on it: serialise
 *     them, or use the entry point with caller scratch. */
#define LOGISMOS_PAGED_DECODE_STATIC_SCRATCH_BYTES (8u * 1024u * 1024u)
uint32_t logismos_launch_paged_attention_decode_noalloc_bf16(
    const void* q_bf16, void* k_pool_bf16, void* v_pool_bf16, const void* new_k_bf16,
    const void* new_v_bf16, const void* block_tables_i32, const void* context_lens_i32,
    const void* chunk_offsets_i32, void* out_bf16, void* status_i32, int32_t n_seqs,
    int32_t total_chunks, int32_t chunk_tokens, int32_t max_blocks, int32_t n_pool_blocks,
    int32_t n_heads, int32_t n_kv_heads, int32_t head_dim, void* stream);

/* KvCache::put for a ragged batch (crates/cache/src/lib.rs:57-82): row i of k/v bf16
 * [n_tokens, row_elems] is stored at physical slot slot_mapping[i] (i64: block * 16 + offset).
 * A slot outside the pool is skipped and sets *status to 1. */
uint32_t logismos_launch_paged_kv_store_bf16(const void* k_bf16, const void* v_bf16,
                                             int32_t src_row_stride, void* k_pool_bf16,
                                             void* v_pool_bf16, const void* slot_mapping_i64,
                                             int32_t n_tokens, int32_t row_elems,
                                             int64_t n_pool_slots, void* status_i32, void* stream);
/* KvCache::get: the first len rows of one sequence gathered through its block table into
 * contiguous bf16 [len, row_elems] buffers (bit-exact copy). */
uint32_t logismos_launch_paged_kv_gather_bf16(const void* k_pool_bf16, const void* v_pool_bf16,
                                              const void* block_table_i32, int32_t table_len,
                                              int32_t len, int32_t row_elems,
                                              int32_t n_pool_blocks, void* k_out_bf16,
                                              void* v_out_bf16, void* status_i32, void* stream);

/* The same cache with TurboQuant 3-bit rows: KvCache::put / get (crates/cache/src/lib.rs:57-82) through
 * encode_turbo3_0_head / decode_turbo3_0_head (crates/quant/src/lib.rs:316-413: L2 norm, 128-point
 * Walsh-Hadamard transform, 8-centroid codebook, four 14-byte blocks per 128-value head chunk). A pool
 * row holds row_elems / 128 chunks of 56 bytes (logismos_turbo3_row_bytes) instead of row_elems bf16:
 * pools are u8 [n_pool_blocks, 16, row_bytes]. The store encodes rows of k / v bf16 [n_tokens,
 * row_elems] (widened to fp32 first) into slot_mapping's slots; the gather decodes the first len rows of
 * one sequence to bf16 [len, row_elems] (fp32 decode rounded once). Bytes and values are identical to
 * the CPU definition (the arithmetic follows it operation by operation). row_elems % 128 == 0. */
size_t logismos_turbo3_row_bytes(int32_t row_elems);
uint32_t logismos_launch_paged_kv_store_turbo3(const void* k_bf16, const void* v_bf16, int32_t src_row_stride,
                                               void* k_pool_t3, void* v_pool_t3, const void* slot_mapping_i64,
                                               int32_t n_tokens, int32_t row_elems, int64_t n_pool_slots,
                                               void* status_i32, void* stream);
uint32_t logismos_launch_paged_kv_gather_turbo3(const void* k_pool_t3, const void* v_pool_t3,
                                                const void* block_table_i32, int32_t table_len, int32_t len,
                                                int32_t row_elems, int32_t n_pool_blocks, void* k_out_bf16,
                                                void* v_out_bf16, void* status_i32, void* stream);

/* dst[r, :] = src[idx[r], :] for fp32 rows (bit-exact copy): picks the last token row of every
 * sequence of a packed step before the final norm and the lm_head. An index outside
 * [0, n_src_rows) yields a zero row and sets *status to 1. width % 4 == 0. */
uint32_t logismos_launch_gather_rows_f32(const void* src_f32, const void* idx_i32, void* dst_f32,
                                         int32_t n_rows, int32_t width, int32_t n_src_rows,
                                         void* status_i32, void* stream);

/* gated_delta_rule_recurrent_fwd (crates/kernels/src/gated_delta_rule/cpu.rs:92-182), one decode
 * step for a batch of sequences and heads: state f32 [n_seqs, heads, K=128, V=128] updated in
 * place; q,k f32/bf16 ... see gdn.cu. q, k bf16 [n_seqs, heads, 128]; v bf16 [n_seqs, heads, 128];
 * g, beta f32 [n_seqs, heads]; o bf16 [n_seqs, heads, 128]. */
uint32_t logismos_launch_gdn_decode_step(void* state_f32, const void* q_bf16, const void* k_bf16,
                                         const void* v_bf16, const void* g_f32,
                                         const void* beta_f32, void* o_bf16, int32_t n_seqs,
                                         int32_t heads, float scale, void* stream);

/* One decode token per sequence straight from the fp32 accumulation workspace of the fused input
 * projection (logismos_launch_qlinear_int4_g32_acc_f32 over the row blocks q | k | v | z | a | b):
 * logismos_launch_gdn_finish and the one-token case of logismos_launch_gdn_prefill (with the output gate)
 * in a single launch, same arithmetic in the same order. acc f32 [n_seqs, ld_acc] is left zeroed. Row i
 * is sequence i; o bf16 [n_seqs, heads, 128]; state pool, state_slots and fresh as below. pair_count i32
 * [n_seqs * heads], all zero on entry and on return. The states, state_slots and fresh must not be
 * written by work still in flight on the stream (they are read ahead of the dependency wait). */
uint32_t logismos_launch_gdn_decode_from_acc(void* state_f32, void* acc_f32, int32_t ld_acc,
                                             const void* A_log_f32, const void* dt_bias_f32, void* o_bf16,
                                             const void* state_slots_i32, const void* fresh_u8,
                                             void* pair_count_i32, int32_t n_seqs, int32_t heads,
                                             float scale, void* stream);

/* gated_delta_rule_chunk_fwd / recurrent_fwd over a ragged batch (cpu.rs:92-249): sequence i owns
 * token rows cu_seqlens[i] .. cu_seqlens[i+1] of q, k, v bf16 [n_tokens, heads, 128], g, beta f32
 * [n_tokens, heads]; state f32 [n_seqs, heads, 128, 128] is the initial state on entry and the
 * final state on return; o bf16 [n_tokens, heads, 128]. Tokens are processed in order.
 * q, k, v may be column blocks of a wider projection output: token t, head h starts at
 * t * qkv_stride + h * 128 (elements; qkv_stride % 8 == 0, 16-byte aligned bases). state_slots i32 [n_seqs] (may be NULL = identity) selects
 * each sequence's slot in a state pool [n_slots, heads, 128, 128]; fresh u8 [n_seqs] (may be NULL)
 * marks sequences that start here and therefore begin from the zero state. gate_z bf16 (may be
 * NULL), addressed like q, k, v, applies the layer's output gate in the same pass:
 * o *= silu(z) in fp32 before the bf16 rounding. mode selects the kernel shape: 1 = throughput (64
 * value columns per CTA; decode and many sequences), 2 = latency (32 columns per CTA: more
 * CTAs per head for a few long sequences), 0 = by the number of (sequence, head) pairs.
 * LG_GDN_STATIC_STATE, or-ed into mode, is the caller's promise that no work still in flight on the
 * stream writes the state pool, cu_seqlens, state_slots or fresh (they were left by an earlier model
 * step that has completed): with dependent launch on, the kernel then reads its states while the
 * kernels that produce q, k, v and the gates are still running. */
enum { LG_GDN_STATIC_STATE = 0x100 };
uint32_t logismos_launch_gdn_prefill(void* state_f32, const void* q_bf16, const void* k_bf16,
                                     const void* v_bf16, const void* g_f32, const void* beta_f32,
                                     void* o_bf16, const void* gate_z_bf16, const void* cu_seqlens_i32,
                                     const void* state_slots_i32, const void* fresh_u8, int32_t n_seqs,
                                     int32_t heads, int32_t qkv_stride, float scale, int32_t mode,
                                     void* stream);
/* The same function in chunk-parallel form (gated_delta_rule_chunk_fwd, cpu.rs:201-249): the 64 tokens
 * of a chunk are resolved together by matrix products (a triangular solve for the in-chunk
 * dependencies, tensor-core products against the carried state), so a long prompt is not bound by a
 * token-serial chain. Arguments as logismos_launch_gdn_prefill. The state stays fp32 and enters the
 * products rounded to bf16: outputs within 2e-2 of the recurrence, final state within 1e-2.
 * scratch (128-byte aligned, logismos_gdn_chunked_scratch_bytes(n_tokens, n_seqs, heads) bytes, n_tokens
 * = cu_seqlens[n_seqs] - cu_seqlens[0] or more) selects the two-launch form: everything of a chunk that
 * does not involve the carried state is computed for all chunks of the batch at once (a CTA per chunk
 * and head) and parked in scratch, then each sequence's chunks are chained with the three products that
 * touch the state. scratch == NULL keeps the one-launch form (a CTA per sequence, head and value-column
 * half does all of it chunk after chunk). Same results within the stated tolerance. */
size_t logismos_gdn_chunked_scratch_bytes(int32_t n_tokens, int32_t n_seqs, int32_t heads);
uint32_t logismos_launch_gdn_chunked(void* state_f32, const void* q_bf16, const void* k_bf16,
                                     const void* v_bf16, const void* g_f32, const void* beta_f32,
                                     void* o_bf16, const void* gate_z_bf16, const void* cu_seqlens_i32,
                                     const void* state_slots_i32, const void* fresh_u8, int32_t n_seqs,
                                     int32_t heads, int32_t qkv_stride, float scale, void* scratch,
                                     int32_t n_tokens, void* stream);
/* Inputs of the recurrence from the layer's projections (no reference code; the formulas are
 * those of research/14-gdn-aiter-preflight.md:190-198, :209-219): q, k bf16 [n_tokens, heads, 128]
 * are L2-normalised per head row in place (l2_norm_in_place, cpu.rs:19-34);
 * g = -exp(A_log[h]) * softplus(a + dt_bias[h]) (softplus(x) = x for x > 20), beta = sigmoid(b),
 * g, beta f32 [n_tokens, heads], A_log, dt_bias f32 [heads]. q, k rows start at
 * t * qk_stride + h * 128; a, b are read at t * ab_stride + h (f32). */
uint32_t logismos_launch_gdn_prepare(void* q_bf16, void* k_bf16, const void* a_f32, const void* b_f32,
                                     const void* A_log_f32, const void* dt_bias_f32, void* g_f32,
                                     void* beta_f32, int32_t n_tokens, int32_t heads,
                                     int32_t qk_stride, int32_t ab_stride, void* stream);
/* logismos_launch_gdn_prepare fused with the finishing of the input projection's fp32 accumulation
 * workspace (logismos_launch_qlinear_int4_g32_acc_f32 into acc f32 [n_tokens, ld_acc], columns
 * q | k | v | z [heads * 128 each] | a | b [heads each]): q and k are L2-normalised in fp32, q, k, v, z
 * are rounded to bf16 once into proj [n_tokens, ld_proj] (columns q | k | v | z), g and beta f32
 * [n_tokens, heads] are computed from a and b, and the workspace is left zeroed. */
uint32_t logismos_launch_gdn_finish(void* acc_f32, int32_t ld_acc, const void* A_log_f32, const void* dt_bias_f32,
                                    void* proj_bf16, int32_t ld_proj, void* g_f32, void* beta_f32,
                                    int32_t n_tokens, int32_t heads, void* stream);
/* x[t, j] *= sigmoid(gate[t, j]) (mode 0) or silu(gate[t, j]) (mode 1), bf16 in place, fp32 math;
 * rows of x and gate have their own strides (elements). The output gates of the hybrid decoder's
 * attention and linear-attention layers. n % 8 == 0. */
uint32_t logismos_launch_gated_mul_bf16(void* x_bf16, int32_t x_stride, const void* gate_bf16,
                                        int32_t gate_stride, int32_t rows, int32_t n, int32_t mode,
                                        void* stream);

/* x[i] += d[i], fp32, n % 4 == 0: joins a partial sum that was reduced across tensor-parallel ranks
 * into the residual stream (no reference counterpart: the reference has no tensor parallelism). */
uint32_t logismos_launch_add_f32(void* x_f32, const void* d_f32, int64_t n, void* stream);

/* decode::greedy (crates/decode/src/lib.rs:73-83): argmax per row, first maximum wins, NaN
 * never selected. logits bf16 or f32 [rows, n]; out u32 [rows]. */
uint32_t logismos_launch_greedy_argmax(const void* logits, int32_t logits_f32, void* out_u32,
                                       int32_t rows, int32_t n, void* stream);

/* ====================================================================================
 * Sampling chain on the device: the logit processors and the multinomial sampler of
 * crates/decode (chain.rs:33-76 runs processors in insertion order, then the sampler), each as one
 * launch over fp32 logits [rows, n] IN PLACE, so a caller keeps the reference's free ordering. Rows are
 * independent. Rows must hold at least one finite logit.
 * ==================================================================================== */

/* TemperatureScale (processors.rs:18-28): t = max(temperature, 1e-6); |t - 1| < 1e-9 is the identity;
 * otherwise every logit is divided by t. */
uint32_t logismos_launch_temperature_f32(void* logits_f32, int32_t rows, int32_t n, float temperature,
                                         void* stream);
/* TopK (processors.rs:50-82): k == 0 or k >= n is the identity; otherwise every NaN and every logit
 * below the k-th largest becomes -inf (ties with the k-th largest survive). Exact. */
uint32_t logismos_launch_top_k_f32(void* logits_f32, int32_t rows, int32_t n, int32_t k, void* stream);
/* TopP (processors.rs:89-122): p clamped to [0, 1]; p >= 1 is the identity; otherwise the smallest
 * prefix of the tokens in order of descending probability (equal probabilities in index order) whose
 * softmax mass reaches p is kept, the rest becomes -inf. The reference normalises by a sequential
 * fp32 sum over the vocabulary (about 1e-5 to 1e-4 of relative rounding error at 151936 terms); the
 * device sums pairwise, so the two nuclei can differ by the tokens whose cumulative mass lies within
 * that error of p. */
uint32_t logismos_launch_top_p_f32(void* logits_f32, int32_t rows, int32_t n, float p, void* stream);
/* MinP (processors.rs:130-146): p clamped; p <= 0 is the identity; tokens whose probability is below
 * p times the largest probability become -inf. */
uint32_t logismos_launch_min_p_f32(void* logits_f32, int32_t rows, int32_t n, float p, void* stream);
/* RepetitionPenalty (processors.rs:160-181): row r lists counts[r] <= max_tokens token ids in
 * tokens_u32 [rows, max_tokens]; for each in order (a token listed twice is penalised twice; ids >= n
 * are skipped) a positive logit is divided by penalty, any other multiplied. |penalty - 1| < 1e-9 is
 * the identity. */
uint32_t logismos_launch_repetition_penalty_f32(void* logits_f32, int32_t rows, int32_t n,
                                                const void* tokens_u32, const void* counts_i32,
                                                int32_t max_tokens, float penalty, void* stream);
/* MultinomialSampler::sample (sampler.rs:31-58) with the uniform draw of every row supplied by the
 * caller (uniforms_f32 [rows], each in [0, 1); the reference draws it from its RNG at that point):
 * probabilities are exp(l - max) of the finite logits over their sum; the token is the first index
 * whose cumulative probability exceeds the draw; a row without mass falls back to greedy; out u32
 * [rows]. */
uint32_t logismos_launch_multinomial_f32(const void* logits_f32, int32_t rows, int32_t n,
                                         const void* uniforms_f32, void* out_u32, void* stream);

/* ====================================================================================
 * Host-side index builders (no device work). crates/sched is an empty scaffold in the reference
 * (src/lib.rs:1-30); these define the packing of a mixed prefill/decode step.
 * ==================================================================================== */

/* For sequence i with cached_lens[i] tokens already in the cache and new_lens[i] new tokens:
 * cu_seqlens [n+1], positions [total] (continuing from the cached length), slot_mapping [total]
 * (block * block_size + offset through block_tables [n, max_blocks]), seq_ids [total].
 * Returns the total token count, or -1 if a needed table entry is negative or >= n_pool_blocks. */
int64_t logismos_build_packing(const int32_t* host_cached_lens, const int32_t* host_new_lens,
                               int32_t n_seqs, const int32_t* host_block_tables,
                               int32_t max_blocks, int32_t block_size, int32_t n_pool_blocks,
                               int32_t* host_cu_seqlens, int32_t* host_positions,
                               int64_t* host_slot_mapping, int32_t* host_seq_ids);
/* chunk_offsets [n+1] for the paged decode kernel; returns total_chunks, or -1 if a context length
 * is below 1 or the chunk count overflows. */
int32_t logismos_build_decode_chunks(const int32_t* host_context_lens, int32_t n_seqs,
                                     int32_t chunk_tokens, int32_t* host_chunk_offsets);
/* chunk_tokens for one step's contexts: the largest of 512, 1024, 2048 that leaves the decode launch at
 * least 32768 / head_dim CTAs (chunks x kv heads); 512 otherwise. Host-side, no device work. */
int32_t logismos_pick_decode_chunk(const int32_t* host_context_lens, int32_t n_seqs,
                                   int32_t n_kv_heads, int32_t head_dim);

#ifdef __cplusplus
}
#endif
#endif
