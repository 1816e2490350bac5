// Attention over ragged batches without materialising scores:
//   - varlen_attention: the score / softmax / PV stage of QwenAttention::forward
//     (crates/transformers/src/attention.rs:226-296), bidirectional (encoder) or causal,
//     sequences delimited by cu_seqlens;
//   - paged_attention_decode: one query token per sequence against a paged KV cache addressed
//     through block tables, with the new token's K/V row appended in the same launch, the
//     context split into chunks (flash-decoding) and merged by a second small kernel.
// Both use the same warp-level building block: a 16-row query tile held as mma.sync A fragments,
// K/V tiles staged in shared memory with cp.async (128-bit, XOR-swizzled 16-byte chunks),
// ldmatrix fragment loads, bf16 tensor-core products with fp32 accumulation and an online
// (running max / running sum) softmax in fp32, exp2 domain.
// Scores are scaled after the dot product (attention.rs:239-241); the GQA mapping is
// q head j -> kv head j / (n_heads / n_kv_heads) (attention.rs:366-382).
#include <cstdio>
#include <mutex>

#include "common.cuh"
#include "logismos_kernels.h"

namespace {

using namespace lg;

// The kernels are templates on the head dimension HD (128 or 256): a head row is HD bf16 values,
// i.e. HD/8 chunks of 16 bytes in shared memory, HD/16 k-steps for Q.K^T and HD/8 output tiles for P.V.
constexpr float kLog2e = 1.4426950408889634f;

// shared-memory address of 16-byte chunk `chunk` of row `row` in a [rows][HD] bf16 tile
template <int HD>
LG_DEVINL uint32_t tile_addr(uint32_t base, int row, int chunk) {
  return base + (uint32_t)row * (HD * 2) + (uint32_t)((chunk ^ (row & 7)) << 4);
}

// A fragments (16 rows x HD) of a query tile staged at `qbase`: qf[ks] covers k = 16ks..16ks+15
template <int HD>
LG_DEVINL void load_q_frags(uint32_t qbase, int lane, uint32_t (&qf)[HD / 16][4]) {
  const int mat = lane >> 3, r = lane & 7;
  const int row = r + 8 * (mat & 1);
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) ldmatrix_x4(qf[ks], tile_addr<HD>(qbase, row, 2 * ks + (mat >> 1)));
}

// s[t][:] = Q(16xHD) . K(tokens tok0+8t .. +7)^T for NT 8-token tiles of the K tile at kbase
template <int NT, int HD>
LG_DEVINL void qk_tile(const uint32_t (&qf)[HD / 16][4], uint32_t kbase, int tok0, int lane, float (&s)[NT][4]) {
  const int mat = lane >> 3, r = lane & 7;
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) s[t][i] = 0.0f;
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
    for (int t = 0; t < NT; t += 2) {
      uint32_t b[4];
      ldmatrix_x4(b, tile_addr<HD>(kbase, tok0 + 8 * (t + (mat >> 1)) + r, 2 * ks + (mat & 1)));
      const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
      mma_bf16_16816(s[t], qf[ks], b0, s[t]);
      mma_bf16_16816(s[t + 1], qf[ks], b1, s[t + 1]);
    }
  }
}

// o(16xHD) += P(16 x 8NT tokens) . V(tokens tok0.. , HD)
template <int NT, int HD>
LG_DEVINL void pv_tile(const float (&p)[NT][4], uint32_t vbase, int tok0, int lane, float (&o)[HD / 8][4]) {
  const int mat = lane >> 3, r = lane & 7;
#pragma unroll
  for (int kt = 0; kt < NT / 2; ++kt) {
    uint32_t a[4];
    a[0] = pack_bf16x2(p[2 * kt][0], p[2 * kt][1]);
    a[1] = pack_bf16x2(p[2 * kt][2], p[2 * kt][3]);
    a[2] = pack_bf16x2(p[2 * kt + 1][0], p[2 * kt + 1][1]);
    a[3] = pack_bf16x2(p[2 * kt + 1][2], p[2 * kt + 1][3]);
#pragma unroll
    for (int j = 0; j < HD / 8; j += 2) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, tile_addr<HD>(vbase, tok0 + 16 * kt + 8 * (mat & 1) + r, j + (mat >> 1)));
      const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
      mma_bf16_16816(o[j], a, b0, o[j]);
      mma_bf16_16816(o[j + 1], a, b1, o[j + 1]);
    }
  }
}

// Online softmax step over s (raw scores, -inf where masked) for the two rows a lane owns
// (g and g+8). m/l are running max (raw domain) and running sum; o is rescaled in place and
// s is overwritten with the probabilities exp2((s - m) * sl2).
template <int NT, int DT>
LG_DEVINL void softmax_step(float (&s)[NT][4], float (&m)[2], float (&l)[2], float (&o)[DT][4], float sl2) {
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    mx0 = fmaxf(mx0, fmaxf(s[t][0], s[t][1]));
    mx1 = fmaxf(mx1, fmaxf(s[t][2], s[t][3]));
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
  const float use0 = (mn0 == -INFINITY) ? 0.0f : mn0, use1 = (mn1 == -INFINITY) ? 0.0f : mn1;
  const float a0 = exp2f((m[0] - use0) * sl2), a1 = exp2f((m[1] - use1) * sl2);
  float rs0 = 0.0f, rs1 = 0.0f;
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    s[t][0] = exp2f((s[t][0] - use0) * sl2);
    s[t][1] = exp2f((s[t][1] - use0) * sl2);
    s[t][2] = exp2f((s[t][2] - use1) * sl2);
    s[t][3] = exp2f((s[t][3] - use1) * sl2);
    rs0 += s[t][0] + s[t][1];
    rs1 += s[t][2] + s[t][3];
  }
  l[0] = l[0] * a0 + rs0;
  l[1] = l[1] * a1 + rs1;
  m[0] = mn0;
  m[1] = mn1;
#pragma unroll
  for (int j = 0; j < DT; ++j) {
    o[j][0] *= a0; o[j][1] *= a0;
    o[j][2] *= a1; o[j][3] *= a1;
  }
}

// ================================ varlen (encoder / prefill) ===================================

constexpr int kQTile = 64, kVarlenThreads = 128;
// key/value tile: 64 tokens at head_dim 128, 32 at head_dim 256 (same bytes, same register budget)
template <int HD> struct KvTile { static constexpr int value = HD == 128 ? 64 : 32; };

// stage ROWS rows [t0, t0+ROWS) of one head (HD bf16 per row) into a swizzled tile; rows >= limit are zeroed
template <int HD, int ROWS>
LG_DEVINL void stage_rows(uint32_t sbase, uint8_t* sgen, const __nv_bfloat16* src, int64_t row_stride,
                          int t0, int limit, int tid) {
  constexpr int CH = HD / 8;
#pragma unroll
  for (int i = 0; i < (ROWS * CH) / kVarlenThreads; ++i) {
    const int u = tid + i * kVarlenThreads;
    const int row = u / CH, chunk = u % CH;
    const uint32_t dst = tile_addr<HD>(sbase, row, chunk);
    if (t0 + row < limit) {
      cp_async16(dst, src + (int64_t)(t0 + row) * row_stride + chunk * 8);
    } else {
      *reinterpret_cast<uint4*>(sgen + (dst - sbase)) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

template <bool CAUSAL, int HD>
__global__ void __launch_bounds__(kVarlenThreads, HD == 128 ? 3 : 1)
varlen_attention_kernel(const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ cu,
                        __nv_bfloat16* __restrict__ out, int n_heads, int n_kv, int row_stride,
                        int k_off, int v_off, float sl2) {
  lg::pdl_prologue();
  extern __shared__ __align__(128) uint8_t smem[];
  const int seq = blockIdx.z, h = blockIdx.y, qt = blockIdx.x;
  const int s0 = cu[seq], len = cu[seq + 1] - s0;
  const int q0 = qt * kQTile;
  if (q0 >= len) return;
  const int kvh = h / (n_heads / n_kv);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  constexpr int D = HD, kRowBytes = HD * 2, kKvTile = KvTile<HD>::value, NT = kKvTile / 8, DT = HD / 8;
  constexpr int KTB = kKvTile * kRowBytes;  // bytes of one K (or V) tile: 16 KB

  // two K/V tile buffers of 16 KB + 16 KB; the query tile is staged in the second buffer (all of
  // it at head_dim 256) and lives in registers from then on, so 64 KB per CTA
  uint8_t* sk[2] = {smem, smem + 2 * KTB};
  uint8_t* sv[2] = {smem + KTB, smem + 3 * KTB};
  uint8_t* sq = sk[1];
  const uint32_t sq_a = smem_u32(sq);
  const uint32_t sk_a[2] = {smem_u32(sk[0]), smem_u32(sk[1])};
  const uint32_t sv_a[2] = {smem_u32(sv[0]), smem_u32(sv[1])};

  const __nv_bfloat16* qsrc = qkv + (int64_t)s0 * row_stride + h * D;
  const __nv_bfloat16* ksrc = qkv + (int64_t)s0 * row_stride + k_off + kvh * D;
  const __nv_bfloat16* vsrc = qkv + (int64_t)s0 * row_stride + v_off + kvh * D;

  const int kv_end = CAUSAL ? min(len, q0 + kQTile) : len;
  const int n_tiles = (kv_end + kKvTile - 1) / kKvTile;

  stage_rows<HD, kQTile>(sq_a, sq, qsrc, row_stride, q0, len, tid);
  stage_rows<HD, kKvTile>(sk_a[0], sk[0], ksrc, row_stride, 0, len, tid);
  stage_rows<HD, kKvTile>(sv_a[0], sv[0], vsrc, row_stride, 0, len, tid);
  cp_async_commit();

  uint32_t qf[HD / 16][4];
  float o[DT][4];
#pragma unroll
  for (int j = 0; j < DT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[j][i] = 0.0f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

  cp_async_wait<0>();
  __syncthreads();
  load_q_frags<HD>(sq_a + warp * 16 * kRowBytes, lane, qf);
  __syncthreads();  // the query tile's buffer is free for K/V tile 1 from here on

  for (int it = 0; it < n_tiles; ++it) {
    const int buf = it & 1;
    if (it + 1 < n_tiles) {
      stage_rows<HD, kKvTile>(sk_a[buf ^ 1], sk[buf ^ 1], ksrc, row_stride, (it + 1) * kKvTile, len, tid);
      stage_rows<HD, kKvTile>(sv_a[buf ^ 1], sv[buf ^ 1], vsrc, row_stride, (it + 1) * kKvTile, len, tid);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    float s[NT][4];
    qk_tile<NT, HD>(qf, sk_a[buf], 0, lane, s);
    // mask keys beyond the sequence and (causal) beyond the query position
    const int kbase = it * kKvTile;
    const int qrow0 = q0 + warp * 16 + g, qrow1 = qrow0 + 8;
    if (kbase + kKvTile > len || (CAUSAL && kbase + kKvTile > q0 + warp * 16)) {
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const int k0 = kbase + 8 * t + 2 * c, k1 = k0 + 1;
        if (k0 >= len || (CAUSAL && k0 > qrow0)) s[t][0] = -INFINITY;
        if (k1 >= len || (CAUSAL && k1 > qrow0)) s[t][1] = -INFINITY;
        if (k0 >= len || (CAUSAL && k0 > qrow1)) s[t][2] = -INFINITY;
        if (k1 >= len || (CAUSAL && k1 > qrow1)) s[t][3] = -INFINITY;
      }
    }
    softmax_step<NT, DT>(s, m, l, o, sl2);
    pv_tile<NT, HD>(s, sv_a[buf], 0, lane, o);
    __syncthreads();  // tile fully consumed before it is overwritten two iterations later
  }

  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
  const float inv0 = l[0] > 0.0f ? 1.0f / l[0] : 0.0f, inv1 = l[1] > 0.0f ? 1.0f / l[1] : 0.0f;
  const int r0 = q0 + warp * 16 + g, r1 = r0 + 8;
  const int64_t ostride = (int64_t)n_heads * D;
#pragma unroll
  for (int j = 0; j < DT; ++j) {
    const int d = 8 * j + 2 * c;
    if (r0 < len)
      *reinterpret_cast<uint32_t*>(out + (int64_t)(s0 + r0) * ostride + h * D + d) = pack_bf16x2(o[j][0] * inv0, o[j][1] * inv0);
    if (r1 < len)
      *reinterpret_cast<uint32_t*>(out + (int64_t)(s0 + r1) * ostride + h * D + d) = pack_bf16x2(o[j][2] * inv1, o[j][3] * inv1);
  }
}

// ================================ paged decode =================================================

inline int lg_sm_count_cached() {
  static int n = 0;
  if (n) return n;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (n <= 0) n = 148;
  return n;
}

constexpr int kBlock = 16;          // tokens per KV block
// W warps per CTA, each with its own ring of S stages
template <int HD, int W, int S>
struct DecCfg {
  static constexpr int kRowBytes = HD * 2;
  static constexpr int kStageBytes = 2 * kBlock * kRowBytes;  // K block + V block of one kv head: 8 KB at head_dim 128
  static constexpr int kSmem = W * S * kStageBytes + 16 * kRowBytes;  // + Q tile
};

// issue the cp.async copies of one 16-token block (K then V) of kv head `kvh` into a warp's stage
template <int HD>
LG_DEVINL void stage_block(uint32_t sbase, const __nv_bfloat16* kpool, const __nv_bfloat16* vpool,
                           int64_t phys_block, int row_elems, int kvh, int lane) {
  constexpr int CH = HD / 8;
  const __nv_bfloat16* kb = kpool + (phys_block * kBlock) * (int64_t)row_elems + kvh * HD;
  const __nv_bfloat16* vb = vpool + (phys_block * kBlock) * (int64_t)row_elems + kvh * HD;
#pragma unroll
  for (int i = 0; i < (kBlock * CH) / 32; ++i) {
    const int u = lane + 32 * i;
    const int row = u / CH, chunk = u % CH;
    cp_async16(tile_addr<HD>(sbase, row, chunk), kb + (int64_t)row * row_elems + chunk * 8);
    cp_async16(tile_addr<HD>(sbase + kBlock * HD * 2, row, chunk), vb + (int64_t)row * row_elems + chunk * 8);
  }
}

template <int HD, int kDecWarps, int kDecStages>
__global__ void __launch_bounds__(kDecWarps * 32)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ kpool,
                    __nv_bfloat16* __restrict__ vpool, const __nv_bfloat16* __restrict__ new_k,
                    const __nv_bfloat16* __restrict__ new_v, const int* __restrict__ tables,
                    const int* __restrict__ ctx_lens, const int* __restrict__ chunk_offsets,
                    __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                    int* __restrict__ status, int n_seqs, int chunk_tokens, int max_blocks, int n_pool_blocks,
                    int n_heads, int n_kv, float sl2) {
  lg::pdl_prologue();
  extern __shared__ __align__(128) uint8_t smem[];
  const int chunk_id = blockIdx.x, kvh = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int n_rep = n_heads / n_kv;
  constexpr int D = HD, kRowBytes = HD * 2, DT = HD / 8, CH = HD / 8;
  constexpr int kDecStageBytes = DecCfg<HD, kDecWarps, kDecStages>::kStageBytes;
  const int row_elems = n_kv * D;

  // which sequence owns this chunk: largest s with chunk_offsets[s] <= chunk_id
  int lo = 0, hi = n_seqs;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (chunk_offsets[mid] <= chunk_id) lo = mid; else hi = mid;
  }
  const int seq = lo;
  const int chunk_in_seq = chunk_id - chunk_offsets[seq];
  const int n_chunks = chunk_offsets[seq + 1] - chunk_offsets[seq];
  const int ctx = ctx_lens[seq];
  const int tok_begin = chunk_in_seq * chunk_tokens;
  const int tok_end = min(ctx, tok_begin + chunk_tokens);
  const int* table = tables + (int64_t)seq * max_blocks;

  // ---- fused append: the CTA of the last chunk stores the new token's K/V slice first ----
  if (new_k != nullptr && chunk_in_seq == n_chunks - 1 && ctx > 0) {
    const int pos = ctx - 1;
    const int pb = (pos / kBlock) < max_blocks ? table[pos / kBlock] : -1;
    if (pb >= 0 && pb < n_pool_blocks) {
      if (tid < 2 * CH) {
        const int64_t dst = ((int64_t)pb * kBlock + pos % kBlock) * row_elems + kvh * D;
        const int64_t src = (int64_t)seq * row_elems + kvh * D;
        const int chunk = tid % CH;
        if (tid < CH)
          *reinterpret_cast<uint4*>(kpool + dst + chunk * 8) = __ldg(reinterpret_cast<const uint4*>(new_k + src + chunk * 8));
        else
          *reinterpret_cast<uint4*>(vpool + dst + chunk * 8) = __ldg(reinterpret_cast<const uint4*>(new_v + src + chunk * 8));
      }
    } else if (tid == 0 && status) {
      atomicExch(status, 1);
    }
    __threadfence();
  }

  // ---- stage the query rows of this kv head's group (rows >= n_rep are zero) ----
  uint8_t* sq = smem + kDecWarps * kDecStages * kDecStageBytes;
  const uint32_t sq_a = smem_u32(sq);
  for (int u = tid; u < 16 * CH; u += kDecWarps * 32) {
    const int row = u / CH, chunk = u % CH;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < n_rep) v = __ldg(reinterpret_cast<const uint4*>(q + ((int64_t)seq * n_heads + kvh * n_rep + row) * D + chunk * 8));
    *reinterpret_cast<uint4*>(sq + (tile_addr<HD>(sq_a, row, chunk) - sq_a)) = v;
  }
  __syncthreads();
  uint32_t qf[HD / 16][4];
  load_q_frags<HD>(sq_a, lane, qf);

  float o[DT][4];
#pragma unroll
  for (int j = 0; j < DT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[j][i] = 0.0f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

  // ---- per-warp pipeline over this warp's blocks: blk = first + warp, + kDecWarps, ... ----
  const int blk_begin = tok_begin / kBlock, blk_end = (tok_end + kBlock - 1) / kBlock;
  const uint32_t wbase = smem_u32(smem) + warp * kDecStages * kDecStageBytes;
  const int my_first = blk_begin + warp;
  const int my_count = my_first < blk_end ? (blk_end - my_first + kDecWarps - 1) / kDecWarps : 0;

  auto issue = [&](int i) {  // i-th block of this warp; always commits a group (possibly empty)
    if (i < my_count) {
      const int bidx = my_first + i * kDecWarps;
      const int pb = bidx < max_blocks ? table[bidx] : -1;
      if (pb >= 0 && pb < n_pool_blocks) {
        stage_block<HD>(wbase + (i % kDecStages) * kDecStageBytes, kpool, vpool, pb, row_elems, kvh, lane);
      } else if (lane == 0 && status) {
        atomicExch(status, 1);
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int i = 0; i < kDecStages - 1; ++i) issue(i);

  for (int i = 0; i < my_count; ++i) {
    issue(i + kDecStages - 1);
    cp_async_wait<kDecStages - 1>();
    __syncwarp();
    const int blk = my_first + i * kDecWarps;
    const int pb = blk < max_blocks ? table[blk] : -1;
    const bool valid_block = pb >= 0 && pb < n_pool_blocks;
    const uint32_t sb = wbase + (i % kDecStages) * kDecStageBytes;
    float s[2][4];
    if (valid_block) {
      qk_tile<2, HD>(qf, sb, 0, lane, s);
    } else {
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[t][e] = -INFINITY;
    }
    const int tbase = blk * kBlock;
    if (tbase + kBlock > tok_end) {
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int k0 = tbase + 8 * t + 2 * c;
        if (k0 >= tok_end) { s[t][0] = -INFINITY; s[t][2] = -INFINITY; }
        if (k0 + 1 >= tok_end) { s[t][1] = -INFINITY; s[t][3] = -INFINITY; }
      }
    }
    softmax_step<2, DT>(s, m, l, o, sl2);
    if (valid_block) {
      // rows of a partially filled block beyond the context may hold stale data: P is 0 there,
      // but 0 * NaN is NaN, so such rows are cleared before the product
      if (tbase + kBlock > tok_end) {
        for (int u = lane; u < kBlock * CH; u += 32) {
          const int row = u / CH, chunk = u % CH;
          if (tbase + row >= tok_end)
            *reinterpret_cast<uint4*>(smem + (tile_addr<HD>(sb + kBlock * kRowBytes, row, chunk) - smem_u32(smem))) = make_uint4(0u, 0u, 0u, 0u);
        }
        __syncwarp();
      }
      pv_tile<2, HD>(s, sb + kBlock * kRowBytes, 0, lane, o);
    }
    __syncwarp();
  }
  cp_async_wait<0>();

  // ---- merge the four warps' partial (m, l, o) through shared memory ----
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
  __syncthreads();
  float* so = reinterpret_cast<float*>(smem);                 // [warp][16][128]
  float* sml = so + kDecWarps * 16 * D;                       // [warp][16][2]
#pragma unroll
  for (int j = 0; j < DT; ++j) {
    const int d = 8 * j + 2 * c;
    *reinterpret_cast<float2*>(so + ((warp * 16 + g) * D + d)) = make_float2(o[j][0], o[j][1]);
    *reinterpret_cast<float2*>(so + ((warp * 16 + g + 8) * D + d)) = make_float2(o[j][2], o[j][3]);
  }
  if (c == 0) {
    sml[(warp * 16 + g) * 2] = m[0];     sml[(warp * 16 + g) * 2 + 1] = l[0];
    sml[(warp * 16 + g + 8) * 2] = m[1]; sml[(warp * 16 + g + 8) * 2 + 1] = l[1];
  }
  __syncthreads();
  // thread t owns columns d = t, t + 128, ...; loops over the group's query heads
  for (int r = 0; r < n_rep; ++r) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, sml[(w * 16 + r) * 2]);
    float L = 0.0f, f[kDecWarps];
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float mw = sml[(w * 16 + r) * 2];
      f[w] = (mw == -INFINITY) ? 0.0f : exp2f((mw - M) * sl2);
      L += sml[(w * 16 + r) * 2 + 1] * f[w];
    }
    const int head = kvh * n_rep + r;
#pragma unroll
    for (int d = tid; d < D; d += kDecWarps * 32) {
      float acc = 0.0f;
#pragma unroll
      for (int w = 0; w < kDecWarps; ++w) acc += so[(w * 16 + r) * D + d] * f[w];
      if (n_chunks == 1) out[((int64_t)seq * n_heads + head) * D + d] = __float2bfloat16_rn(L > 0.0f ? acc / L : 0.0f);
      else part_o[((int64_t)chunk_id * n_heads + head) * D + d] = acc;
    }
    if (n_chunks != 1 && tid == 0) {
      part_ml[((int64_t)chunk_id * n_heads + head) * 2] = M;
      part_ml[((int64_t)chunk_id * n_heads + head) * 2 + 1] = L;
    }
  }
}

// merges the per-chunk partial results of sequences that were split into several chunks
__global__ void paged_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                          const int* __restrict__ chunk_offsets, __nv_bfloat16* __restrict__ out,
                                          int n_heads, int D, float sl2) {
  lg::pdl_prologue();
  const int seq = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
  const int c0 = chunk_offsets[seq], c1 = chunk_offsets[seq + 1];
  if (c1 - c0 <= 1) return;  // single-chunk sequences were finished by the main kernel
  float M = -INFINITY;
  for (int ck = c0; ck < c1; ++ck) M = fmaxf(M, part_ml[((int64_t)ck * n_heads + head) * 2]);
  float L = 0.0f, acc = 0.0f;
  for (int ck = c0; ck < c1; ++ck) {
    const float mw = part_ml[((int64_t)ck * n_heads + head) * 2];
    const float f = (mw == -INFINITY) ? 0.0f : exp2f((mw - M) * sl2);
    L += part_ml[((int64_t)ck * n_heads + head) * 2 + 1] * f;
    acc += part_o[((int64_t)ck * n_heads + head) * D + d] * f;
  }
  out[((int64_t)seq * n_heads + head) * D + d] = __float2bfloat16_rn(L > 0.0f ? acc / L : 0.0f);
}

// ================================ paged KV store / gather ======================================

__global__ void paged_kv_store_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                      int src_stride, __nv_bfloat16* __restrict__ kpool,
                                      __nv_bfloat16* __restrict__ vpool, const int64_t* __restrict__ slots,
                                      int n_tokens, int row_elems, int64_t n_slots, int* __restrict__ status) {
  lg::pdl_prologue();
  const int chunks = row_elems >> 3;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)n_tokens * chunks) return;
  const int t = (int)(idx / chunks), ch = (int)(idx % chunks);
  const int64_t slot = slots[t];
  if (slot < 0 || slot >= n_slots) {
    if (ch == 0 && status) atomicExch(status, 1);
    return;
  }
  *reinterpret_cast<uint4*>(kpool + slot * row_elems + ch * 8) = __ldg(reinterpret_cast<const uint4*>(k + (int64_t)t * src_stride + ch * 8));
  *reinterpret_cast<uint4*>(vpool + slot * row_elems + ch * 8) = __ldg(reinterpret_cast<const uint4*>(v + (int64_t)t * src_stride + ch * 8));
}

__global__ void paged_kv_gather_kernel(const __nv_bfloat16* __restrict__ kpool, const __nv_bfloat16* __restrict__ vpool,
                                       const int* __restrict__ table, int table_len, int len, int row_elems,
                                       int n_pool_blocks, __nv_bfloat16* __restrict__ kout,
                                       __nv_bfloat16* __restrict__ vout, int* __restrict__ status) {
  lg::pdl_prologue();
  const int chunks = row_elems >> 3;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)len * chunks) return;
  const int t = (int)(idx / chunks), ch = (int)(idx % chunks);
  const int bi = t / kBlock;
  const int pb = bi < table_len ? table[bi] : -1;
  if (pb < 0 || pb >= n_pool_blocks) {
    if (ch == 0 && status) atomicExch(status, 1);
    return;
  }
  const int64_t src = ((int64_t)pb * kBlock + t % kBlock) * row_elems + ch * 8;
  *reinterpret_cast<uint4*>(kout + (int64_t)t * row_elems + ch * 8) = __ldg(reinterpret_cast<const uint4*>(kpool + src));
  *reinterpret_cast<uint4*>(vout + (int64_t)t * row_elems + ch * 8) = __ldg(reinterpret_cast<const uint4*>(vpool + src));
}

}  // namespace

extern "C" {

uint32_t logismos_launch_varlen_attention_bf16(const void* qkv, const void* cu_seqlens, void* out, int32_t n_seqs,
                                               int32_t max_seqlen, int32_t n_heads, int32_t n_kv_heads,
                                               int32_t head_dim, int32_t row_stride, int32_t k_off, int32_t v_off,
                                               int32_t causal, void* stream) {
  lg::LaunchScope launch_scope_;
  if (n_seqs < 0 || max_seqlen < 0 || n_heads <= 0 || n_kv_heads <= 0 || (head_dim != 128 && head_dim != 256) || (n_heads % n_kv_heads) ||
      (row_stride % 8) || (k_off % 8) || (v_off % 8) || ((uintptr_t)qkv & 15) || ((uintptr_t)out & 3))
    return lg::kInvalidValue;
  if (n_seqs == 0 || max_seqlen == 0) return 0;
  const size_t smem = 4 * 16384;
  const float sl2 = kLog2e / sqrtf((float)head_dim);
  dim3 grid((max_seqlen + kQTile - 1) / kQTile, n_heads, n_seqs);
  auto launch = [&](auto kern) -> uint32_t {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (uint32_t)e;
    lg::launch(kern, grid, dim3(kVarlenThreads), smem, (cudaStream_t)stream, (const __nv_bfloat16*)qkv, (const int*)cu_seqlens, (__nv_bfloat16*)out,
                                                             n_heads, n_kv_heads, row_stride, k_off, v_off, sl2);
    return lg::launch_status();
  };
  if (head_dim == 128) return causal ? launch(varlen_attention_kernel<true, 128>) : launch(varlen_attention_kernel<false, 128>);
  return causal ? launch(varlen_attention_kernel<true, 256>) : launch(varlen_attention_kernel<false, 256>);
}

size_t logismos_paged_decode_scratch_bytes(int32_t total_chunks, int32_t n_heads, int32_t head_dim) {
  if (total_chunks <= 0 || n_heads <= 0 || head_dim <= 0) return 0;
  return (size_t)total_chunks * n_heads * (head_dim + 2) * sizeof(float);
}

uint32_t logismos_launch_paged_attention_decode_bf16(
    const void* q, void* k_pool, void* v_pool, const void* new_k, const void* new_v, const void* block_tables,
    const void* context_lens, const void* chunk_offsets, void* out, void* scratch, void* status, int32_t n_seqs,
    int32_t total_chunks, int32_t chunk_tokens, int32_t max_blocks, int32_t n_pool_blocks, int32_t n_heads,
    int32_t n_kv_heads, int32_t head_dim, void* stream) {
  lg::LaunchScope launch_scope_;
  if (n_seqs < 0 || total_chunks < 0 || chunk_tokens <= 0 || (chunk_tokens % 64) || max_blocks <= 0 ||
      n_pool_blocks <= 0 || n_heads <= 0 || n_kv_heads <= 0 || (head_dim != 128 && head_dim != 256) || (n_heads % n_kv_heads) ||
      n_heads / n_kv_heads > 16 || (new_k == nullptr) != (new_v == nullptr))
    return lg::kInvalidValue;
  if (n_seqs == 0 || total_chunks == 0) return 0;
  if (scratch == nullptr || ((uintptr_t)scratch & 15)) return lg::kInvalidValue;
  float* part_o = (float*)scratch;
  float* part_ml = part_o + (size_t)total_chunks * n_heads * head_dim;
  const float sl2 = kLog2e / sqrtf((float)head_dim);
  dim3 grid(total_chunks, n_kv_heads);
  auto launch = [&](auto kern, int warps, int smem) -> uint32_t {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (uint32_t)e;
    lg::launch(kern, grid, dim3(warps * 32), smem, (cudaStream_t)stream, 
        (const __nv_bfloat16*)q, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, (const __nv_bfloat16*)new_k,
        (const __nv_bfloat16*)new_v, (const int*)block_tables, (const int*)context_lens, (const int*)chunk_offsets,
        (__nv_bfloat16*)out, part_o, part_ml, (int*)status, n_seqs, chunk_tokens, max_blocks, n_pool_blocks, n_heads,
        n_kv_heads, sl2);
    return lg::launch_status();
  };
  uint32_t rc;
  if (head_dim == 128)
    // 4 warps x 2 stages = 68 KB: three CTAs per SM (256 sequences log-uniform in [128, 32768]: 234 us against
    // 242 us with 3 stages and two CTAs; 64 sequences in [256, 8192]: 36 against 43 us)
    rc = launch(paged_decode_kernel<128, 4, 2>, 4, DecCfg<128, 4, 2>::kSmem);
  else if ((int64_t)total_chunks * n_kv_heads >= 2 * lg_sm_count_cached())
    // head_dim 256, many CTAs: 3 warps x 2 stages = 104 KB so that two CTAs share an SM (256 sequences of
    // 1-2 K tokens: 152 us against 182 us with one CTA of 4 warps x 3 stages)
    rc = launch(paged_decode_kernel<256, 3, 2>, 3, DecCfg<256, 3, 2>::kSmem);
  else  // few CTAs: one CTA of 6 warps x 2 stages per SM (64 such sequences: 49 against 56 us)
    rc = launch(paged_decode_kernel<256, 6, 2>, 6, DecCfg<256, 6, 2>::kSmem);
  if (rc) return rc;
  if (total_chunks > n_seqs) {  // at least one sequence spans several chunks
    dim3 mgrid(n_seqs, n_heads);
    lg::launch(paged_decode_merge_kernel, mgrid, dim3(head_dim), 0, (cudaStream_t)stream, part_o, part_ml, (const int*)chunk_offsets,
                                                                           (__nv_bfloat16*)out, n_heads, head_dim, sl2);
    rc = lg::launch_status();
  }
  return rc;
}

uint32_t logismos_launch_paged_kv_store_bf16(const void* k, const void* v, int32_t src_row_stride, void* k_pool,
                                             void* v_pool, const void* slot_mapping, int32_t n_tokens,
                                             int32_t row_elems, int64_t n_pool_slots, void* status, void* stream) {
  lg::LaunchScope launch_scope_;
  if (n_tokens < 0 || row_elems <= 0 || (row_elems % 8) || (src_row_stride % 8) || src_row_stride < row_elems)
    return lg::kInvalidValue;
  if (n_tokens == 0) return 0;
  const int64_t total = (int64_t)n_tokens * (row_elems / 8);
  lg::launch(paged_kv_store_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, 
      (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, src_row_stride, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool,
      (const int64_t*)slot_mapping, n_tokens, row_elems, n_pool_slots, (int*)status);
  return lg::launch_status();
}

uint32_t logismos_launch_paged_kv_gather_bf16(const void* k_pool, const void* v_pool, const void* block_table,
                                              int32_t table_len, int32_t len, int32_t row_elems,
                                              int32_t n_pool_blocks, void* k_out, void* v_out, void* status,
                                              void* stream) {
  lg::LaunchScope launch_scope_;
  if (table_len < 0 || len < 0 || row_elems <= 0 || (row_elems % 8)) return lg::kInvalidValue;
  if (len == 0) return 0;
  const int64_t total = (int64_t)len * (row_elems / 8);
  lg::launch(paged_kv_gather_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, 
      (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, (const int*)block_table, table_len, len, row_elems,
      n_pool_blocks, (__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out, (int*)status);
  return lg::launch_status();
}

}  // extern "C"

// ================================ paged decode without caller scratch ==========================
//
// Some hosts of this library may not allocate device memory at the point where they decode: an
// engine that has already handed every free byte of HBM to its KV pool and weight buffers, or a
// decode thread in which the implicit device-wide synchronisation of an allocation call is not
// acceptable. For them the per-chunk partial results live in a fixed buffer inside the library
// image instead of a caller-provided scratch buffer. Every GPU that loads the library holds these
// LOGISMOS_PAGED_DECODE_STATIC_SCRATCH_BYTES until the process exits.
namespace {

static __device__ __align__(256) unsigned char g_paged_decode_static_scratch[LOGISMOS_PAGED_DECODE_STATIC_SCRATCH_BYTES];

constexpr int kMaxStaticDevices = 64;
std::mutex g_static_scratch_mutex;
void* g_static_scratch_ptr[kMaxStaticDevices] = {nullptr};

// The array's name is a host-side handle, not a device address: the address on the CURRENT device
// is looked up once per device and cached. Returns cudaSuccess and the pointer, or the error.
cudaError_t static_scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxStaticDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_paged_decode_static_scratch);
    if (e != cudaSuccess) return e;
    g_static_scratch_ptr[dev] = p;
  }
  *out = g_static_scratch_ptr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" uint32_t logismos_launch_paged_attention_decode_noalloc_bf16(
    const void* q, void* k_pool, void* v_pool, const void* new_k, const void* new_v, const void* block_tables,
    const void* context_lens, const void* chunk_offsets, void* out, void* status, int32_t n_seqs,
    int32_t total_chunks, int32_t chunk_tokens, int32_t max_blocks, int32_t n_pool_blocks, int32_t n_heads,
    int32_t n_kv_heads, int32_t head_dim, void* stream) {
  lg::LaunchScope launch_scope_;
  if (total_chunks < 0 || n_heads <= 0 || head_dim <= 0) return lg::kInvalidValue;
  const size_t need = logismos_paged_decode_scratch_bytes(total_chunks, n_heads, head_dim);
  if (need > (size_t)LOGISMOS_PAGED_DECODE_STATIC_SCRATCH_BYTES) {
    std::fprintf(stderr,
                 "logismos_launch_paged_attention_decode_noalloc_bf16: %d chunks x %d heads need %zu bytes of "
                 "scratch, the built-in buffer holds %zu; use more tokens per chunk, fewer sequences per call, or "
                 "the entry point that takes caller scratch\n",
                 total_chunks, n_heads, need, (size_t)LOGISMOS_PAGED_DECODE_STATIC_SCRATCH_BYTES);
    return (uint32_t)cudaErrorMemoryAllocation;
  }
  void* scratch = nullptr;
  cudaError_t e = static_scratch_for_current_device(&scratch);
  if (e != cudaSuccess) return (uint32_t)e;
  // Nothing in the buffer has to start at zero: every partial a launch reads, the same launch wrote.
  return logismos_launch_paged_attention_decode_bf16(q, k_pool, v_pool, new_k, new_v, block_tables, context_lens,
                                                     chunk_offsets, out, scratch, status, n_seqs, total_chunks,
                                                     chunk_tokens, max_blocks, n_pool_blocks, n_heads, n_kv_heads,
                                                     head_dim, stream);
}
