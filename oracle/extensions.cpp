// CPU oracle, part 3: gated delta rule, TurboQuant nibble packing, int4 group-32
// weights, flat and paged KV caches, decode attention, ragged packing indices,
// greedy argmax and the fp16 op references. Test infrastructure only; see oracle.h.
#include "oracle.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

namespace {

inline float f16_to_f32(uint16_t h) {
  _Float16 v;
  std::memcpy(&v, &h, 2);
  return (float)v;
}
inline uint16_t f32_to_f16(float f) {  // round to nearest even, as the `half` crate does
  _Float16 v = (_Float16)f;
  uint16_t h;
  std::memcpy(&h, &v, 2);
  return h;
}
inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_bf16(float f) {  // round to nearest even; NaN stays quiet NaN
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

}  // namespace

extern "C" {

void orc_f32_to_bf16(const float* x, size_t n, uint16_t* y) { for (size_t i = 0; i < n; ++i) y[i] = f32_to_bf16(x[i]); }
void orc_bf16_to_f32(const uint16_t* x, size_t n, float* y) { for (size_t i = 0; i < n; ++i) y[i] = bf16_to_f32(x[i]); }
void orc_f32_to_f16(const float* x, size_t n, uint16_t* y) { for (size_t i = 0; i < n; ++i) y[i] = f32_to_f16(x[i]); }
void orc_f16_to_f32(const uint16_t* x, size_t n, float* y) { for (size_t i = 0; i < n; ++i) y[i] = f16_to_f32(x[i]); }

/* ===== crates/kernels/src/gated_delta_rule/cpu.rs ========================== */

// cpu.rs:19-34: rows of length k scaled to unit L2 norm, norm clamped at 1e-12
void orc_l2_norm_rows(float* x, size_t len, size_t k) {
  size_t rows = len / k;
  for (size_t r = 0; r < rows; ++r) {
    float* row = x + r * k;
    float sq = 0.0f;
    for (size_t i = 0; i < k; ++i) sq += row[i] * row[i];
    float inv = 1.0f / std::max(std::sqrt(sq), 1e-12f);
    for (size_t i = 0; i < k; ++i) row[i] *= inv;
  }
}

// cpu.rs:46-54
void orc_cumsum(const float* g, size_t n, float* out) {
  float acc = 0.0f;
  for (size_t i = 0; i < n; ++i) { acc += g[i]; out[i] = acc; }
}

// cpu.rs:92-182. State h is [K,V] row-major. Per token: decay, h^T k, delta, rank-1 update,
// output o[v] = sum_k h[k,v] * q[k] * scale (product order as in the reference: (h*q)*scale).
void orc_gdn_recurrent_fwd(const float* q, const float* k, const float* v, const float* beta,
                           const float* g, size_t t, float scale, const float* state_in,
                           size_t k_dim, size_t v_dim, float* o, float* state_out) {
  std::vector<float> h(state_in, state_in + k_dim * v_dim), htk(v_dim), vd(v_dim);
  for (size_t ti = 0; ti < t; ++ti) {
    const float* qt = q + ti * k_dim;
    const float* kt = k + ti * k_dim;
    const float* vt = v + ti * v_dim;
    float decay = std::exp(g[ti]);
    for (float& hv : h) hv *= decay;
    std::fill(htk.begin(), htk.end(), 0.0f);
    for (size_t ki = 0; ki < k_dim; ++ki)
      for (size_t vi = 0; vi < v_dim; ++vi) htk[vi] += h[ki * v_dim + vi] * kt[ki];
    for (size_t vi = 0; vi < v_dim; ++vi) vd[vi] = beta[ti] * (vt[vi] - htk[vi]);
    for (size_t ki = 0; ki < k_dim; ++ki)
      for (size_t vi = 0; vi < v_dim; ++vi) h[ki * v_dim + vi] += kt[ki] * vd[vi];
    for (size_t vi = 0; vi < v_dim; ++vi) {
      float acc = 0.0f;
      for (size_t ki = 0; ki < k_dim; ++ki) acc += h[ki * v_dim + vi] * qt[ki] * scale;
      o[ti * v_dim + vi] = acc;
    }
  }
  std::memcpy(state_out, h.data(), k_dim * v_dim * sizeof(float));
}

// cpu.rs:201-249: the recurrence applied chunk by chunk with the state carried;
// chunk_states is [ceil(t/bt), K, V].
void orc_gdn_chunk_fwd(const float* q, const float* k, const float* v, const float* beta,
                       const float* g, size_t t, float scale, const float* state_in, size_t k_dim,
                       size_t v_dim, size_t bt, float* o, float* chunk_states) {
  size_t n_chunks = (t + bt - 1) / bt;
  std::vector<float> state(state_in, state_in + k_dim * v_dim), next(k_dim * v_dim);
  for (size_t c = 0; c < n_chunks; ++c) {
    size_t t0 = c * bt, t1 = std::min(t0 + bt, t);
    orc_gdn_recurrent_fwd(q + t0 * k_dim, k + t0 * k_dim, v + t0 * v_dim, beta + t0, g + t0,
                          t1 - t0, scale, state.data(), k_dim, v_dim, o + t0 * v_dim, next.data());
    std::memcpy(chunk_states + c * k_dim * v_dim, next.data(), k_dim * v_dim * sizeof(float));
    state = next;
  }
}

// [NEW] research/14-gdn-aiter-preflight.md:190-198, :209-219: per head h and token t,
// g = -exp(A_log[h]) * softplus(a[t,h] + dt_bias[h]) with softplus(x) = x for x > 20,
// beta = sigmoid(b[t,h]); all fp32.
void orc_gdn_gates(const float* a, const float* b, const float* A_log, const float* dt_bias,
                   size_t t, size_t heads, float* g, float* beta) {
  for (size_t ti = 0; ti < t; ++ti)
    for (size_t h = 0; h < heads; ++h) {
      float x = a[ti * heads + h] + dt_bias[h];
      float sp = x > 20.0f ? x : std::log1p(std::exp(x));
      g[ti * heads + h] = -std::exp(A_log[h]) * sp;
      beta[ti * heads + h] = 1.0f / (1.0f + std::exp(-b[ti * heads + h]));
    }
}

/* ===== crates/quant/src/lib.rs ============================================ */

// lib.rs:272-285: index p occupies bits [4p, 4p+4) of a little-endian 128-bit word,
// i.e. byte j = idx[2j] | idx[2j+1] << 4. An index > 15 is IndexOutOfRange (returns 1).
int orc_pack_turbo4(const uint8_t idx[32], uint8_t out[16]) {
  for (int p = 0; p < 32; ++p) if (idx[p] > 15) return 1;
  for (int j = 0; j < 16; ++j) out[j] = (uint8_t)(idx[2 * j] | (idx[2 * j + 1] << 4));
  return 0;
}
// lib.rs:289-301
void orc_unpack_turbo4(const uint8_t packed[16], uint8_t idx[32]) {
  for (int j = 0; j < 16; ++j) { idx[2 * j] = packed[j] & 0x0f; idx[2 * j + 1] = packed[j] >> 4; }
}
// lib.rs:224-246: index p occupies bits [3p, 3p+3) of a little-endian bitstream of 96 bits
int orc_pack_turbo3(const uint8_t idx[32], uint8_t out[12]) {
  for (int p = 0; p < 32; ++p) if (idx[p] > 7) return 1;
  std::memset(out, 0, 12);
  for (int p = 0; p < 32; ++p)
    for (int b = 0; b < 3; ++b)
      if (idx[p] & (1 << b)) { int bit = 3 * p + b; out[bit >> 3] |= (uint8_t)(1u << (bit & 7)); }
  return 0;
}
// lib.rs:250-268
void orc_unpack_turbo3(const uint8_t packed[12], uint8_t idx[32]) {
  for (int p = 0; p < 32; ++p) {
    uint8_t v = 0;
    for (int b = 0; b < 3; ++b) { int bit = 3 * p + b; if (packed[bit >> 3] & (1u << (bit & 7))) v |= (uint8_t)(1u << b); }
    idx[p] = v;
  }
}

/* ---- TurboQuant 3-bit head codec (crates/quant/src/lib.rs:73-114, :316-413) ---------------------
 * One 128-value head chunk -> four 14-byte blocks (2-byte little-endian fp16 norm, repeated in every
 * block, + 12 bytes of 3-bit codebook indices): L2 norm (sequential fp32 sum of squares), v / norm,
 * normalised Walsh-Hadamard transform over 128 points, nearest of 8 Lloyd-Max centroids (first minimum
 * wins), indices packed as above. Decoding looks the centroids up, applies the same transform (it is
 * its own inverse) and multiplies by the stored norm. */
static const float kTurbo3Codebook[8] = {-0.1883972972f, -0.1181399059f, -0.0665857641f, -0.0216044751f,
                                         0.0216041461f,  0.0665854520f,  0.1181396281f,  0.1883970748f};  // lib.rs:73-82

// lib.rs:90-114: butterflies with h = 1, 2, ..., 64 (lo' = lo + hi, hi' = lo - hi), then * 1/sqrt(128)
void orc_fwht_128(float* d) {
  for (int h = 1; h < 128; h *= 2)
    for (int base = 0; base < 128; base += 2 * h)
      for (int i = 0; i < h; ++i) {
        const float x = d[base + i], y = d[base + h + i];
        d[base + i] = x + y;
        d[base + h + i] = x - y;
      }
  const float scale = 0.08838834764831844f;
  for (int i = 0; i < 128; ++i) d[i] *= scale;
}

// lib.rs:316-360; out = 4 blocks x 14 bytes
void orc_turbo3_encode_head(const float* values, uint8_t* out) {
  float sum_sq = 0.0f;
  for (int i = 0; i < 128; ++i) sum_sq += values[i] * values[i];
  const float norm = std::sqrt(sum_sq);
  const uint16_t nb = f32_to_f16(norm);
  float t[128];
  for (int i = 0; i < 128; ++i) t[i] = norm > 1e-12f ? values[i] / norm : 0.0f;
  orc_fwht_128(t);
  for (int bi = 0; bi < 4; ++bi) {
    uint8_t idx[32];
    for (int i = 0; i < 32; ++i) {
      const float v = t[bi * 32 + i];
      int best = 0;
      float bd = std::fabs(v - kTurbo3Codebook[0]);
      for (int c = 1; c < 8; ++c) {
        const float dd = std::fabs(v - kTurbo3Codebook[c]);
        if (dd < bd) { bd = dd; best = c; }
      }
      idx[i] = (uint8_t)best;
    }
    uint8_t* blk = out + bi * 14;
    blk[0] = (uint8_t)(nb & 0xff);
    blk[1] = (uint8_t)(nb >> 8);
    orc_pack_turbo3(idx, blk + 2);
  }
}

// lib.rs:378-413
void orc_turbo3_decode_head(const uint8_t* in, float* out) {
  for (int bi = 0; bi < 4; ++bi) {
    uint8_t idx[32];
    orc_unpack_turbo3(in + bi * 14 + 2, idx);
    for (int i = 0; i < 32; ++i) out[bi * 32 + i] = kTurbo3Codebook[idx[i]];
  }
  orc_fwht_128(out);
  const float norm = f16_to_f32((uint16_t)(in[0] | (in[1] << 8)));
  for (int i = 0; i < 128; ++i) out[i] *= norm;
}

/* ===== [NEW] int4 group-32 weights ========================================
 * Layout anchored on Turbo4Block's nibble order (lib.rs:272-301): weight row n, column k
 * lives in byte packed[n*k_dim/2 + k/2], low nibble for even k, high nibble for odd k, as a
 * two's-complement 4-bit integer in [-8, 7]; one fp16 scale per 32 consecutive k.       */

int orc_int4_pack(const int8_t* codes, size_t n, size_t k, uint8_t* packed) {
  for (size_t i = 0; i < n * k; ++i) if (codes[i] < -8 || codes[i] > 7) return 1;
  for (size_t i = 0; i < n * k / 2; ++i)
    packed[i] = (uint8_t)((codes[2 * i] & 0x0f) | ((codes[2 * i + 1] & 0x0f) << 4));
  return 0;
}
void orc_int4_unpack(const uint8_t* packed, size_t n, size_t k, int8_t* codes) {
  for (size_t i = 0; i < n * k / 2; ++i) {
    int lo = packed[i] & 0x0f, hi = packed[i] >> 4;
    codes[2 * i] = (int8_t)(lo >= 8 ? lo - 16 : lo);
    codes[2 * i + 1] = (int8_t)(hi >= 8 ? hi - 16 : hi);
  }
}
void orc_int4_quantize(const float* w, size_t n, size_t k, uint8_t* packed, uint16_t* scales_f16) {
  size_t groups = k / 32;
  std::vector<int8_t> codes(n * k);
  for (size_t r = 0; r < n; ++r)
    for (size_t gi = 0; gi < groups; ++gi) {
      const float* src = w + r * k + gi * 32;
      float amax = 0.0f;
      for (int j = 0; j < 32; ++j) amax = std::max(amax, std::fabs(src[j]));
      uint16_t sh = f32_to_f16(amax / 7.0f);
      float s = f16_to_f32(sh);
      scales_f16[r * groups + gi] = sh;
      for (int j = 0; j < 32; ++j) {
        float qv = s > 0.0f ? std::nearbyint(src[j] / s) : 0.0f;
        codes[r * k + gi * 32 + j] = (int8_t)std::min(7.0f, std::max(-8.0f, qv));
      }
    }
  orc_int4_pack(codes.data(), n, k, packed);
}
void orc_int4_dequant(const uint8_t* packed, const uint16_t* scales_f16, size_t n, size_t k, float* w) {
  size_t groups = k / 32;
  std::vector<int8_t> codes(n * k);
  orc_int4_unpack(packed, n, k, codes.data());
  for (size_t r = 0; r < n; ++r)
    for (size_t c = 0; c < k; ++c)
      w[r * k + c] = f16_to_f32(scales_f16[r * groups + c / 32]) * (float)codes[r * k + c];
}
// Group-wise: the integer-times-activation partial sum of each group is formed first (fp32,
// ascending k), then scaled, then added to the row accumulator in ascending group order.
void orc_int4_gemv(const uint8_t* packed, const uint16_t* scales_f16, size_t n, size_t k,
                   const float* x, size_t batch, float* y) {
  size_t groups = k / 32;
  std::vector<int8_t> codes(k);
  for (size_t r = 0; r < n; ++r) {
    orc_int4_unpack(packed + r * k / 2, 1, k, codes.data());
    for (size_t b = 0; b < batch; ++b) {
      const float* xb = x + b * k;
      float acc = 0.0f;
      for (size_t gi = 0; gi < groups; ++gi) {
        float part = 0.0f;
        for (int j = 0; j < 32; ++j) part += (float)codes[gi * 32 + j] * xb[gi * 32 + j];
        acc += f16_to_f32(scales_f16[r * groups + gi]) * part;
      }
      y[b * n + r] = acc;
    }
  }
}

/* ===== crates/cache/src/flat.rs =========================================== */
}  // extern "C"

namespace {
struct FlatKv {
  size_t num_layers, row_bytes, max_seq_len;
  std::vector<std::vector<uint8_t>> k, v;
  std::vector<size_t> lens;
};
}  // namespace

extern "C" {

// flat.rs:84-110: one zeroed [max_seq_len, row_bytes] buffer per layer for K and for V
void* orc_flatkv_create(size_t num_layers, size_t row_bytes, size_t max_seq_len) {
  FlatKv* c = new FlatKv{num_layers, row_bytes, max_seq_len, {}, {}, {}};
  c->k.assign(num_layers, std::vector<uint8_t>(row_bytes * max_seq_len, 0));
  c->v.assign(num_layers, std::vector<uint8_t>(row_bytes * max_seq_len, 0));
  c->lens.assign(num_layers, 0);
  return c;
}
void orc_flatkv_destroy(void* c) { delete static_cast<FlatKv*>(c); }
// flat.rs:180-252: rows appended at lens[layer]; overflow of max_seq_len is LenOverflow
int orc_flatkv_put(void* cp, size_t layer, const uint8_t* k, const uint8_t* v, size_t n_tokens) {
  FlatKv* c = static_cast<FlatKv*>(cp);
  if (layer >= c->num_layers) return 1;
  size_t cur = c->lens[layer];
  if (cur + n_tokens > c->max_seq_len) return 2;
  std::memcpy(c->k[layer].data() + cur * c->row_bytes, k, n_tokens * c->row_bytes);
  std::memcpy(c->v[layer].data() + cur * c->row_bytes, v, n_tokens * c->row_bytes);
  c->lens[layer] = cur + n_tokens;
  return 0;
}
// flat.rs:254-304: the first `len` rows; len beyond what was written is ReadBeyondWritten
int orc_flatkv_get(void* cp, size_t layer, size_t len, uint8_t* k_out, uint8_t* v_out) {
  FlatKv* c = static_cast<FlatKv*>(cp);
  if (layer >= c->num_layers) return 1;
  if (len > c->lens[layer]) return 3;
  std::memcpy(k_out, c->k[layer].data(), len * c->row_bytes);
  std::memcpy(v_out, c->v[layer].data(), len * c->row_bytes);
  return 0;
}
long orc_flatkv_len_of(void* cp, size_t layer) {
  FlatKv* c = static_cast<FlatKv*>(cp);
  return layer < c->num_layers ? (long)c->lens[layer] : -1;
}
void orc_flatkv_reset(void* cp) {
  FlatKv* c = static_cast<FlatKv*>(cp);
  std::fill(c->lens.begin(), c->lens.end(), 0);
}

/* ===== [NEW] paged KV cache =============================================== */

// Writes one token row at logical position pos. 1: table too short, 2: bad block id.
int orc_paged_append(uint8_t* k_pool, uint8_t* v_pool, size_t n_blocks, size_t block_size,
                     size_t row_bytes, const int32_t* table, size_t table_len, size_t pos,
                     const uint8_t* k_row, const uint8_t* v_row) {
  size_t bi = pos / block_size, off = pos % block_size;
  if (bi >= table_len) return 1;
  if (table[bi] < 0 || (size_t)table[bi] >= n_blocks) return 2;
  size_t dst = ((size_t)table[bi] * block_size + off) * row_bytes;
  std::memcpy(k_pool + dst, k_row, row_bytes);
  std::memcpy(v_pool + dst, v_row, row_bytes);
  return 0;
}
// The first `len` logical rows, in order: must equal FlatKvCache::get for the same puts.
int orc_paged_gather(const uint8_t* k_pool, const uint8_t* v_pool, size_t n_blocks,
                     size_t block_size, size_t row_bytes, const int32_t* table, size_t table_len,
                     size_t len, uint8_t* k_out, uint8_t* v_out) {
  for (size_t t = 0; t < len; ++t) {
    size_t bi = t / block_size, off = t % block_size;
    if (bi >= table_len) return 1;
    if (table[bi] < 0 || (size_t)table[bi] >= n_blocks) return 2;
    size_t src = ((size_t)table[bi] * block_size + off) * row_bytes;
    std::memcpy(k_out + t * row_bytes, k_pool + src, row_bytes);
    std::memcpy(v_out + t * row_bytes, v_pool + src, row_bytes);
  }
  return 0;
}

// One query token attending to `len` cached rows: the last row of the causal variant of
// attention.rs:226-296 (scores = q.k then * 1/sqrt(d); max-subtracted softmax; P.V), with the
// GQA mapping q head j -> kv head j / (n_heads / n_kv) of attention.rs:366-382.
void orc_decode_attention(const float* q, const float* k, const float* v, size_t len,
                          size_t n_heads, size_t n_kv, size_t d, float* out) {
  size_t groups = n_heads / n_kv, row = n_kv * d;
  float scale = 1.0f / std::sqrt((float)d);
  std::vector<float> s(len), p(len);
  for (size_t h = 0; h < n_heads; ++h) {
    size_t kvh = h / groups;
    for (size_t t = 0; t < len; ++t) {
      float acc = 0.0f;
      for (size_t i = 0; i < d; ++i) acc += q[h * d + i] * k[t * row + kvh * d + i];
      s[t] = acc * scale;
    }
    orc_softmax_last_dim(s.data(), 1, len, p.data());
    for (size_t i = 0; i < d; ++i) {
      float acc = 0.0f;
      for (size_t t = 0; t < len; ++t) acc += p[t] * v[t * row + kvh * d + i];
      out[h * d + i] = acc;
    }
  }
}

/* ===== [NEW] ragged packing =============================================== */

long orc_build_packing(const int32_t* cached_lens, const int32_t* new_lens, size_t n_seq,
                       const int32_t* tables, size_t max_blocks, size_t block_size,
                       size_t n_pool_blocks, int32_t* cu_seqlens, int32_t* positions,
                       int64_t* slot_mapping, int32_t* seq_ids) {
  long total = 0;
  cu_seqlens[0] = 0;
  for (size_t i = 0; i < n_seq; ++i) {
    for (int32_t j = 0; j < new_lens[i]; ++j) {
      size_t pos = (size_t)cached_lens[i] + (size_t)j;
      size_t bi = pos / block_size;
      if (bi >= max_blocks) return -1;
      int32_t blk = tables[i * max_blocks + bi];
      if (blk < 0 || (size_t)blk >= n_pool_blocks) return -1;
      positions[total] = (int32_t)pos;
      slot_mapping[total] = (int64_t)blk * (int64_t)block_size + (int64_t)(pos % block_size);
      seq_ids[total] = (int32_t)i;
      ++total;
    }
    cu_seqlens[i + 1] = (int32_t)total;
  }
  return total;
}

/* ===== crates/decode/src/lib.rs:73-83 ===================================== */

// First maximum wins; NaN is never selected (strict > starting from -inf).
uint32_t orc_greedy(const float* logits, size_t n) {
  size_t best_i = 0;
  float best = -INFINITY;
  for (size_t i = 0; i < n; ++i)
    if (logits[i] > best) { best = logits[i]; best_i = i; }
  return best_i > 0xffffffffull ? 0xffffffffu : (uint32_t)best_i;
}

/* ===== fp16 op references ================================================= */

// crates/kernels/src/matmul/cpu.rs: D[M,N] = A[M,K] B[K,N], fp32 accumulate in ascending k
void orc_matmul_fp16_ref(const uint16_t* a, const uint16_t* b, size_t m, size_t n, size_t k, uint16_t* d) {
  for (size_t i = 0; i < m; ++i)
    for (size_t j = 0; j < n; ++j) {
      float acc = 0.0f;
      for (size_t kk = 0; kk < k; ++kk) acc += f16_to_f32(a[i * k + kk]) * f16_to_f32(b[kk * n + j]);
      d[i * n + j] = f32_to_f16(acc);
    }
}
// crates/kernels/src/rms_norm/cpu.rs
void orc_rms_norm_fp16_ref(const uint16_t* x, const uint16_t* w, size_t m, size_t n, float eps, uint16_t* y) {
  for (size_t r = 0; r < m; ++r) {
    float sum_sq = 0.0f;
    for (size_t j = 0; j < n; ++j) { float f = f16_to_f32(x[r * n + j]); sum_sq += f * f; }
    float inv = 1.0f / std::sqrt(sum_sq / (float)n + eps);
    for (size_t j = 0; j < n; ++j)
      y[r * n + j] = f32_to_f16(f16_to_f32(x[r * n + j]) * inv * f16_to_f32(w[j]));
  }
}
// crates/kernels/src/softmax/cpu.rs: a length mismatch is UnsupportedShape (returns 1);
// an all -inf row becomes uniform
int orc_softmax_fp16_ref(const uint16_t* x, size_t x_len, size_t m, size_t n, uint16_t* y) {
  if (x_len != m * n) return 1;
  std::vector<float> e(n);
  for (size_t r = 0; r < m; ++r) {
    float mx = -INFINITY;
    for (size_t j = 0; j < n; ++j) { float f = f16_to_f32(x[r * n + j]); if (f > mx) mx = f; }
    if (std::isinf(mx) && mx < 0) {
      float u = n == 0 ? 0.0f : 1.0f / (float)n;
      for (size_t j = 0; j < n; ++j) y[r * n + j] = f32_to_f16(u);
      continue;
    }
    float denom = 0.0f;
    for (size_t j = 0; j < n; ++j) { e[j] = std::exp(f16_to_f32(x[r * n + j]) - mx); denom += e[j]; }
    float inv = 1.0f / denom;
    for (size_t j = 0; j < n; ++j) y[r * n + j] = f32_to_f16(e[j] * inv);
  }
  return 0;
}
// crates/kernels/src/rope/cpu.rs:19-39: interleaved (cos, sin) pairs, all in f32 with powf
void orc_build_cos_sin_table(size_t seq, size_t head_dim, float theta, float* table) {
  size_t pairs = head_dim / 2;
  for (size_t pos = 0; pos < seq; ++pos)
    for (size_t i = 0; i < pairs; ++i) {
      float e = -(2.0f * (float)i) / (float)head_dim;
      float freq = std::pow(theta, e);
      float angle = (float)pos * freq;
      table[pos * head_dim + 2 * i] = std::cos(angle);
      table[pos * head_dim + 2 * i + 1] = std::sin(angle);
    }
}
// crates/kernels/src/rope/cpu.rs:41-110: interleaved-pair rotation on (B,S,H,D) fp16
int orc_rope_apply_fp16_ref(uint16_t* qk, size_t qk_len, const float* cos_sin, size_t cs_len,
                            size_t batch, size_t seq, size_t heads, size_t head_dim) {
  if (qk_len != batch * seq * heads * head_dim) return 1;
  if (cs_len != seq * head_dim) return 2;
  size_t pairs = head_dim / 2;
  for (size_t b = 0; b < batch; ++b)
    for (size_t s = 0; s < seq; ++s)
      for (size_t h = 0; h < heads; ++h) {
        size_t base = ((b * seq + s) * heads + h) * head_dim;
        for (size_t i = 0; i < pairs; ++i) {
          float c = cos_sin[s * head_dim + 2 * i], sn = cos_sin[s * head_dim + 2 * i + 1];
          float x0 = f16_to_f32(qk[base + 2 * i]), x1 = f16_to_f32(qk[base + 2 * i + 1]);
          qk[base + 2 * i] = f32_to_f16(x0 * c - x1 * sn);
          qk[base + 2 * i + 1] = f32_to_f16(x0 * sn + x1 * c);
        }
      }
  return 0;
}

}  // extern "C"
