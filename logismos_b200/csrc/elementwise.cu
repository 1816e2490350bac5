// Memory-bound pieces of the encoder/decoder layer: embedding gather, RMSNorm over the fp32
// residual stream, halves-RoPE on packed q/k, SwiGLU, pooled embedding head, greedy argmax.
// Each restates one function of crates/kernels/src/cpu_f32/mod.rs (cited per kernel) with
// 128-bit coalesced accesses and warp-shuffle reductions.
#include "common.cuh"
#include "logismos_kernels.h"

namespace {

using namespace lg;

// cpu_f32::embed_lookup (mod.rs:106-127). One warp per token row; 8 bf16 per lane per step.
__global__ void embed_lookup_kernel(const __nv_bfloat16* __restrict__ table,
                                    const uint32_t* __restrict__ ids, float* __restrict__ out,
                                    int n_ids, int hidden, int vocab) {
  lg::pdl_prologue();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_ids) return;
  const int lane = threadIdx.x & 31;
  const uint32_t id = ids[row];
  float* dst = out + (size_t)row * hidden;
  if (id >= (uint32_t)vocab) {  // out-of-range id: zero row, not an error (mod.rs:96-104)
    for (int j = lane * 4; j < hidden; j += 128) *reinterpret_cast<float4*>(dst + j) = make_float4(0, 0, 0, 0);
    return;
  }
  const __nv_bfloat16* src = table + (size_t)id * hidden;
  for (int j = lane * 8; j < hidden; j += 256) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + j));
    const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
    *reinterpret_cast<float4*>(dst + j) = make_float4(a.x, a.y, b.x, b.y);
    *reinterpret_cast<float4*>(dst + j + 4) = make_float4(c.x, c.y, d.x, d.y);
  }
}

// cpu_f32::rms_norm (mod.rs:137-159). One CTA per row, the row held in registers between the
// two passes (n <= 8 * 4 * blockDim).
template <bool OUT_F32>
__global__ void rms_norm_f32_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                    void* __restrict__ y, int n, float eps) {
  lg::pdl_prologue();
  __shared__ float red[32];
  const float* row = x + (size_t)blockIdx.x * n;
  float4 v[8];
  float ss = 0.0f;
  int cnt = 0;
  for (int j = threadIdx.x * 4; j < n && cnt < 8; j += blockDim.x * 4, ++cnt) {
    v[cnt] = *reinterpret_cast<const float4*>(row + j);
    ss += v[cnt].x * v[cnt].x + v[cnt].y * v[cnt].y + v[cnt].z * v[cnt].z + v[cnt].w * v[cnt].w;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  cnt = 0;
  for (int j = threadIdx.x * 4; j < n && cnt < 8; j += blockDim.x * 4, ++cnt) {
    const float4 g = __ldg(reinterpret_cast<const float4*>(w + j));
    const float o0 = v[cnt].x * inv * g.x, o1 = v[cnt].y * inv * g.y;
    const float o2 = v[cnt].z * inv * g.z, o3 = v[cnt].w * inv * g.w;
    if (OUT_F32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(y) + (size_t)blockIdx.x * n + j) = make_float4(o0, o1, o2, o3);
    } else {
      uint2 p;
      p.x = pack_bf16x2(o0, o1);
      p.y = pack_bf16x2(o2, o3);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(y) + (size_t)blockIdx.x * n + j) = p;
    }
  }
}

// The same normalisation with one WARP per row (no block barrier, shuffle reduction only) for tall
// inputs: NV float4 per lane hold the row between the two passes (n <= 128 * NV).
template <bool OUT_F32, int NV>
__global__ void __launch_bounds__(256)
rms_norm_f32_warp_kernel(const float* __restrict__ x, const float* __restrict__ w, void* __restrict__ y,
                         int rows, int n, float eps) {
  lg::pdl_prologue();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float* src = x + (size_t)row * n;
  float4 v[NV];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int j = (i * 32 + lane) * 4;
    v[i] = j < n ? *reinterpret_cast<const float4*>(src + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int j = (i * 32 + lane) * 4;
    if (j < n) {
      const float4 g = __ldg(reinterpret_cast<const float4*>(w + j));
      const float o0 = v[i].x * inv * g.x, o1 = v[i].y * inv * g.y;
      const float o2 = v[i].z * inv * g.z, o3 = v[i].w * inv * g.w;
      if (OUT_F32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(y) + (size_t)row * n + j) = make_float4(o0, o1, o2, o3);
      } else {
        uint2 p;
        p.x = pack_bf16x2(o0, o1);
        p.y = pack_bf16x2(o2, o3);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(y) + (size_t)row * n + j) = p;
      }
    }
  }
}

template <bool OUT_F32, int NV>
void launch_rms_warp(const void* x, const void* w, void* y, int rows, int n, float eps, cudaStream_t s) {
  lg::launch(rms_norm_f32_warp_kernel<OUT_F32, NV>, dim3((rows + 7) / 8), dim3(256), 0, s, (const float*)x, (const float*)w, y, rows, n, eps);
}

template <bool OUT_F32>
void launch_rms_warp_nv(const void* x, const void* w, void* y, int rows, int n, float eps, cudaStream_t s) {
  if (n <= 512) launch_rms_warp<OUT_F32, 4>(x, w, y, rows, n, eps, s);
  else if (n <= 1024) launch_rms_warp<OUT_F32, 8>(x, w, y, rows, n, eps, s);
  else if (n <= 1536) launch_rms_warp<OUT_F32, 12>(x, w, y, rows, n, eps, s);
  else launch_rms_warp<OUT_F32, 16>(x, w, y, rows, n, eps, s);
}

// cpu_f32::rope_halves_in_place (mod.rs:502-547): y[i] = x[i] c - x[i+d/2] s,
// y[i+d/2] = x[i] s + x[i+d/2] c, in fp32, on bf16 storage. One thread per (token, head, pair of
// adjacent i), i.e. bf16x2 accesses in both halves.
__global__ void rope_halves_kernel(__nv_bfloat16* __restrict__ qk, const float* __restrict__ cosT,
                                   const float* __restrict__ sinT, const int* __restrict__ positions,
                                   int n_tokens, int n_heads, int head_dim, int row_stride,
                                   int max_pos, int* __restrict__ status) {
  lg::pdl_prologue();
  const int half = head_dim >> 1, pairs = half >> 1;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)n_tokens * n_heads * pairs;
  if (idx >= total) return;
  const int p = (int)(idx % pairs);
  const int h = (int)((idx / pairs) % n_heads);
  const int t = (int)(idx / ((int64_t)pairs * n_heads));
  const int pos = positions[t];
  if (pos < 0 || pos >= max_pos) {  // RopeTable::gather rejects it (rope.rs:57-66)
    if (status) atomicExch(status, 1);
    return;
  }
  __nv_bfloat16* base = qk + (size_t)t * row_stride + h * head_dim;
  const float2 c = *reinterpret_cast<const float2*>(cosT + (size_t)pos * half + 2 * p);
  const float2 s = *reinterpret_cast<const float2*>(sinT + (size_t)pos * half + 2 * p);
  uint32_t* lo = reinterpret_cast<uint32_t*>(base + 2 * p);
  uint32_t* hi = reinterpret_cast<uint32_t*>(base + half + 2 * p);
  const float2 x0 = unpack_bf16x2(*lo), x1 = unpack_bf16x2(*hi);
  *lo = pack_bf16x2(x0.x * c.x - x1.x * s.x, x0.y * c.y - x1.y * s.y);
  *hi = pack_bf16x2(x0.x * s.x + x1.x * c.x, x0.y * s.y + x1.y * c.y);
}

// The same rotation with 128-bit accesses: one thread per (token, head, 8 adjacent i); head_dim % 16 == 0.
__global__ void rope_halves_vec8_kernel(__nv_bfloat16* __restrict__ qk, const float* __restrict__ cosT,
                                        const float* __restrict__ sinT, const int* __restrict__ positions,
                                        int n_tokens, int n_heads, int head_dim, int row_stride,
                                        int max_pos, int* __restrict__ status) {
  lg::pdl_prologue();
  const int half = head_dim >> 1, octs = half >> 3;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)n_tokens * n_heads * octs;
  if (idx >= total) return;
  const int p = (int)(idx % octs);
  const int h = (int)((idx / octs) % n_heads);
  const int t = (int)(idx / ((int64_t)octs * n_heads));
  const int pos = positions[t];
  if (pos < 0 || pos >= max_pos) {  // RopeTable::gather rejects it (rope.rs:57-66)
    if (status) atomicExch(status, 1);
    return;
  }
  __nv_bfloat16* base = qk + (size_t)t * row_stride + h * head_dim + 8 * p;
  const float4* cp = reinterpret_cast<const float4*>(cosT + (size_t)pos * half + 8 * p);
  const float4* sp = reinterpret_cast<const float4*>(sinT + (size_t)pos * half + 8 * p);
  const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
  const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  uint4* lo = reinterpret_cast<uint4*>(base);
  uint4* hi = reinterpret_cast<uint4*>(base + half);
  const uint4 a = *lo, b = *hi;
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
  uint32_t ow[4], pw[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x0 = unpack_bf16x2(aw[i]), x1 = unpack_bf16x2(bw[i]);
    ow[i] = pack_bf16x2(x0.x * c[2 * i] - x1.x * s[2 * i], x0.y * c[2 * i + 1] - x1.y * s[2 * i + 1]);
    pw[i] = pack_bf16x2(x0.x * s[2 * i] + x1.x * c[2 * i], x0.y * s[2 * i + 1] + x1.y * c[2 * i + 1]);
  }
  *lo = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  *hi = make_uint4(pw[0], pw[1], pw[2], pw[3]);
}

// cpu_f32::silu (x / (1 + e^-x), mod.rs:349-351) times up (hadamard, :365-374).
__global__ void swiglu_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                              int rows, int inter) {
  lg::pdl_prologue();
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // 8 outputs per thread
  const int per_row = inter >> 3;
  if (idx >= (int64_t)rows * per_row) return;
  const int r = (int)(idx / per_row), j = (int)(idx % per_row) * 8;
  const uint4 g = __ldg(reinterpret_cast<const uint4*>(gu + (size_t)r * 2 * inter + j));
  const uint4 u = __ldg(reinterpret_cast<const uint4*>(gu + (size_t)r * 2 * inter + inter + j));
  const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
  uint32_t ow[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = unpack_bf16x2(gw[i]), b = unpack_bf16x2(uw[i]);
    ow[i] = pack_bf16x2(a.x / (1.0f + __expf(-a.x)) * b.x, a.y / (1.0f + __expf(-a.y)) * b.y);
  }
  *reinterpret_cast<uint4*>(out + (size_t)r * inter + j) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

// StellaModel::encode_raw tail (crates/embed/src/stella.rs:231-246): masked mean (mask all
// ones; zero-length sequence -> denominator 1) -> L2 (clamp 1e-12) -> W p + b -> L2, as three
// small kernels so that the token rows and the head weights are read by many CTAs:
//   pool_mean: CTA = (sequence, 128 columns), tokens summed in order (the reference's order)
//   head_rows: CTA = (sequence, 64 output rows), normalises the pooled vector on the fly
//   l2_rows:   CTA = sequence
__global__ void pool_mean_kernel(const float* __restrict__ hs, const int* __restrict__ cu,
                                 float* __restrict__ pooled, int hidden) {
  lg::pdl_prologue();
  const int s0 = cu[blockIdx.x], s1 = cu[blockIdx.x + 1];
  const int j = blockIdx.y * blockDim.x + threadIdx.x;
  if (j >= hidden) return;
  const float* p = hs + (size_t)s0 * hidden + j;
  float acc = 0.0f;
  int t = s0;
  for (; t + 8 <= s1; t += 8) {  // eight rows in flight, added in token order
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = p[(size_t)i * hidden];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += v[i];
    p += (size_t)8 * hidden;
  }
  for (; t < s1; ++t) { acc += *p; p += hidden; }
  const int len = s1 - s0;
  pooled[(size_t)blockIdx.x * hidden + j] = acc * (len > 0 ? 1.0f / (float)len : 1.0f);
}

__global__ void head_rows_kernel(const float* __restrict__ pooled, const __nv_bfloat16* __restrict__ hw,
                                 const float* __restrict__ hb, float* __restrict__ out, int hidden, int dim) {
  lg::pdl_prologue();
  extern __shared__ float pn[];  // normalised pooled vector
  __shared__ float red[32];
  const float* pv = pooled + (size_t)blockIdx.x * hidden;
  float sq = 0.0f;
  for (int j = threadIdx.x; j < hidden; j += blockDim.x) { const float v = pv[j]; pn[j] = v; sq += v * v; }
  sq = block_sum(sq, red);
  const float inv = 1.0f / fmaxf(sqrtf(sq), 1e-12f);
  for (int j = threadIdx.x; j < hidden; j += blockDim.x) pn[j] *= inv;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int o_end = min(dim, (int)(blockIdx.y + 1) * 64);
  for (int o = blockIdx.y * 64 + warp; o < o_end; o += nw) {
    const __nv_bfloat16* wr = hw + (size_t)o * hidden;
    float acc = 0.0f;
    for (int j = lane * 8; j < hidden; j += 256) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(wr + j));
      const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
      acc += a.x * pn[j] + a.y * pn[j + 1] + b.x * pn[j + 2] + b.y * pn[j + 3] +
             c.x * pn[j + 4] + c.y * pn[j + 5] + d.x * pn[j + 6] + d.y * pn[j + 7];
    }
    acc = warp_sum(acc);
    if (lane == 0) out[(size_t)blockIdx.x * dim + o] = acc + hb[o];
  }
}

__global__ void l2_rows_kernel(float* __restrict__ y, int dim) {
  lg::pdl_prologue();
  __shared__ float red[32];
  float* row = y + (size_t)blockIdx.x * dim;
  float sq = 0.0f;
  for (int j = threadIdx.x; j < dim; j += blockDim.x) sq += row[j] * row[j];
  sq = block_sum(sq, red);
  const float inv = 1.0f / fmaxf(sqrtf(sq), 1e-12f);
  for (int j = threadIdx.x; j < dim; j += blockDim.x) row[j] *= inv;
}

// decode::greedy (crates/decode/src/lib.rs:73-83): strict > from -inf, so the first maximum wins
// and NaN is never selected. One CTA per row; ties across threads resolve to the lowest index.
template <typename T>
__global__ void greedy_argmax_kernel(const T* __restrict__ logits, uint32_t* __restrict__ out, int n) {
  lg::pdl_prologue();
  __shared__ float bv[32];
  __shared__ int bi[32];
  const T* row = logits + (size_t)blockIdx.x * n;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  constexpr int V = 16 / (int)sizeof(T);  // elements per 128-bit load
  if ((n % V) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    // a thread walks its own ascending index sequence, so strict > keeps its first maximum
    for (int j = threadIdx.x * V; j < n; j += blockDim.x * V) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(row + j));
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float v = (float)e[i];
        if (v > best) { best = v; best_i = j + i; }
      }
    }
  } else {
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
      const float v = (float)row[j];
      if (v > best) { best = v; best_i = j; }
    }
  }
  auto better = [](float v, int i, float bvv, int bii) { return v > bvv || (v == bvv && i < bii); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) { bv[warp] = best; bi[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    best = lane < nw ? bv[lane] : -INFINITY;
    best_i = lane < nw ? bi[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    // nothing exceeded -inf (all -inf or NaN): the reference returns index 0
    if (lane == 0) out[blockIdx.x] = (best_i == 0x7fffffff) ? 0u : (uint32_t)best_i;
  }
}

}  // namespace

extern "C" {

uint32_t logismos_launch_embed_lookup_bf16(const void* table, const void* ids, void* out,
                                           int32_t n_ids, int32_t hidden, int32_t vocab,
                                           void* stream) {
  lg::LaunchScope launch_scope_;
  if (n_ids < 0 || hidden <= 0 || vocab <= 0 || (hidden % 8)) return lg::kInvalidValue;
  if (n_ids == 0) return 0;
  const int wpb = 8;
  // an ordered launch: the first kernel of every model step is the barrier between steps
  lg::launch_ordered(embed_lookup_kernel, dim3((n_ids + wpb - 1) / wpb), dim3(wpb * 32), 0, (cudaStream_t)stream,
      (const __nv_bfloat16*)table, (const uint32_t*)ids, (float*)out, n_ids, hidden, vocab);
  return lg::launch_status();
}

uint32_t logismos_launch_rms_norm_f32(const void* x, const void* w, void* y, int32_t rows,
                                      int32_t n, float eps, int32_t out_f32, void* stream) {
  lg::LaunchScope launch_scope_;
  if (rows < 0 || n <= 0 || (n % 4) || n > 8 * 4 * 256) return lg::kInvalidValue;
  if (rows == 0) return 0;
  if (rows >= 1024 && n <= 2048) {  // tall input: a warp per row
    if (out_f32) launch_rms_warp_nv<true>(x, w, y, rows, n, eps, (cudaStream_t)stream);
    else launch_rms_warp_nv<false>(x, w, y, rows, n, eps, (cudaStream_t)stream);
    return lg::launch_status();
  }
  int bs = 32;
  while (bs * 4 * 2 < n && bs < 256) bs <<= 1;  // aim for ~2 float4 per thread
  if (out_f32)
    lg::launch(rms_norm_f32_kernel<true>, dim3(rows), dim3(bs), 0, (cudaStream_t)stream, (const float*)x, (const float*)w, y, n, eps);
  else
    lg::launch(rms_norm_f32_kernel<false>, dim3(rows), dim3(bs), 0, (cudaStream_t)stream, (const float*)x, (const float*)w, y, n, eps);
  return lg::launch_status();
}

uint32_t logismos_launch_rope_halves_bf16(void* qk, const void* cos_f32, const void* sin_f32,
                                          const void* positions, int32_t n_tokens,
                                          int32_t n_rot_heads, int32_t head_dim,
                                          int32_t row_stride, int32_t max_pos, void* status,
                                          void* stream) {
  lg::LaunchScope launch_scope_;
  if (n_tokens < 0 || n_rot_heads <= 0 || head_dim <= 0 || (head_dim % 4) || max_pos <= 0 ||
      row_stride < n_rot_heads * head_dim || (row_stride % 2))
    return lg::kInvalidValue;
  if (n_tokens == 0) return 0;
  const int bs = 256;
  if (head_dim % 16 == 0 && row_stride % 8 == 0 && (((uintptr_t)qk | (uintptr_t)cos_f32 | (uintptr_t)sin_f32) % 16) == 0) {
    const int64_t total8 = (int64_t)n_tokens * n_rot_heads * (head_dim / 16);
    lg::launch(rope_halves_vec8_kernel, dim3((unsigned)((total8 + bs - 1) / bs)), dim3(bs), 0, (cudaStream_t)stream, 
        (__nv_bfloat16*)qk, (const float*)cos_f32, (const float*)sin_f32, (const int*)positions,
        n_tokens, n_rot_heads, head_dim, row_stride, max_pos, (int*)status);
    return lg::launch_status();
  }
  const int64_t total = (int64_t)n_tokens * n_rot_heads * (head_dim / 4);
  lg::launch(rope_halves_kernel, dim3((unsigned)((total + bs - 1) / bs)), dim3(bs), 0, (cudaStream_t)stream, 
      (__nv_bfloat16*)qk, (const float*)cos_f32, (const float*)sin_f32, (const int*)positions,
      n_tokens, n_rot_heads, head_dim, row_stride, max_pos, (int*)status);
  return lg::launch_status();
}

uint32_t logismos_launch_swiglu_bf16(const void* gu, void* out, int32_t rows, int32_t inter,
                                     void* stream) {
  lg::LaunchScope launch_scope_;
  if (rows < 0 || inter <= 0 || (inter % 8)) return lg::kInvalidValue;
  if (rows == 0) return 0;
  const int64_t total = (int64_t)rows * (inter / 8);
  const int bs = 256;
  lg::launch(swiglu_kernel, dim3((unsigned)((total + bs - 1) / bs)), dim3(bs), 0, (cudaStream_t)stream, 
      (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows, inter);
  return lg::launch_status();
}

uint32_t logismos_launch_pool_head_f32(const void* hidden_f32, const void* cu, const void* head_w,
                                       const void* head_b, void* out, void* scratch_f32, int32_t n_seqs,
                                       int32_t hidden, int32_t dim, void* stream) {
  lg::LaunchScope launch_scope_;
  if (n_seqs < 0 || hidden <= 0 || dim <= 0 || (hidden % 8) || (size_t)hidden * 4 > 48 * 1024 || !scratch_f32)
    return lg::kInvalidValue;
  if (n_seqs == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  lg::launch(pool_mean_kernel, dim3(n_seqs, (hidden + 127) / 128), dim3(128), 0, s, (const float*)hidden_f32, (const int*)cu,
                                                                      (float*)scratch_f32, hidden);
  uint32_t rc = lg::launch_status();
  if (rc) return rc;
  lg::launch(head_rows_kernel, dim3(n_seqs, (dim + 63) / 64), dim3(256), (size_t)hidden * 4, s, 
      (const float*)scratch_f32, (const __nv_bfloat16*)head_w, (const float*)head_b, (float*)out, hidden, dim);
  rc = lg::launch_status();
  if (rc) return rc;
  lg::launch(l2_rows_kernel, dim3(n_seqs), dim3(256), 0, s, (float*)out, dim);
  return lg::launch_status();
}

uint32_t logismos_launch_greedy_argmax(const void* logits, int32_t logits_f32, void* out,
                                       int32_t rows, int32_t n, void* stream) {
  lg::LaunchScope launch_scope_;
  if (rows < 0 || n <= 0) return lg::kInvalidValue;
  if (rows == 0) return 0;
  if (logits_f32)
    lg::launch(greedy_argmax_kernel<float>, dim3(rows), dim3(1024), 0, (cudaStream_t)stream, (const float*)logits, (uint32_t*)out, n);
  else
    lg::launch(greedy_argmax_kernel<__nv_bfloat16>, dim3(rows), dim3(1024), 0, (cudaStream_t)stream, (const __nv_bfloat16*)logits, (uint32_t*)out, n);
  return lg::launch_status();
}

}  // extern "C"

// ---- row gather (last token of each sequence before the final norm / lm_head) -------------------
namespace {
__global__ void gather_rows_f32_kernel(const float* __restrict__ src, const int* __restrict__ idx,
                                       float* __restrict__ dst, int n_rows, int width, int n_src_rows,
                                       int* __restrict__ status) {
  lg::pdl_prologue();
  const int r = blockIdx.x;
  const int s = idx[r];
  if (s < 0 || s >= n_src_rows) {
    if (threadIdx.x == 0 && status) atomicExch(status, 1);
    for (int j = threadIdx.x * 4; j < width; j += blockDim.x * 4)
      *reinterpret_cast<float4*>(dst + (size_t)r * width + j) = make_float4(0.f, 0.f, 0.f, 0.f);
    return;
  }
  for (int j = threadIdx.x * 4; j < width; j += blockDim.x * 4)
    *reinterpret_cast<float4*>(dst + (size_t)r * width + j) = *reinterpret_cast<const float4*>(src + (size_t)s * width + j);
}
}  // namespace

extern "C" uint32_t logismos_launch_gather_rows_f32(const void* src_f32, const void* idx_i32, void* dst_f32,
                                                    int32_t n_rows, int32_t width, int32_t n_src_rows,
                                                    void* status_i32, void* stream) {
  lg::LaunchScope launch_scope_;
  if (n_rows < 0 || width <= 0 || (width % 4) || n_src_rows < 0) return lg::kInvalidValue;
  if (n_rows == 0) return 0;
  lg::launch(gather_rows_f32_kernel, dim3(n_rows), dim3(128), 0, (cudaStream_t)stream, (const float*)src_f32, (const int*)idx_i32,
                                                                  (float*)dst_f32, n_rows, width, n_src_rows,
                                                                  (int*)status_i32);
  return lg::launch_status();
}

// ---- output gates of the hybrid decoder layers -----------------------------------------------------
namespace {
__global__ void gated_mul_kernel(__nv_bfloat16* __restrict__ x, int x_stride, const __nv_bfloat16* __restrict__ gate,
                                 int gate_stride, int rows, int n, int mode) {
  lg::pdl_prologue();
  const int per_row = n >> 3;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)rows * per_row) return;
  const int r = (int)(idx / per_row), j = (int)(idx % per_row) * 8;
  uint4* xp = reinterpret_cast<uint4*>(x + (size_t)r * x_stride + j);
  const uint4 xv = *xp;
  const uint4 gv = __ldg(reinterpret_cast<const uint4*>(gate + (size_t)r * gate_stride + j));
  const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
  uint32_t ow[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = unpack_bf16x2(xw[i]), g = unpack_bf16x2(gw[i]);
    const float s0 = 1.0f / (1.0f + __expf(-g.x)), s1 = 1.0f / (1.0f + __expf(-g.y));
    ow[i] = mode ? pack_bf16x2(a.x * g.x * s0, a.y * g.y * s1) : pack_bf16x2(a.x * s0, a.y * s1);
  }
  *xp = make_uint4(ow[0], ow[1], ow[2], ow[3]);
}
}  // namespace

extern "C" uint32_t logismos_launch_gated_mul_bf16(void* x, int32_t x_stride, const void* gate, int32_t gate_stride,
                                                   int32_t rows, int32_t n, int32_t mode, void* stream) {
  lg::LaunchScope launch_scope_;
  if (rows < 0 || n <= 0 || (n % 8) || (x_stride % 8) || (gate_stride % 8) || x_stride < n || gate_stride < n) return lg::kInvalidValue;
  if (rows == 0) return 0;
  const int64_t total = (int64_t)rows * (n / 8);
  lg::launch(gated_mul_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, 
      (__nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)gate, gate_stride, rows, n, mode);
  return lg::launch_status();
}

// ---- x += d (fp32): joins an all-reduced partial sum into the residual stream ------------------
namespace {
__global__ void add_f32_kernel(float* __restrict__ x, const float* __restrict__ d, int64_t n4) {
  lg::pdl_prologue();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  float4 a = reinterpret_cast<float4*>(x)[i];
  const float4 b = __ldg(reinterpret_cast<const float4*>(d) + i);
  a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
  reinterpret_cast<float4*>(x)[i] = a;
}
}  // namespace

extern "C" uint32_t logismos_launch_add_f32(void* x, const void* d, int64_t n, void* stream) {
  lg::LaunchScope launch_scope_;
  if (n < 0 || (n % 4) || ((uintptr_t)x & 15) || ((uintptr_t)d & 15)) return lg::kInvalidValue;
  if (n == 0) return 0;
  lg::launch(add_f32_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, (float*)x, (const float*)d, n / 4);
  return lg::launch_status();
}
