// Gated delta rule, one decode step per (sequence, head): the T = 1 case of
// gated_delta_rule_recurrent_fwd (crates/kernels/src/gated_delta_rule/cpu.rs:92-182) over a
// batch, with the fp32 state [K=128, V=128] (row-major, k rows) updated in place.
//
//   h <- h * exp(g);  hk[v] = sum_k h[k,v] k[k];  vd = beta * (v - hk);
//   h[k,v] += k[k] * vd[v];  o[v] = sum_k h[k,v] * q[k] * scale
//
// The reference walks the 64 KB state three times per token; here each CTA (4 warps) reads it
// once into registers (warp w holds k rows 32w..32w+31 as float4 per lane, i.e. every load and
// store is a full 512-byte row), and the two column sums are reduced across the four warps
// through shared memory. The kernel is bound by the state read + write (128 KB per head).
#include "common.cuh"
#include "logismos_kernels.h"

namespace {

using namespace lg;
constexpr int KD = 128, VD = 128;

__global__ void __launch_bounds__(128)
gdn_decode_step_kernel(float* __restrict__ state, const __nv_bfloat16* __restrict__ q,
                       const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                       const float* __restrict__ g, const float* __restrict__ beta,
                       __nv_bfloat16* __restrict__ o, float scale) {
  __shared__ float ks[KD], qs[KD];
  __shared__ float4 red[4][32];
  const int64_t sh = blockIdx.x;  // seq * heads + head
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  ks[tid] = __bfloat162float(k[sh * KD + tid]);
  qs[tid] = __bfloat162float(q[sh * KD + tid]);
  const float decay = expf(g[sh]);
  const float bt = beta[sh];
  float* hp = state + sh * (int64_t)(KD * VD) + (int64_t)(warp * 32) * VD + lane * 4;
  float4 h[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) h[i] = *reinterpret_cast<const float4*>(hp + i * VD);
  __syncthreads();
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    h[i].x *= decay; h[i].y *= decay; h[i].z *= decay; h[i].w *= decay;
    const float kk = ks[warp * 32 + i];
    acc.x += h[i].x * kk; acc.y += h[i].y * kk; acc.z += h[i].z * kk; acc.w += h[i].w * kk;
  }
  red[warp][lane] = acc;
  __syncthreads();
  float4 hk = red[0][lane];
#pragma unroll
  for (int w = 1; w < 4; ++w) { const float4 t = red[w][lane]; hk.x += t.x; hk.y += t.y; hk.z += t.z; hk.w += t.w; }
  const uint2 vraw = *reinterpret_cast<const uint2*>(v + sh * VD + lane * 4);
  const float2 v01 = unpack_bf16x2(vraw.x), v23 = unpack_bf16x2(vraw.y);
  const float4 vd = make_float4(bt * (v01.x - hk.x), bt * (v01.y - hk.y), bt * (v23.x - hk.z), bt * (v23.y - hk.w));
  __syncthreads();  // red is reused below
  acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float kk = ks[warp * 32 + i], qq = qs[warp * 32 + i];
    h[i].x += kk * vd.x; h[i].y += kk * vd.y; h[i].z += kk * vd.z; h[i].w += kk * vd.w;
    *reinterpret_cast<float4*>(hp + i * VD) = h[i];
    acc.x += h[i].x * qq * scale; acc.y += h[i].y * qq * scale;
    acc.z += h[i].z * qq * scale; acc.w += h[i].w * qq * scale;
  }
  red[warp][lane] = acc;
  __syncthreads();
  if (warp == 0) {
    float4 ov = red[0][lane];
#pragma unroll
    for (int w = 1; w < 4; ++w) { const float4 t = red[w][lane]; ov.x += t.x; ov.y += t.y; ov.z += t.z; ov.w += t.w; }
    uint2 p;
    p.x = pack_bf16x2(ov.x, ov.y);
    p.y = pack_bf16x2(ov.z, ov.w);
    *reinterpret_cast<uint2*>(o + sh * VD + lane * 4) = p;
  }
}


// The same recurrence over the tokens of each sequence of a ragged batch (prefill, and decode as
// sequences of one token): tokens are taken in order, which is what gated_delta_rule_chunk_fwd
// specifies (the recurrence applied chunk by chunk with the state carried, cpu.rs:201-249).
//
// The latency of one token is what bounds a long prompt, so the 128 x 128 state of a (sequence,
// head) is spread over 512 threads: CTA = (sequence, head, 32 value columns), 128 threads; a
// thread owns one value column and one quarter of the key rows (32 floats in registers), the four
// quarter-owners of a column are neighbouring lanes, and both column sums are two shuffles. There
// is no cross-warp reduction; the only barrier per token is the one that publishes the next token's
// k and q, which were fetched from global memory while the current token was being computed.
constexpr int kPfCols = 32;            // value columns per CTA
constexpr int kPfQuarterPitch = 36;    // floats between the quarters of k / q in shared memory (bank offset 4)

__global__ void __launch_bounds__(128)
gdn_prefill_kernel(float* __restrict__ state, const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                   const __nv_bfloat16* __restrict__ v, const float* __restrict__ g, const float* __restrict__ beta,
                   __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ z, const int* __restrict__ cu,
                   const int* __restrict__ slots, const uint8_t* __restrict__ fresh, int heads, int64_t qkv_stride, float scale) {
  __shared__ __align__(16) float ks[2][4 * kPfQuarterPitch], qs[2][4 * kPfQuarterPitch];
  const int part = blockIdx.x & 3, sh = blockIdx.x >> 2;
  const int seq = sh / heads, head = sh % heads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kq = lane & 3;                                   // quarter of the key rows: 32 kq .. 32 kq + 31
  const int col = part * kPfCols + warp * 8 + (lane >> 2);   // value column
  const int t0 = cu[seq], t1 = cu[seq + 1];
  if (t1 <= t0) return;
  const int64_t slot = slots ? slots[seq] : seq;
  float* hp = state + (slot * heads + head) * (int64_t)(KD * VD) + (int64_t)(kq * 32) * VD + col;
  const bool zero_start = fresh && fresh[seq];  // a sequence that starts here begins from the zero state
  float h[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) h[i] = zero_start ? 0.f : hp[i * VD];
  const int stage_at = (tid >> 5) * kPfQuarterPitch + (tid & 31);  // where this thread's k / q element lands
  {
    const int64_t tq = (int64_t)t0 * qkv_stride + head * KD;
    ks[0][stage_at] = __bfloat162float(k[tq + tid]);
    qs[0][stage_at] = __bfloat162float(q[tq + tid]);
  }
  float v_cur = __bfloat162float(v[(int64_t)t0 * qkv_stride + head * KD + col]);
  float z_cur = z ? __bfloat162float(z[(int64_t)t0 * qkv_stride + head * KD + col]) : 0.f;
  float g_cur = g[(int64_t)t0 * heads + head], b_cur = beta[(int64_t)t0 * heads + head];
  __syncthreads();
  for (int t = t0; t < t1; ++t) {
    const int b = (t - t0) & 1;
    // fetch the next token while this one is computed
    float k_nx = 0.f, q_nx = 0.f, v_nx = 0.f, g_nx = 0.f, b_nx = 0.f, z_nx = 0.f;
    if (t + 1 < t1) {
      const int64_t tq = (int64_t)(t + 1) * qkv_stride + head * KD;
      k_nx = __bfloat162float(k[tq + tid]);
      q_nx = __bfloat162float(q[tq + tid]);
      v_nx = __bfloat162float(v[tq + col]);
      if (z) z_nx = __bfloat162float(z[tq + col]);
      g_nx = g[(int64_t)(t + 1) * heads + head];
      b_nx = beta[(int64_t)(t + 1) * heads + head];
    }
    const float decay = expf(g_cur);
    const float4* k4 = reinterpret_cast<const float4*>(&ks[b][kq * kPfQuarterPitch]);
    const float4* q4 = reinterpret_cast<const float4*>(&qs[b][kq * kPfQuarterPitch]);
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 kk = k4[i];
      h[4 * i] *= decay; h[4 * i + 1] *= decay; h[4 * i + 2] *= decay; h[4 * i + 3] *= decay;
      a0 += h[4 * i] * kk.x; a1 += h[4 * i + 1] * kk.y; a2 += h[4 * i + 2] * kk.z; a3 += h[4 * i + 3] * kk.w;
    }
    float hk = (a0 + a1) + (a2 + a3);
    hk += __shfl_xor_sync(0xffffffffu, hk, 1);
    hk += __shfl_xor_sync(0xffffffffu, hk, 2);
    const float vd = b_cur * (v_cur - hk);
    a0 = a1 = a2 = a3 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 kk = k4[i], qq = q4[i];
      h[4 * i] += kk.x * vd; h[4 * i + 1] += kk.y * vd; h[4 * i + 2] += kk.z * vd; h[4 * i + 3] += kk.w * vd;
      a0 += h[4 * i] * qq.x; a1 += h[4 * i + 1] * qq.y; a2 += h[4 * i + 2] * qq.z; a3 += h[4 * i + 3] * qq.w;
    }
    float ov = (a0 + a1) + (a2 + a3);
    ov += __shfl_xor_sync(0xffffffffu, ov, 1);
    ov += __shfl_xor_sync(0xffffffffu, ov, 2);
    ov *= scale;
    if (z) ov *= z_cur / (1.0f + __expf(-z_cur));  // output gate silu(z), fused
    if (kq == 0) o[((int64_t)t * heads + head) * VD + col] = __float2bfloat16(ov);
    ks[b ^ 1][stage_at] = k_nx;
    qs[b ^ 1][stage_at] = q_nx;
    v_cur = v_nx; g_cur = g_nx; b_cur = b_nx; z_cur = z_nx;
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) hp[i * VD] = h[i];
}

// Per (token, head): g = -exp(A_log[h]) * softplus(a + dt_bias[h]) with softplus(x) = x for
// x > 20, beta = sigmoid(b), all fp32; and q, k rows of 128 scaled to unit L2 norm in place
// (l2_norm_in_place, cpu.rs:19-34, norm clamped at 1e-12). One warp per (token, head).
__global__ void gdn_prepare_kernel(__nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                                   const float* __restrict__ a, const float* __restrict__ b,
                                   const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                   float* __restrict__ g, float* __restrict__ beta, int64_t rows, int heads,
                                   int64_t qk_stride, int ab_stride) {
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    __nv_bfloat16* p = (which ? k : q) + (r / heads) * qk_stride + (r % heads) * KD + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 x01 = unpack_bf16x2(raw.x), x23 = unpack_bf16x2(raw.y);
    float sq = x01.x * x01.x + x01.y * x01.y + x23.x * x23.x + x23.y * x23.y;
    sq = warp_sum(sq);
    const float inv = 1.0f / fmaxf(sqrtf(sq), 1e-12f);
    uint2 w;
    w.x = pack_bf16x2(x01.x * inv, x01.y * inv);
    w.y = pack_bf16x2(x23.x * inv, x23.y * inv);
    *reinterpret_cast<uint2*>(p) = w;
  }
  if (lane == 0) {
    const int h = (int)(r % heads);
    const int64_t ab = (r / heads) * ab_stride + h;
    const float x = a[ab] + dt_bias[h];
    const float sp = x > 20.0f ? x : log1pf(expf(x));
    g[r] = -expf(A_log[h]) * sp;
    beta[r] = 1.0f / (1.0f + expf(-b[ab]));
  }
}

// The same preparation straight from the fp32 accumulation workspace of the input projection
// (columns q | k | v | z | a | b of every token row): one warp per (token, head) normalises q and k in
// fp32, rounds q, k, v, z to bf16 once, computes the gates, and leaves the workspace zeroed.
__global__ void gdn_finish_kernel(float* __restrict__ acc, int64_t ld_acc, const float* __restrict__ A_log,
                                  const float* __restrict__ dt_bias, __nv_bfloat16* __restrict__ proj, int64_t ld_proj,
                                  float* __restrict__ g, float* __restrict__ beta, int64_t rows, int heads) {
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const int64_t t = r / heads;
  const int h = (int)(r % heads);
  const int w = heads * KD;
  float* arow = acc + t * ld_acc + h * KD + lane * 4;
  __nv_bfloat16* prow = proj + t * ld_proj + h * KD + lane * 4;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int which = 0; which < 4; ++which) {  // q, k, v, z
    float4* src = reinterpret_cast<float4*>(arow + which * w);
    float4 x = *src;
    *src = zero;
    if (which < 2) {
      const float sq = warp_sum(x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w);
      const float inv = 1.0f / fmaxf(sqrtf(sq), 1e-12f);
      x.x *= inv; x.y *= inv; x.z *= inv; x.w *= inv;
    }
    uint2 o;
    o.x = pack_bf16x2(x.x, x.y);
    o.y = pack_bf16x2(x.z, x.w);
    *reinterpret_cast<uint2*>(prow + which * w) = o;
  }
  if (lane == 0) {
    float* ab = acc + t * ld_acc + 4 * w;
    const float x = ab[h] + dt_bias[h];
    const float sp = x > 20.0f ? x : log1pf(expf(x));
    g[r] = -expf(A_log[h]) * sp;
    beta[r] = 1.0f / (1.0f + expf(-ab[heads + h]));
    ab[h] = 0.0f;
    ab[heads + h] = 0.0f;
  }
}

}  // namespace

extern "C" uint32_t logismos_launch_gdn_finish(void* acc, int32_t ld_acc, const void* A_log, const void* dt_bias, void* proj,
                                               int32_t ld_proj, void* g, void* beta, int32_t n_tokens, int32_t heads,
                                               void* stream) {
  lg::LaunchScope launch_scope_;
  const int w = heads * KD;
  if (n_tokens < 0 || heads <= 0 || ld_acc < 4 * w + 2 * heads || (ld_acc % 4) || ld_proj < 4 * w || (ld_proj % 4)) return lg::kInvalidValue;
  if (n_tokens == 0) return 0;
  if (((uintptr_t)acc & 15) || ((uintptr_t)proj & 7)) return lg::kInvalidValue;
  const int64_t rows = (int64_t)n_tokens * heads;
  const int wpb = 8;
  gdn_finish_kernel<<<(unsigned)((rows + wpb - 1) / wpb), wpb * 32, 0, (cudaStream_t)stream>>>(
      (float*)acc, (int64_t)ld_acc, (const float*)A_log, (const float*)dt_bias, (__nv_bfloat16*)proj, (int64_t)ld_proj, (float*)g,
      (float*)beta, rows, heads);
  return lg::launch_status();
}

extern "C" uint32_t logismos_launch_gdn_decode_step(void* state, const void* q, const void* k, const void* v,
                                                    const void* g, const void* beta, void* o, int32_t n_seqs,
                                                    int32_t heads, float scale, void* stream) {
  lg::LaunchScope launch_scope_;
  if (n_seqs < 0 || heads <= 0) return lg::kInvalidValue;
  if (n_seqs == 0) return 0;
  if (((uintptr_t)state & 15) || ((uintptr_t)v & 7) || ((uintptr_t)o & 7)) return lg::kInvalidValue;
  const int64_t ctas = (int64_t)n_seqs * heads;
  if (ctas > 2147483647ll) return lg::kInvalidValue;
  gdn_decode_step_kernel<<<(unsigned)ctas, 128, 0, (cudaStream_t)stream>>>(
      (float*)state, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const float*)g,
      (const float*)beta, (__nv_bfloat16*)o, scale);
  return lg::launch_status();
}

extern "C" uint32_t logismos_launch_gdn_prefill(void* state, const void* q, const void* k, const void* v, const void* g,
                                                const void* beta, void* o, const void* gate_z, const void* cu_seqlens,
                                                const void* state_slots, const void* fresh, int32_t n_seqs,
                                                int32_t heads, int32_t qkv_stride, float scale, void* stream) {
  lg::LaunchScope launch_scope_;
  if (n_seqs < 0 || heads <= 0 || qkv_stride < heads * KD || (qkv_stride % 4)) return lg::kInvalidValue;
  if (n_seqs == 0) return 0;
  if (((uintptr_t)state & 15) || ((uintptr_t)v & 7) || ((uintptr_t)o & 7)) return lg::kInvalidValue;
  const int64_t ctas = (int64_t)n_seqs * heads * (VD / kPfCols);
  if (ctas > 2147483647ll) return lg::kInvalidValue;
  gdn_prefill_kernel<<<(unsigned)ctas, 128, 0, (cudaStream_t)stream>>>(
      (float*)state, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const float*)g,
      (const float*)beta, (__nv_bfloat16*)o, (const __nv_bfloat16*)gate_z, (const int*)cu_seqlens, (const int*)state_slots, (const uint8_t*)fresh, heads,
      (int64_t)qkv_stride, scale);
  return lg::launch_status();
}

extern "C" uint32_t logismos_launch_gdn_prepare(void* q, void* k, const void* a, const void* b, const void* A_log,
                                                const void* dt_bias, void* g, void* beta, int32_t n_tokens,
                                                int32_t heads, int32_t qk_stride, int32_t ab_stride, void* stream) {
  lg::LaunchScope launch_scope_;
  if (n_tokens < 0 || heads <= 0 || qk_stride < heads * KD || (qk_stride % 4) || ab_stride < heads) return lg::kInvalidValue;
  if (n_tokens == 0) return 0;
  if (((uintptr_t)q & 7) || ((uintptr_t)k & 7)) return lg::kInvalidValue;
  const int64_t rows = (int64_t)n_tokens * heads;
  const int wpb = 8;
  gdn_prepare_kernel<<<(unsigned)((rows + wpb - 1) / wpb), wpb * 32, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)q, (__nv_bfloat16*)k, (const float*)a, (const float*)b, (const float*)A_log, (const float*)dt_bias,
      (float*)g, (float*)beta, rows, heads, (int64_t)qk_stride, ab_stride);
  return lg::launch_status();
}
