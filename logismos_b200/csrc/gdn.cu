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


// The same recurrence over the tokens of each sequence of a ragged batch (prefill): CTA =
// (sequence, head), the state stays in registers for the whole sequence and is read and written
// once; tokens are taken in order, which is what gated_delta_rule_chunk_fwd specifies (the
// recurrence applied chunk by chunk with the state carried, cpu.rs:201-249).
__global__ void __launch_bounds__(128)
gdn_prefill_kernel(float* __restrict__ state, const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                   const __nv_bfloat16* __restrict__ v, const float* __restrict__ g, const float* __restrict__ beta,
                   __nv_bfloat16* __restrict__ o, const int* __restrict__ cu, int heads, float scale) {
  __shared__ float ks[2][KD], qs[2][KD];
  __shared__ float4 red[2][4][32];
  const int seq = blockIdx.x / heads, head = blockIdx.x % heads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t0 = cu[seq], t1 = cu[seq + 1];
  float* hp = state + ((int64_t)seq * heads + head) * (int64_t)(KD * VD) + (int64_t)(warp * 32) * VD + lane * 4;
  float4 h[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) h[i] = *reinterpret_cast<const float4*>(hp + i * VD);
  for (int t = t0; t < t1; ++t) {
    const int64_t th = (int64_t)t * heads + head;
    const int b = (t - t0) & 1;  // double-buffered staging: one barrier per reduction, none for the loads
    ks[b][tid] = __bfloat162float(k[th * KD + tid]);
    qs[b][tid] = __bfloat162float(q[th * KD + tid]);
    const float decay = expf(g[th]);
    const float bt = beta[th];
    const uint2 vraw = *reinterpret_cast<const uint2*>(v + th * VD + lane * 4);
    __syncthreads();
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      h[i].x *= decay; h[i].y *= decay; h[i].z *= decay; h[i].w *= decay;
      const float kk = ks[b][warp * 32 + i];
      acc.x += h[i].x * kk; acc.y += h[i].y * kk; acc.z += h[i].z * kk; acc.w += h[i].w * kk;
    }
    red[0][warp][lane] = acc;
    __syncthreads();
    float4 hk = red[0][0][lane];
#pragma unroll
    for (int w = 1; w < 4; ++w) { const float4 x = red[0][w][lane]; hk.x += x.x; hk.y += x.y; hk.z += x.z; hk.w += x.w; }
    const float2 v01 = unpack_bf16x2(vraw.x), v23 = unpack_bf16x2(vraw.y);
    const float4 vd = make_float4(bt * (v01.x - hk.x), bt * (v01.y - hk.y), bt * (v23.x - hk.z), bt * (v23.y - hk.w));
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float kk = ks[b][warp * 32 + i], qq = qs[b][warp * 32 + i];
      h[i].x += kk * vd.x; h[i].y += kk * vd.y; h[i].z += kk * vd.z; h[i].w += kk * vd.w;
      acc.x += h[i].x * qq * scale; acc.y += h[i].y * qq * scale;
      acc.z += h[i].z * qq * scale; acc.w += h[i].w * qq * scale;
    }
    red[1][warp][lane] = acc;
    __syncthreads();
    if (warp == 0) {
      float4 ov = red[1][0][lane];
#pragma unroll
      for (int w = 1; w < 4; ++w) { const float4 x = red[1][w][lane]; ov.x += x.x; ov.y += x.y; ov.z += x.z; ov.w += x.w; }
      uint2 pk;
      pk.x = pack_bf16x2(ov.x, ov.y);
      pk.y = pack_bf16x2(ov.z, ov.w);
      *reinterpret_cast<uint2*>(o + th * VD + lane * 4) = pk;
    }
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) *reinterpret_cast<float4*>(hp + i * VD) = h[i];
}

// Per (token, head): g = -exp(A_log[h]) * softplus(a + dt_bias[h]) with softplus(x) = x for
// x > 20, beta = sigmoid(b), all fp32; and q, k rows of 128 scaled to unit L2 norm in place
// (l2_norm_in_place, cpu.rs:19-34, norm clamped at 1e-12). One warp per (token, head).
__global__ void gdn_prepare_kernel(__nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                                   const float* __restrict__ a, const float* __restrict__ b,
                                   const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                   float* __restrict__ g, float* __restrict__ beta, int64_t rows, int heads) {
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    __nv_bfloat16* p = (which ? k : q) + r * KD + lane * 4;
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
    const float x = a[r] + dt_bias[h];
    const float sp = x > 20.0f ? x : log1pf(expf(x));
    g[r] = -expf(A_log[h]) * sp;
    beta[r] = 1.0f / (1.0f + expf(-b[r]));
  }
}

}  // namespace

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
                                                const void* beta, void* o, const void* cu_seqlens, int32_t n_seqs,
                                                int32_t heads, float scale, void* stream) {
  lg::LaunchScope launch_scope_;
  if (n_seqs < 0 || heads <= 0) return lg::kInvalidValue;
  if (n_seqs == 0) return 0;
  if (((uintptr_t)state & 15) || ((uintptr_t)v & 7) || ((uintptr_t)o & 7)) return lg::kInvalidValue;
  const int64_t ctas = (int64_t)n_seqs * heads;
  if (ctas > 2147483647ll) return lg::kInvalidValue;
  gdn_prefill_kernel<<<(unsigned)ctas, 128, 0, (cudaStream_t)stream>>>(
      (float*)state, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const float*)g,
      (const float*)beta, (__nv_bfloat16*)o, (const int*)cu_seqlens, heads, scale);
  return lg::launch_status();
}

extern "C" uint32_t logismos_launch_gdn_prepare(void* q, void* k, const void* a, const void* b, const void* A_log,
                                                const void* dt_bias, void* g, void* beta, int32_t n_tokens,
                                                int32_t heads, void* stream) {
  lg::LaunchScope launch_scope_;
  if (n_tokens < 0 || heads <= 0) return lg::kInvalidValue;
  if (n_tokens == 0) return 0;
  if (((uintptr_t)q & 7) || ((uintptr_t)k & 7)) return lg::kInvalidValue;
  const int64_t rows = (int64_t)n_tokens * heads;
  const int wpb = 8;
  gdn_prepare_kernel<<<(unsigned)((rows + wpb - 1) / wpb), wpb * 32, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)q, (__nv_bfloat16*)k, (const float*)a, (const float*)b, (const float*)A_log, (const float*)dt_bias,
      (float*)g, (float*)beta, rows, heads);
  return lg::launch_status();
}
