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
