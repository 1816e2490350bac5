// int4 group-32 -> bf16 expansion of a weight matrix: w[n,k] = bf16(scale[n,k/32] * q[n,k]).
// Used on the prefill side of a mixed step, where hundreds of token rows share the weights and the
// contraction belongs on the tcgen05 GEMM: the codes are expanded once per layer into a bf16
// scratch matrix that the GEMM then reads. Same storage contract as the GEMV kernel (nibble order
// of Turbo4Block, crates/quant/src/lib.rs:272-301; two's-complement codes; fp16 scale per 32).
// The fp32 product of an fp16 scale and a 4-bit integer is exact, so the only rounding is the
// final bf16 store. HBM-bound: 0.5625 B read + 2 B written per weight.
#include "common.cuh"
#include "logismos_kernels.h"

namespace {

using namespace lg;

__global__ void dequant_int4_g32_kernel(const uint32_t* __restrict__ codes, const __half* __restrict__ scales,
                                        __nv_bfloat16* __restrict__ out, int64_t n_words, int words_per_row) {
  lg::pdl_prologue();
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one 32-bit word = 8 weights
  if (idx >= n_words) return;
  const int64_t row = idx / words_per_row;
  const int wi = (int)(idx % words_per_row);
  const uint32_t w = __ldg(codes + idx);
  const float s = __half2float(__ldg(scales + row * (words_per_row >> 2) + (wi >> 2)));
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int lo = (int)((w >> (8 * i)) & 0xf), hi = (int)((w >> (8 * i + 4)) & 0xf);
    o[i] = pack_bf16x2(s * (float)((lo ^ 8) - 8), s * (float)((hi ^ 8) - 8));
  }
  *reinterpret_cast<uint4*>(out + idx * 8) = make_uint4(o[0], o[1], o[2], o[3]);
}

// fp32 [n, k] -> int4 group-32: one thread per group of 32 values. scale = fp16(max|w| / 7) (round to
// nearest even), code = clamp(round-half-even(w / scale), -8, 7), 0 when the scale is 0; codes packed
// two per byte, even k in the low nibble. Integer output: bit-exact against the CPU definition.
__global__ void quantize_int4_g32_kernel(const float* __restrict__ w, uint32_t* __restrict__ codes, __half* __restrict__ scales,
                                         int64_t n_groups) {
  lg::pdl_prologue();
  const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= n_groups) return;
  const float4* src = reinterpret_cast<const float4*>(w + g * 32);
  float v[32];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 t = __ldg(src + i);
    v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
  }
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const __half sh = __float2half_rn(__fdiv_rn(amax, 7.0f));
  const float s = __half2float(sh);
  scales[g] = sh;
  uint32_t out[4];
#pragma unroll
  for (int wi = 0; wi < 4; ++wi) {
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float q = s > 0.0f ? rintf(__fdiv_rn(v[wi * 8 + j], s)) : 0.0f;
      const int c = (int)fminf(7.0f, fmaxf(-8.0f, q));
      word |= (uint32_t)(c & 0xf) << (4 * j);
    }
    out[wi] = word;
  }
  *reinterpret_cast<uint4*>(codes + g * 4) = make_uint4(out[0], out[1], out[2], out[3]);
}

}  // namespace

extern "C" uint32_t logismos_launch_quantize_int4_g32(const void* w_f32, void* codes_u8, void* scales_f16, int32_t n, int32_t k,
                                                      void* stream) {
  lg::LaunchScope launch_scope_;
  if (n <= 0 || k <= 0 || (k % 32) || ((uintptr_t)w_f32 & 15) || ((uintptr_t)codes_u8 & 15) || ((uintptr_t)scales_f16 & 1))
    return lg::kInvalidValue;
  const int64_t groups = (int64_t)n * (k / 32);
  const int64_t blocks = (groups + 127) / 128;
  if (blocks > 2147483647ll) return lg::kInvalidValue;
  lg::launch(quantize_int4_g32_kernel, dim3((unsigned)blocks), dim3(128), 0, (cudaStream_t)stream, (const float*)w_f32, (uint32_t*)codes_u8, (__half*)scales_f16, groups);
  return lg::launch_status();
}

extern "C" uint32_t logismos_launch_dequant_int4_g32_bf16(const void* codes, const void* scales, void* out_bf16,
                                                          int32_t n, int32_t k, void* stream) {
  lg::LaunchScope launch_scope_;
  if (n <= 0 || k <= 0 || (k % 32) || ((uintptr_t)codes & 3) || ((uintptr_t)out_bf16 & 15)) return lg::kInvalidValue;
  const int64_t n_words = (int64_t)n * (k / 8);
  const int bs = 256;
  const int64_t blocks = (n_words + bs - 1) / bs;
  if (blocks > 2147483647ll) return lg::kInvalidValue;
  lg::launch(dequant_int4_g32_kernel, dim3((unsigned)blocks), dim3(bs), 0, (cudaStream_t)stream, 
      (const uint32_t*)codes, (const __half*)scales, (__nv_bfloat16*)out_bf16, n_words, k / 8);
  return lg::launch_status();
}
