// TurboQuant 3-bit head codec on a warp: the device form of encode_turbo3_0_head /
// decode_turbo3_0_head (crates/quant/src/lib.rs:316-413), fwht_128 (:90-114) and the codebook of
// :73-82. One warp handles one 128-value head chunk; a lane holds values 4 lane .. 4 lane + 3. The
// arithmetic follows the reference operation by operation (sequential sum of squares with separate
// multiply and add, true divisions, the reference's butterflies, first-minimum centroid) so that the
// 56 bytes of a chunk come out identical.
#pragma once
#include "common.cuh"

namespace lg {
namespace t3 {

__device__ __constant__ static float kCodebook3[8] = {-0.1883972972f, -0.1181399059f, -0.0665857641f, -0.0216044751f,
                                    0.0216041461f,  0.0665854520f,  0.1181396281f,  0.1883970748f};
constexpr float kFwhtScale = 0.08838834764831844f;  // 1 / sqrt(128)
constexpr int kBlockBytes = 14, kChunkBytes = 56;

// Walsh-Hadamard transform over the 128 values a warp holds (lane: elements 4 lane + j), then the scale
LG_DEVINL void fwht_warp(float (&x)[4], int lane) {
  // h = 1, 2: partners inside the lane
  float a = __fadd_rn(x[0], x[1]), b = __fsub_rn(x[0], x[1]), c = __fadd_rn(x[2], x[3]), d = __fsub_rn(x[2], x[3]);
  x[0] = __fadd_rn(a, c); x[2] = __fsub_rn(a, c); x[1] = __fadd_rn(b, d); x[3] = __fsub_rn(b, d);
  // h = 4 .. 64: partner lane = lane ^ (h / 4); the lane with the bit clear holds the "lo" element
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
    const bool hi = (lane & m) != 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float p = __shfl_xor_sync(0xffffffffu, x[j], m);
      x[j] = hi ? __fsub_rn(p, x[j]) : __fadd_rn(x[j], p);
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) x[j] = __fmul_rn(x[j], kFwhtScale);
}

LG_DEVINL int nearest3(float v) {
  int best = 0;
  float bd = fabsf(__fsub_rn(v, kCodebook3[0]));
#pragma unroll
  for (int c = 1; c < 8; ++c) {
    const float dd = fabsf(__fsub_rn(v, kCodebook3[c]));
    if (dd < bd) { bd = dd; best = c; }
  }
  return best;
}

// one head chunk: 128 values in the warp's registers -> 56 bytes at dst (8-byte aligned)
LG_DEVINL void encode_chunk(const float (&v)[4], uint8_t* dst, float* sq /* shared, 128 floats of this warp */, int lane) {
#pragma unroll
  for (int j = 0; j < 4; ++j) sq[lane * 4 + j] = __fmul_rn(v[j], v[j]);
  __syncwarp();
  float sum = 0.0f;
  if (lane == 0)
    for (int i = 0; i < 128; ++i) sum = __fadd_rn(sum, sq[i]);  // the reference's order
  sum = __shfl_sync(0xffffffffu, sum, 0);
  __syncwarp();
  const float norm = sqrtf(sum);  // IEEE square root
  const unsigned short nb = __half_as_ushort(__float2half_rn(norm));
  float t[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) t[j] = norm > 1e-12f ? __fdiv_rn(v[j], norm) : 0.0f;
  fwht_warp(t, lane);
  // 12 bits of this lane: indices 4l .. 4l + 3 of block lane / 8 at bit 12 (lane % 8) of its 96-bit field
  const uint32_t bits = (uint32_t)nearest3(t[0]) | ((uint32_t)nearest3(t[1]) << 3) | ((uint32_t)nearest3(t[2]) << 6) | ((uint32_t)nearest3(t[3]) << 9);
  uint32_t* words = reinterpret_cast<uint32_t*>(sq);  // reuse as 14 words of staging
  if (lane < 14) words[lane] = 0u;
  __syncwarp();
  const int blk = lane >> 3, l = lane & 7;
  const int bit0 = (blk * kBlockBytes + 2) * 8 + 12 * l;  // absolute bit position in the 56-byte chunk
  atomicOr(&words[bit0 >> 5], bits << (bit0 & 31));
  if ((bit0 & 31) > 20) atomicOr(&words[(bit0 >> 5) + 1], bits >> (32 - (bit0 & 31)));
  if (l == 0) {
    const int nb0 = blk * kBlockBytes * 8;  // the block's norm: 16 bits at byte 14 blk (may straddle a word: byte offsets 0, 14, 28, 42)
    atomicOr(&words[nb0 >> 5], (uint32_t)nb << (nb0 & 31));
    if ((nb0 & 31) > 16) atomicOr(&words[(nb0 >> 5) + 1], (uint32_t)nb >> (32 - (nb0 & 31)));
  }
  __syncwarp();
  if (lane < 14) reinterpret_cast<uint32_t*>(dst)[lane] = words[lane];
  __syncwarp();
}

// 56 bytes at src -> 128 values in the warp's registers
LG_DEVINL void decode_chunk(const uint8_t* src, float (&out)[4], uint32_t* words /* shared, 14 words of this warp */, int lane) {
  if (lane < 14) words[lane] = __ldg(reinterpret_cast<const uint32_t*>(src) + lane);
  __syncwarp();
  const int blk = lane >> 3, l = lane & 7;
  const int bit0 = (blk * kBlockBytes + 2) * 8 + 12 * l;
  uint32_t bits = words[bit0 >> 5] >> (bit0 & 31);
  if ((bit0 & 31) > 20) bits |= words[(bit0 >> 5) + 1] << (32 - (bit0 & 31));
  const uint32_t nbits = (words[0] & 0xffffu);  // the first block's norm (decode reads blocks[0], lib.rs:399-407)
  __syncwarp();
#pragma unroll
  for (int j = 0; j < 4; ++j) out[j] = kCodebook3[(bits >> (3 * j)) & 7u];
  fwht_warp(out, lane);
  const float norm = __half2float(__ushort_as_half((unsigned short)nbits));
#pragma unroll
  for (int j = 0; j < 4; ++j) out[j] = __fmul_rn(out[j], norm);
}

}  // namespace t3
}  // namespace lg
