// int4 group-32 codes -> bf16 operand values in registers, shared by the tensor-core kernels that fuse
// the dequantisation into their operand pipeline. Storage contract: byte k/2 of a row holds value k,
// even k in the low nibble (the nibble order of Turbo4Block, crates/quant/src/lib.rs:272-301), as a
// two's-complement 4-bit integer; one fp16 scale per 32 values. A weight enters the MMA as
// bf16(code) * bf16(scale).
#pragma once
#include "common.cuh"

namespace lg {

// two nibbles of byte p of a code word (k even in the low nibble) -> bf16x2 {136 + q_even, 136 + q_odd}:
// the permute puts byte p of w under bits 0-7 and byte p of w >> 4 under bits 16-23; one logic op
// keeps the two low nibbles, flips their sign bit and ors in the exponent 0x4300
LG_DEVINL uint32_t nib_pair_136(uint32_t w, uint32_t w_shr4, uint32_t sel) {
  uint32_t t;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(t) : "r"(w), "r"(w_shr4), "r"(sel));
  return (t & 0x000f000fu) ^ 0x43084308u;
}

LG_DEVINL uint32_t bf16x2_sub_mul(uint32_t v, uint32_t c136, uint32_t s2) {
  __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&v);
  const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(&c136);
  const __nv_bfloat162 s = *reinterpret_cast<const __nv_bfloat162*>(&s2);
  a = __hmul2(__hsub2(a, c), s);
  return *reinterpret_cast<uint32_t*>(&a);
}

// 8 codes of one 32-bit word -> 8 bf16 (one 16-byte chunk of the operand tile), scaled
LG_DEVINL uint4 dequant_word(uint32_t w, uint32_t s2) {
  const uint32_t c136 = 0x43084308u;
  const uint32_t lo = w, hi = w >> 4;
  uint4 o;
  o.x = bf16x2_sub_mul(nib_pair_136(lo, hi, 0x0400u), c136, s2);  // bytes {lo.b0, x, hi.b0, x}
  o.y = bf16x2_sub_mul(nib_pair_136(lo, hi, 0x0501u), c136, s2);
  o.z = bf16x2_sub_mul(nib_pair_136(lo, hi, 0x0602u), c136, s2);
  o.w = bf16x2_sub_mul(nib_pair_136(lo, hi, 0x0703u), c136, s2);
  return o;
}

LG_DEVINL uint32_t scale_bf16x2(uint32_t packed_f16, int which) {
  const __half h = __ushort_as_half((unsigned short)(which ? (packed_f16 >> 16) : (packed_f16 & 0xffffu)));
  const __nv_bfloat16 sb = __float2bfloat16_rn(__half2float(h));
  const __nv_bfloat162 sb2 = __halves2bfloat162(sb, sb);
  return *reinterpret_cast<const uint32_t*>(&sb2);
}

}  // namespace lg
