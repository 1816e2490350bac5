// Gated delta rule over a ragged batch, chunk-parallel form: the same function as
// gated_delta_rule_chunk_fwd (crates/kernels/src/gated_delta_rule/cpu.rs:201-249, the recurrence of
// :92-182 applied chunk by chunk with the state carried), but with the 64 tokens of a chunk resolved
// together by matrix products instead of one after the other, so that a long prompt is no longer
// bound by a token-serial dependency chain.
//
// For a chunk with incoming state S [K, V], cumulative log-decays c_i = g_1 + .. + g_i, gamma_i = exp(c_i):
//   A = strict_tril( diag(beta) (K K^T) * exp(c_i - c_j) )            [64 x 64]
//   T = (I + A)^-1 (forward substitution, fp32, then bf16);  [W | U] = T diag(beta) [K * gamma | V]
//   dV = U - W S                                                       the values the chunk really adds
//   O  = scale * ( gamma_i (Q S) + tril( (Q K^T) * exp(c_i - c_j) ) dV )
//   S' = gamma_64 S + K^T ( dV * exp(c_64 - c_i) )
// which equals the recurrence exactly in exact arithmetic. The products run on mma.sync m16n8k16
// (bf16 operands, fp32 accumulation); the state is kept in fp32 and enters the products rounded to
// bf16, the triangular inverse is computed in fp32 (and applied in bf16), all decay factors are fp32.
//
// CTA = (sequence, head, half of the value columns), 256 threads, chunks of the sequence in order.
#include "common.cuh"
#include "logismos_kernels.h"

namespace {

using namespace lg;

constexpr int KD = 128;    // key dim
constexpr int VDIM = 128;  // value dim
constexpr int VW = 64;     // value columns per CTA
constexpr int CH = 64;     // tokens per chunk
constexpr int kThreads = 256;
constexpr int kAPitch = CH + 4;  // floats per row of the coefficient matrix (16-byte aligned rows)

// byte address of 16-byte piece `piece` of row `row` in a bf16 tile with RB bytes per row (256 or 128)
template <int RB>
LG_DEVINL uint32_t taddr(uint32_t base, int row, int piece) {
  return base + (uint32_t)row * RB + (uint32_t)((piece ^ (row & 7)) << 4);
}

// A fragments (16 rows r0.., KT k-steps of 16) of a row-major [rows][k] tile
template <int RB, int KT>
LG_DEVINL void load_a(uint32_t base, int r0, int lane, uint32_t (&a)[KT][4]) {
  const int mat = lane >> 3, r = lane & 7;
#pragma unroll
  for (int ks = 0; ks < KT; ++ks) ldmatrix_x4(a[ks], taddr<RB>(base, r0 + r + 8 * (mat & 1), 2 * ks + (mat >> 1)));
}

// A fragments of the TRANSPOSE of a row-major [k][m] tile: rows m0..m0+15 of the transpose, KT k-steps
template <int RB, int KT>
LG_DEVINL void load_at(uint32_t base, int m0, int lane, uint32_t (&a)[KT][4]) {
  const int mat = lane >> 3, r = lane & 7;
#pragma unroll
  for (int ks = 0; ks < KT; ++ks) ldmatrix_x4_trans(a[ks], taddr<RB>(base, 16 * ks + 8 * (mat >> 1) + r, m0 / 8 + (mat & 1)));
}

// c[16 x 8 NT] += A B^T with B a row-major [n][k] tile, output columns n0 .. n0 + 8 NT - 1
template <int RB, int KT, int NT>
LG_DEVINL void mma_abt(const uint32_t (&a)[KT][4], uint32_t bbase, int n0, int lane, float (&c)[NT][4]) {
  const int mat = lane >> 3, r = lane & 7;
#pragma unroll
  for (int ks = 0; ks < KT; ++ks)
#pragma unroll
    for (int t = 0; t < NT; t += 2) {
      uint32_t b[4];
      ldmatrix_x4(b, taddr<RB>(bbase, n0 + 8 * (t + (mat >> 1)) + r, 2 * ks + (mat & 1)));
      const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
      mma_bf16_16816(c[t], a[ks], b0, c[t]);
      mma_bf16_16816(c[t + 1], a[ks], b1, c[t + 1]);
    }
}

// c[16 x 8 NT] += A B with B a row-major [k][n] tile, output columns 8 p0 .. 8 (p0 + NT) - 1
template <int RB, int KT, int NT>
LG_DEVINL void mma_ab(const uint32_t (&a)[KT][4], uint32_t bbase, int p0, int lane, float (&c)[NT][4]) {
  const int mat = lane >> 3, r = lane & 7;
#pragma unroll
  for (int ks = 0; ks < KT; ++ks)
#pragma unroll
    for (int j = 0; j < NT; j += 2) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, taddr<RB>(bbase, 16 * ks + 8 * (mat & 1) + r, p0 + j + (mat >> 1)));
      const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
      mma_bf16_16816(c[j], a[ks], b0, c[j]);
      mma_bf16_16816(c[j + 1], a[ks], b1, c[j + 1]);
    }
}

template <int NT>
LG_DEVINL void zero_acc(float (&c)[NT][4]) {
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) c[t][i] = 0.f;
}

struct Smem {
  float S32[KD][VW];                       // state slice, fp32
  float A32[CH][kAPitch];                  // strictly lower triangular coefficients, stored transposed: [j][i] = A[i][j]
  float U32[CH][VW];                       // U of the solve
  float cg[CH], gam[CH], bet[CH];
  __align__(128) __nv_bfloat16 Sb[KD * VW];      // state slice rounded to bf16, [k][v] rows of 128 B
  __align__(128) __nv_bfloat16 Kt[CH * KD];      // [token][k] rows of 256 B
  __align__(128) __nv_bfloat16 Qt[CH * KD];
  __align__(128) __nv_bfloat16 Wb[CH * KD];      // W of the solve, [token][k]
  __align__(128) __nv_bfloat16 Vt[CH * VW];      // [token][v] rows of 128 B
  __align__(128) __nv_bfloat16 Zt[CH * VW];
  __align__(128) __nv_bfloat16 Pb[CH * CH];      // tril((Q K^T) * decay), [token i][token j] rows of 128 B
  __align__(128) __nv_bfloat16 dVb[CH * VW];     // dV, [token][v]
  __align__(128) __nv_bfloat16 dVs[CH * VW];     // dV * exp(c_64 - c_i)
  __align__(128) __nv_bfloat16 Ks[CH * KD];      // beta gamma K, [token][k]
  __align__(128) __nv_bfloat16 Vs[CH * VW];      // beta V, [token][v]
  __align__(128) __nv_bfloat16 Tb[CH * CH];      // (I + A)^-1 rounded to bf16, [i][j] rows of 128 B
};

__global__ void __launch_bounds__(kThreads, 1)
gdn_chunk_kernel(float* __restrict__ state, const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                 const __nv_bfloat16* __restrict__ v, const float* __restrict__ g, const float* __restrict__ beta,
                 __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ z, const int* __restrict__ cu,
                 const int* __restrict__ slots, const uint8_t* __restrict__ fresh, int heads, int64_t qkv_stride, float scale) {
  lg::pdl_prologue();
  extern __shared__ uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>(smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u));
  const int part = blockIdx.x & 1, sh = blockIdx.x >> 1;
  const int seq = sh / heads, head = sh % heads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int fg = lane >> 2, fc = lane & 3;  // fragment row (and +8) and column pair inside an 8-wide tile
  const int t0 = cu[seq], t1 = cu[seq + 1];
  if (t1 <= t0) return;
  const int64_t slot = slots ? slots[seq] : seq;
  float* gstate = state + (slot * heads + head) * (int64_t)(KD * VDIM) + part * VW;
  const bool zero_start = fresh && fresh[seq];
  const uint32_t Sb_a = smem_u32(sm.Sb), Kt_a = smem_u32(sm.Kt), Qt_a = smem_u32(sm.Qt), Wb_a = smem_u32(sm.Wb), Vt_a = smem_u32(sm.Vt),
                 Zt_a = smem_u32(sm.Zt), Pb_a = smem_u32(sm.Pb), dVb_a = smem_u32(sm.dVb), dVs_a = smem_u32(sm.dVs), Ks_a = smem_u32(sm.Ks),
                 Vs_a = smem_u32(sm.Vs), Tb_a = smem_u32(sm.Tb);
  auto bf16_at = [&](__nv_bfloat16* tile, uint32_t tile_a, int rb, int row, int col) -> __nv_bfloat16* {
    // generic pointer to element (row, col) of a swizzled tile with rb bytes per row
    const uint32_t off = (uint32_t)row * rb + (uint32_t)((((col >> 3) ^ (row & 7)) << 4) + (col & 7) * 2);
    (void)tile_a;
    return reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(tile) + off);
  };

  // incoming state slice -> fp32 and bf16 copies
  for (int i = tid; i < KD * VW / 4; i += kThreads) {
    const int row = i / (VW / 4), c4 = (i % (VW / 4)) * 4;
    const float4 x = zero_start ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(gstate + (int64_t)row * VDIM + c4);
    *reinterpret_cast<float4*>(&sm.S32[row][c4]) = x;
    uint2 pk;
    pk.x = pack_bf16x2(x.x, x.y);
    pk.y = pack_bf16x2(x.z, x.w);
    *reinterpret_cast<uint2*>(bf16_at(sm.Sb, Sb_a, 128, row, c4)) = pk;
  }

  const int n_chunks = (t1 - t0 + CH - 1) / CH;
  for (int c = 0; c < n_chunks; ++c) {
    const int tb = t0 + c * CH;
    const int n = min(CH, t1 - tb);
    __syncthreads();  // previous chunk fully consumed (and, for c == 0, the state copies written)
    // ---- stage 1: the chunk's rows; rows >= n are zero (they then contribute nothing anywhere)
    for (int i = tid; i < CH * 16; i += kThreads) {
      const int row = i >> 4, piece = i & 15;
      const uint32_t dk = taddr<256>(Kt_a, row, piece), dq = taddr<256>(Qt_a, row, piece);
      if (row < n) {
        const int64_t src = (int64_t)(tb + row) * qkv_stride + head * KD + piece * 8;
        cp_async16(dk, k + src);
        cp_async16(dq, q + src);
      } else {
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sm.Kt) + (dk - Kt_a)) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sm.Qt) + (dq - Qt_a)) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    for (int i = tid; i < CH * 8; i += kThreads) {
      const int row = i >> 3, piece = i & 7;
      const uint32_t dv = taddr<128>(Vt_a, row, piece), dz = taddr<128>(Zt_a, row, piece);
      if (row < n) {
        const int64_t src = (int64_t)(tb + row) * qkv_stride + head * KD + part * VW + piece * 8;
        cp_async16(dv, v + src);
        if (z) cp_async16(dz, z + src);
      } else {
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sm.Vt) + (dv - Vt_a)) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    if (tid < CH) {
      const bool ok = tid < n;
      sm.cg[tid] = ok ? g[(int64_t)(tb + tid) * heads + head] : 0.f;      // raw g for now
      sm.bet[tid] = ok ? beta[(int64_t)(tb + tid) * heads + head] : 0.f;
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    // ---- stage 2: cumulative log-decay (inclusive) and its exponential
    if (warp == 0) {
      float a = sm.cg[lane], b = sm.cg[lane + 32];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const float ua = __shfl_up_sync(0xffffffffu, a, d), ub = __shfl_up_sync(0xffffffffu, b, d);
        if (lane >= d) { a += ua; b += ub; }
      }
      b += __shfl_sync(0xffffffffu, a, 31);
      sm.cg[lane] = a; sm.cg[lane + 32] = b;
      sm.gam[lane] = expf(a); sm.gam[lane + 32] = expf(b);
    }
    __syncthreads();
    // ---- stage 3: A = strict_tril(beta_i (k_i . k_j) exp(c_i - c_j)) (warps 0-3), P = tril((q_i . k_j) exp(c_i - c_j)) (warps 4-7)
    {
      const int r0 = (warp & 3) * 16;
      uint32_t af[KD / 16][4];
      load_a<256, KD / 16>(warp < 4 ? Kt_a : Qt_a, r0, lane, af);
      float s[CH / 8][4];
      zero_acc(s);
      mma_abt<256, KD / 16, CH / 8>(af, Kt_a, 0, lane, s);
      const int i0 = r0 + fg, i1 = i0 + 8;
      const float ci0 = sm.cg[i0], ci1 = sm.cg[i1];
      if (warp < 4) {
        const float b0 = sm.bet[i0], b1 = sm.bet[i1];
#pragma unroll
        for (int t = 0; t < CH / 8; ++t) {
          const int j0 = 8 * t + 2 * fc, j1 = j0 + 1;
          const float cj0 = sm.cg[j0], cj1 = sm.cg[j1];
          // stored transposed (At[j][i] = A[i][j]): the inverse below walks A by columns
          sm.A32[j0][i0] = i0 > j0 ? b0 * s[t][0] * __expf(ci0 - cj0) : 0.f;
          sm.A32[j1][i0] = i0 > j1 ? b0 * s[t][1] * __expf(ci0 - cj1) : 0.f;
          sm.A32[j0][i1] = i1 > j0 ? b1 * s[t][2] * __expf(ci1 - cj0) : 0.f;
          sm.A32[j1][i1] = i1 > j1 ? b1 * s[t][3] * __expf(ci1 - cj1) : 0.f;
        }
      } else {
#pragma unroll
        for (int t = 0; t < CH / 8; ++t) {
          const int j0 = 8 * t + 2 * fc, j1 = j0 + 1;
          const float cj0 = sm.cg[j0], cj1 = sm.cg[j1];
          const float p00 = i0 >= j0 ? s[t][0] * __expf(ci0 - cj0) : 0.f, p01 = i0 >= j1 ? s[t][1] * __expf(ci0 - cj1) : 0.f;
          const float p10 = i1 >= j0 ? s[t][2] * __expf(ci1 - cj0) : 0.f, p11 = i1 >= j1 ? s[t][3] * __expf(ci1 - cj1) : 0.f;
          *reinterpret_cast<uint32_t*>(bf16_at(sm.Pb, Pb_a, 128, i0, j0)) = pack_bf16x2(p00, p01);
          *reinterpret_cast<uint32_t*>(bf16_at(sm.Pb, Pb_a, 128, i1, j0)) = pack_bf16x2(p10, p11);
        }
      }
    }
    __syncthreads();
    // ---- stage 4a: scale the right-hand sides (Ks = beta gamma K, Vs = beta V), then T = (I + A)^-1 by
    // forward substitution: four neighbouring lanes per column, rows dealt round-robin (row i to lane
    // i % 4), right-looking: the owner of row j broadcasts x_j with one shuffle and every lane takes that
    // term out of its later rows at once, so the updates of a step are independent of each other; the
    // coefficients of step j + 1 are fetched before the shuffle of step j. (Measured: this stage takes
    // about 7500 cycles per chunk however the 64 x 64 substitution is spread over threads - one, two or
    // four lanes per column, unrolled or looped - and is a third of the kernel.)
    for (int e = tid; e < CH * (KD / 8); e += kThreads) {  // 16-byte pieces of K
      const int row = e / (KD / 8), piece = e % (KD / 8);
      const float f = sm.bet[row] * sm.gam[row];
      const uint4 in = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(sm.Kt) + (taddr<256>(Kt_a, row, piece) - Kt_a));
      uint4 out;
      float2 t;
      t = unpack_bf16x2(in.x); out.x = pack_bf16x2(t.x * f, t.y * f);
      t = unpack_bf16x2(in.y); out.y = pack_bf16x2(t.x * f, t.y * f);
      t = unpack_bf16x2(in.z); out.z = pack_bf16x2(t.x * f, t.y * f);
      t = unpack_bf16x2(in.w); out.w = pack_bf16x2(t.x * f, t.y * f);
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sm.Ks) + (taddr<256>(Ks_a, row, piece) - Ks_a)) = out;
    }
    for (int e = tid; e < CH * (VW / 8); e += kThreads) {  // 16-byte pieces of V
      const int row = e / (VW / 8), piece = e % (VW / 8);
      const float f = sm.bet[row];
      const uint4 in = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(sm.Vt) + (taddr<128>(Vt_a, row, piece) - Vt_a));
      uint4 out;
      float2 t;
      t = unpack_bf16x2(in.x); out.x = pack_bf16x2(t.x * f, t.y * f);
      t = unpack_bf16x2(in.y); out.y = pack_bf16x2(t.x * f, t.y * f);
      t = unpack_bf16x2(in.z); out.z = pack_bf16x2(t.x * f, t.y * f);
      t = unpack_bf16x2(in.w); out.w = pack_bf16x2(t.x * f, t.y * f);
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sm.Vs) + (taddr<128>(Vs_a, row, piece) - Vs_a)) = out;
    }
    {
      const int col = tid >> 2, part = tid & 3;
      float acc[CH / 4];  // acc[m] is row 4 m + part of column `col`
#pragma unroll
      for (int m = 0; m < CH / 4; ++m) acc[m] = (4 * m + part) == col ? 1.f : 0.f;
      float a_cur[CH / 4];
#pragma unroll
      for (int m = 0; m < CH / 4; ++m) a_cur[m] = sm.A32[0][4 * m + part];
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        float a_nxt[CH / 4];
#pragma unroll
        for (int m = 0; m < CH / 4; ++m) a_nxt[m] = (j + 1 < CH && m >= ((j + 1) >> 2)) ? sm.A32[(j + 1) % CH][4 * m + part] : 0.f;
        const float xj = __shfl_sync(0xffffffffu, acc[j >> 2], (lane & ~3) | (j & 3));
        if (part == (j & 3)) *bf16_at(sm.Tb, Tb_a, 128, j, col) = __float2bfloat16(xj);
#pragma unroll
        for (int m = j >> 2; m < CH / 4; ++m) acc[m] -= a_cur[m] * xj;  // A[i][j], zero where i <= j
#pragma unroll
        for (int m = 0; m < CH / 4; ++m) a_cur[m] = a_nxt[m];
      }
    }
    __syncthreads();
    // ---- stage 4b: W = T Ks (bf16, the row operand of stage 5), U = T Vs (fp32)  (warp: 16 rows x half of the columns)
    {
      const int rr = (warp & 3) * 16, hh = warp >> 2;
      uint32_t tf[CH / 16][4];
      load_a<128, CH / 16>(Tb_a, rr, lane, tf);
      float wacc[8][4];
      zero_acc(wacc);
      mma_ab<256, CH / 16, 8>(tf, Ks_a, hh * 8, lane, wacc);
      float uacc[4][4];
      zero_acc(uacc);
      mma_ab<128, CH / 16, 4>(tf, Vs_a, hh * 4, lane, uacc);
      const int i0 = rr + fg, i1 = i0 + 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int col = 8 * (hh * 8 + j) + 2 * fc;
        *reinterpret_cast<uint32_t*>(bf16_at(sm.Wb, Wb_a, 256, i0, col)) = pack_bf16x2(wacc[j][0], wacc[j][1]);
        *reinterpret_cast<uint32_t*>(bf16_at(sm.Wb, Wb_a, 256, i1, col)) = pack_bf16x2(wacc[j][2], wacc[j][3]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = 8 * (hh * 4 + j) + 2 * fc;
        *reinterpret_cast<float2*>(&sm.U32[i0][col]) = make_float2(uacc[j][0], uacc[j][1]);
        *reinterpret_cast<float2*>(&sm.U32[i1][col]) = make_float2(uacc[j][2], uacc[j][3]);
      }
    }
    __syncthreads();
    // ---- stage 5: dV = U - W S  (warp: 16 token rows x 32 value columns)
    const int r0 = (warp & 3) * 16, p0 = (warp >> 2) * 4;  // p0: first 8-column tile of this warp's 32 columns
    {
      uint32_t wf[KD / 16][4];
      load_a<256, KD / 16>(Wb_a, r0, lane, wf);
      float acc[4][4];
      zero_acc(acc);
      mma_ab<128, KD / 16, 4>(wf, Sb_a, p0, lane, acc);
      const int i0 = r0 + fg, i1 = i0 + 8;
      const float cl = sm.cg[CH - 1];
      const float e0 = expf(cl - sm.cg[i0]), e1 = expf(cl - sm.cg[i1]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = 8 * (p0 + j) + 2 * fc;
        const float d00 = sm.U32[i0][col] - acc[j][0], d01 = sm.U32[i0][col + 1] - acc[j][1];
        const float d10 = sm.U32[i1][col] - acc[j][2], d11 = sm.U32[i1][col + 1] - acc[j][3];
        *reinterpret_cast<uint32_t*>(bf16_at(sm.dVb, dVb_a, 128, i0, col)) = pack_bf16x2(d00, d01);
        *reinterpret_cast<uint32_t*>(bf16_at(sm.dVb, dVb_a, 128, i1, col)) = pack_bf16x2(d10, d11);
        *reinterpret_cast<uint32_t*>(bf16_at(sm.dVs, dVs_a, 128, i0, col)) = pack_bf16x2(d00 * e0, d01 * e0);
        *reinterpret_cast<uint32_t*>(bf16_at(sm.dVs, dVs_a, 128, i1, col)) = pack_bf16x2(d10 * e1, d11 * e1);
      }
    }
    __syncthreads();
    // ---- stage 6: O = scale (gamma_i (Q S) + P dV), output gate, store
    {
      uint32_t qf[KD / 16][4];
      load_a<256, KD / 16>(Qt_a, r0, lane, qf);
      float acc[4][4];
      zero_acc(acc);
      mma_ab<128, KD / 16, 4>(qf, Sb_a, p0, lane, acc);
      const int i0 = r0 + fg, i1 = i0 + 8;
      const float g0 = sm.gam[i0], g1 = sm.gam[i1];
#pragma unroll
      for (int j = 0; j < 4; ++j) { acc[j][0] *= g0; acc[j][1] *= g0; acc[j][2] *= g1; acc[j][3] *= g1; }
      uint32_t pf[CH / 16][4];
      load_a<128, CH / 16>(Pb_a, r0, lane, pf);
      mma_ab<128, CH / 16, 4>(pf, dVb_a, p0, lane, acc);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = 8 * (p0 + j) + 2 * fc;
        float o00 = acc[j][0] * scale, o01 = acc[j][1] * scale, o10 = acc[j][2] * scale, o11 = acc[j][3] * scale;
        if (z) {
          const float2 z0 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(bf16_at(sm.Zt, Zt_a, 128, i0, col)));
          const float2 z1 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(bf16_at(sm.Zt, Zt_a, 128, i1, col)));
          o00 *= z0.x / (1.0f + __expf(-z0.x)); o01 *= z0.y / (1.0f + __expf(-z0.y));
          o10 *= z1.x / (1.0f + __expf(-z1.x)); o11 *= z1.y / (1.0f + __expf(-z1.y));
        }
        const int64_t ocol = (int64_t)head * VDIM + part * VW + col;
        if (i0 < n) *reinterpret_cast<uint32_t*>(o + (int64_t)(tb + i0) * heads * VDIM + ocol) = pack_bf16x2(o00, o01);
        if (i1 < n) *reinterpret_cast<uint32_t*>(o + (int64_t)(tb + i1) * heads * VDIM + ocol) = pack_bf16x2(o10, o11);
      }
    }
    __syncthreads();  // every read of Sb for this chunk is done before it changes
    // ---- stage 7: S = gamma_64 S + K^T (dV exp(c_64 - c_i))  (warp: 16 key rows x all 64 value columns)
    {
      const int m0 = warp * 16;
      uint32_t kf[CH / 16][4];
      load_at<256, CH / 16>(Kt_a, m0, lane, kf);
      float acc[VW / 8][4];
      zero_acc(acc);
      mma_ab<128, CH / 16, VW / 8>(kf, dVs_a, 0, lane, acc);
      const float gl = sm.gam[CH - 1];
      const int k0 = m0 + fg, k1 = k0 + 8;
#pragma unroll
      for (int j = 0; j < VW / 8; ++j) {
        const int col = 8 * j + 2 * fc;
        float2 s0 = *reinterpret_cast<float2*>(&sm.S32[k0][col]), s1 = *reinterpret_cast<float2*>(&sm.S32[k1][col]);
        s0.x = gl * s0.x + acc[j][0]; s0.y = gl * s0.y + acc[j][1];
        s1.x = gl * s1.x + acc[j][2]; s1.y = gl * s1.y + acc[j][3];
        *reinterpret_cast<float2*>(&sm.S32[k0][col]) = s0;
        *reinterpret_cast<float2*>(&sm.S32[k1][col]) = s1;
        *reinterpret_cast<uint32_t*>(bf16_at(sm.Sb, Sb_a, 128, k0, col)) = pack_bf16x2(s0.x, s0.y);
        *reinterpret_cast<uint32_t*>(bf16_at(sm.Sb, Sb_a, 128, k1, col)) = pack_bf16x2(s1.x, s1.y);
      }
    }
  }
  __syncthreads();
  for (int i = tid; i < KD * VW / 4; i += kThreads) {
    const int row = i / (VW / 4), c4 = (i % (VW / 4)) * 4;
    *reinterpret_cast<float4*>(gstate + (int64_t)row * VDIM + c4) = *reinterpret_cast<const float4*>(&sm.S32[row][c4]);
  }
}


// ---------------------------------------------------------------------------------------------------
// The same function as two launches. Everything in a chunk that does not involve the carried state
// (the coefficient matrix, its inverse, W, U, the masked Q K^T) is independent from chunk to chunk, so
// gdn_chunk_intra_kernel computes it for ALL chunks of all sequences at once (one CTA per chunk and
// head, the whole GPU busy whatever the number of sequences) and leaves it in a scratch buffer;
// gdn_chunk_state_kernel then walks each sequence's chunks in order with only the three products that
// touch the state (dV = U - W S, O, S'), its operands prefetched one chunk ahead. For one long prompt
// the serial chain per chunk shrinks to about a third.
//
// Scratch slot of (chunk, head), kSlotBytes each, chunks numbered over the batch in sequence order:
//   W   bf16 [64][128]  the shared-memory image of the tile (16-byte pieces swizzled by row)   16384 B
//   P   bf16 [64][64]   likewise                                                               8192 B
//   U   f32  [2][64][64] value-column halves                                                  32768 B
//   cg  f32  [64], gam f32 [64]                                                                 512 B
constexpr int kOffW = 0, kOffP = 16384, kOffU = 24576, kOffC = 57344, kSlotBytes = 57856;

// (sequence, chunk inside it, first chunk of the sequence in batch order) of batch chunk `gc`, or seq = -1.
// Warp 0 calls it; the result is the same in every lane.
LG_DEVINL void find_chunk(const int* __restrict__ cu, int n_seqs, int gc, int lane, int& seq, int& local, int& base) {
  seq = -1; local = 0; base = 0;
  int acc = 0;
  for (int s0 = 0; s0 < n_seqs; s0 += 32) {
    const int s = s0 + lane;
    const int nc = s < n_seqs ? (max(cu[s + 1] - cu[s], 0) + CH - 1) / CH : 0;
    int incl = nc;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += u;
    }
    const bool mine = nc > 0 && gc >= acc + incl - nc && gc < acc + incl;
    const uint32_t hit = __ballot_sync(0xffffffffu, mine);
    if (hit) {
      const int src = __ffs(hit) - 1;
      const int b = __shfl_sync(0xffffffffu, acc + incl - nc, src);
      seq = s0 + src; base = b; local = gc - b;
      return;
    }
    acc += __shfl_sync(0xffffffffu, incl, 31);
  }
}

// first batch chunk of sequence `seq` (warp 0; same result in every lane)
LG_DEVINL int chunk_base(const int* __restrict__ cu, int seq, int lane) {
  int acc = 0;
  for (int s0 = 0; s0 < seq; s0 += 32) {
    const int s = s0 + lane;
    int nc = s < seq ? (max(cu[s + 1] - cu[s], 0) + CH - 1) / CH : 0;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) nc += __shfl_xor_sync(0xffffffffu, nc, d);
    acc += nc;
  }
  return acc;
}

struct IntraSmem {
  float A32[CH][kAPitch];
  float cg[CH], gam[CH], bet[CH];
  int where[4];
  __align__(128) __nv_bfloat16 Kt[CH * KD];      // [token][k] rows of 256 B; scaled in place to beta gamma K
  __align__(128) __nv_bfloat16 Qt[CH * KD];
  __align__(128) __nv_bfloat16 Vt[CH * VDIM];    // [token][v] rows of 256 B; scaled in place to beta V
  __align__(128) __nv_bfloat16 Tb[CH * CH];
};

__global__ void __launch_bounds__(kThreads, 2)
gdn_chunk_intra_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                       const float* __restrict__ g, const float* __restrict__ beta, const int* __restrict__ cu, int n_seqs, int heads,
                       int64_t qkv_stride, uint8_t* __restrict__ scratch) {
  lg::pdl_prologue();
  extern __shared__ uint8_t smem_raw[];
  IntraSmem& sm = *reinterpret_cast<IntraSmem*>(smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int fg = lane >> 2, fc = lane & 3;
  const int head = blockIdx.y;
  if (warp == 0) {
    int seq, local, base;
    find_chunk(cu, n_seqs, (int)blockIdx.x, lane, seq, local, base);
    if (lane == 0) { sm.where[0] = seq; sm.where[1] = local; }
  }
  __syncthreads();
  const int seq = sm.where[0];
  if (seq < 0) return;  // beyond the batch's last chunk
  const int tb = cu[seq] + sm.where[1] * CH;
  const int n = min(CH, cu[seq + 1] - tb);
  uint8_t* slot = scratch + ((size_t)blockIdx.x * heads + head) * kSlotBytes;
  const uint32_t Kt_a = smem_u32(sm.Kt), Qt_a = smem_u32(sm.Qt), Vt_a = smem_u32(sm.Vt), Tb_a = smem_u32(sm.Tb);
  auto tile_off = [](int rb, int row, int col) -> uint32_t {  // byte offset of element (row, col) in a swizzled tile
    return (uint32_t)row * rb + (uint32_t)((((col >> 3) ^ (row & 7)) << 4) + (col & 7) * 2);
  };
  // ---- the chunk's rows; rows >= n are zero (they then contribute nothing anywhere)
  for (int i = tid; i < CH * 16; i += kThreads) {
    const int row = i >> 4, piece = i & 15;
    const uint32_t off = taddr<256>(0u, row, piece);
    if (row < n) {
      const int64_t src = (int64_t)(tb + row) * qkv_stride + head * KD + piece * 8;
      cp_async16(Kt_a + off, k + src);
      cp_async16(Qt_a + off, q + src);
      cp_async16(Vt_a + off, v + src);
    } else {
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sm.Kt) + off) = make_uint4(0u, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sm.Qt) + off) = make_uint4(0u, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sm.Vt) + off) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  if (tid < CH) {
    const bool ok = tid < n;
    sm.cg[tid] = ok ? g[(int64_t)(tb + tid) * heads + head] : 0.f;
    sm.bet[tid] = ok ? beta[(int64_t)(tb + tid) * heads + head] : 0.f;
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  // ---- cumulative log-decay (inclusive) and its exponential
  if (warp == 0) {
    float a = sm.cg[lane], b = sm.cg[lane + 32];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float ua = __shfl_up_sync(0xffffffffu, a, d), ub = __shfl_up_sync(0xffffffffu, b, d);
      if (lane >= d) { a += ua; b += ub; }
    }
    b += __shfl_sync(0xffffffffu, a, 31);
    sm.cg[lane] = a; sm.cg[lane + 32] = b;
    sm.gam[lane] = expf(a); sm.gam[lane + 32] = expf(b);
  }
  __syncthreads();
  if (tid < CH) {
    float* cgo = reinterpret_cast<float*>(slot + kOffC);
    cgo[tid] = sm.cg[tid];
    cgo[CH + tid] = sm.gam[tid];
  }
  // ---- A = strict_tril(beta_i (k_i . k_j) exp(c_i - c_j)) (warps 0-3), P = tril((q_i . k_j) exp(c_i - c_j)) (warps 4-7, to the slot)
  {
    const int r0 = (warp & 3) * 16;
    uint32_t af[KD / 16][4];
    load_a<256, KD / 16>(warp < 4 ? Kt_a : Qt_a, r0, lane, af);
    float s[CH / 8][4];
    zero_acc(s);
    mma_abt<256, KD / 16, CH / 8>(af, Kt_a, 0, lane, s);
    const int i0 = r0 + fg, i1 = i0 + 8;
    const float ci0 = sm.cg[i0], ci1 = sm.cg[i1];
    if (warp < 4) {
      const float b0 = sm.bet[i0], b1 = sm.bet[i1];
#pragma unroll
      for (int t = 0; t < CH / 8; ++t) {
        const int j0 = 8 * t + 2 * fc, j1 = j0 + 1;
        const float cj0 = sm.cg[j0], cj1 = sm.cg[j1];
        sm.A32[j0][i0] = i0 > j0 ? b0 * s[t][0] * __expf(ci0 - cj0) : 0.f;
        sm.A32[j1][i0] = i0 > j1 ? b0 * s[t][1] * __expf(ci0 - cj1) : 0.f;
        sm.A32[j0][i1] = i1 > j0 ? b1 * s[t][2] * __expf(ci1 - cj0) : 0.f;
        sm.A32[j1][i1] = i1 > j1 ? b1 * s[t][3] * __expf(ci1 - cj1) : 0.f;
      }
    } else {
      uint8_t* pg = slot + kOffP;
#pragma unroll
      for (int t = 0; t < CH / 8; ++t) {
        const int j0 = 8 * t + 2 * fc, j1 = j0 + 1;
        const float cj0 = sm.cg[j0], cj1 = sm.cg[j1];
        const float p00 = i0 >= j0 ? s[t][0] * __expf(ci0 - cj0) : 0.f, p01 = i0 >= j1 ? s[t][1] * __expf(ci0 - cj1) : 0.f;
        const float p10 = i1 >= j0 ? s[t][2] * __expf(ci1 - cj0) : 0.f, p11 = i1 >= j1 ? s[t][3] * __expf(ci1 - cj1) : 0.f;
        *reinterpret_cast<uint32_t*>(pg + tile_off(128, i0, j0)) = pack_bf16x2(p00, p01);
        *reinterpret_cast<uint32_t*>(pg + tile_off(128, i1, j0)) = pack_bf16x2(p10, p11);
      }
    }
  }
  __syncthreads();
  // ---- right-hand sides in place (K <- beta gamma K, V <- beta V), then T = (I + A)^-1 by forward
  // substitution (see the one-launch kernel above for the scheme)
  for (int e = tid; e < CH * 16; e += kThreads) {
    const int row = e >> 4, piece = e & 15;
    const uint32_t off = taddr<256>(0u, row, piece);
    const float fk = sm.bet[row] * sm.gam[row], fv = sm.bet[row];
    uint4* pk = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sm.Kt) + off);
    uint4* pv = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sm.Vt) + off);
    uint4 x = *pk, y = *pv;
    float2 t;
    t = unpack_bf16x2(x.x); x.x = pack_bf16x2(t.x * fk, t.y * fk);
    t = unpack_bf16x2(x.y); x.y = pack_bf16x2(t.x * fk, t.y * fk);
    t = unpack_bf16x2(x.z); x.z = pack_bf16x2(t.x * fk, t.y * fk);
    t = unpack_bf16x2(x.w); x.w = pack_bf16x2(t.x * fk, t.y * fk);
    t = unpack_bf16x2(y.x); y.x = pack_bf16x2(t.x * fv, t.y * fv);
    t = unpack_bf16x2(y.y); y.y = pack_bf16x2(t.x * fv, t.y * fv);
    t = unpack_bf16x2(y.z); y.z = pack_bf16x2(t.x * fv, t.y * fv);
    t = unpack_bf16x2(y.w); y.w = pack_bf16x2(t.x * fv, t.y * fv);
    *pk = x; *pv = y;
  }
  {
    const int col = tid >> 2, part = tid & 3;
    float acc[CH / 4];  // acc[m] is row 4 m + part of column `col`
#pragma unroll
    for (int m = 0; m < CH / 4; ++m) acc[m] = (4 * m + part) == col ? 1.f : 0.f;
    float a_cur[CH / 4];
#pragma unroll
    for (int m = 0; m < CH / 4; ++m) a_cur[m] = sm.A32[0][4 * m + part];
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      float a_nxt[CH / 4];
#pragma unroll
      for (int m = 0; m < CH / 4; ++m) a_nxt[m] = (j + 1 < CH && m >= ((j + 1) >> 2)) ? sm.A32[(j + 1) % CH][4 * m + part] : 0.f;
      const float xj = __shfl_sync(0xffffffffu, acc[j >> 2], (lane & ~3) | (j & 3));
      if (part == (j & 3)) *reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(sm.Tb) + tile_off(128, j, col)) = __float2bfloat16(xj);
#pragma unroll
      for (int m = j >> 2; m < CH / 4; ++m) acc[m] -= a_cur[m] * xj;
#pragma unroll
      for (int m = 0; m < CH / 4; ++m) a_cur[m] = a_nxt[m];
    }
  }
  __syncthreads();
  // ---- W = T (beta gamma K) (bf16 image), U = T (beta V) (fp32, by value-column half): straight to the slot
  {
    const int rr = (warp & 3) * 16, hh = warp >> 2;
    uint32_t tf[CH / 16][4];
    load_a<128, CH / 16>(Tb_a, rr, lane, tf);
    const int i0 = rr + fg, i1 = i0 + 8;
    {
      float wacc[8][4];
      zero_acc(wacc);
      mma_ab<256, CH / 16, 8>(tf, Kt_a, hh * 8, lane, wacc);
      uint8_t* wg = slot + kOffW;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int col = 8 * (hh * 8 + j) + 2 * fc;
        *reinterpret_cast<uint32_t*>(wg + tile_off(256, i0, col)) = pack_bf16x2(wacc[j][0], wacc[j][1]);
        *reinterpret_cast<uint32_t*>(wg + tile_off(256, i1, col)) = pack_bf16x2(wacc[j][2], wacc[j][3]);
      }
    }
    {
      float uacc[8][4];
      zero_acc(uacc);
      mma_ab<256, CH / 16, 8>(tf, Vt_a, hh * 8, lane, uacc);
      float* ug = reinterpret_cast<float*>(slot + kOffU) + hh * (CH * VW);  // this warp's columns are value half hh
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int col = 8 * j + 2 * fc;
        *reinterpret_cast<float2*>(ug + i0 * VW + col) = make_float2(uacc[j][0], uacc[j][1]);
        *reinterpret_cast<float2*>(ug + i1 * VW + col) = make_float2(uacc[j][2], uacc[j][3]);
      }
    }
  }
}

struct StateBuf {  // one chunk's operands as they arrive
  float U32[CH][VW];
  float cg[CH], gam[CH];
  __align__(128) __nv_bfloat16 Wb[CH * KD];
  __align__(128) __nv_bfloat16 Pb[CH * CH];
  __align__(128) __nv_bfloat16 Qt[CH * KD];
  __align__(128) __nv_bfloat16 Kt[CH * KD];
  __align__(128) __nv_bfloat16 Zt[CH * VW];
};

struct StateSmem {
  float S32[KD][VW];
  __align__(128) __nv_bfloat16 Sb[KD * VW];
  __align__(128) __nv_bfloat16 dVb[CH * VW];
  __align__(128) __nv_bfloat16 dVs[CH * VW];
  __align__(128) StateBuf buf[2];
  int base;
};

__global__ void __launch_bounds__(kThreads, 1)
gdn_chunk_state_kernel(float* __restrict__ state, const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                       __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ z, const int* __restrict__ cu,
                       const int* __restrict__ slots, const uint8_t* __restrict__ fresh, int heads, int64_t qkv_stride, float scale,
                       const uint8_t* __restrict__ scratch) {
  lg::pdl_prologue();
  extern __shared__ uint8_t smem_raw[];
  StateSmem& sm = *reinterpret_cast<StateSmem*>(smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u));
  const int part = blockIdx.x & 1, sh = blockIdx.x >> 1;
  const int seq = sh / heads, head = sh % heads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int fg = lane >> 2, fc = lane & 3;
  const int t0 = cu[seq], t1 = cu[seq + 1];
  if (t1 <= t0) return;
  if (warp == 0) {
    const int b = chunk_base(cu, seq, lane);
    if (lane == 0) sm.base = b;
  }
  const int64_t slot_id = slots ? slots[seq] : seq;
  float* gstate = state + (slot_id * heads + head) * (int64_t)(KD * VDIM) + part * VW;
  const bool zero_start = fresh && fresh[seq];
  const uint32_t Sb_a = smem_u32(sm.Sb), dVb_a = smem_u32(sm.dVb), dVs_a = smem_u32(sm.dVs);
  auto tile_off = [](int rb, int row, int col) -> uint32_t {
    return (uint32_t)row * rb + (uint32_t)((((col >> 3) ^ (row & 7)) << 4) + (col & 7) * 2);
  };
  for (int i = tid; i < KD * VW / 4; i += kThreads) {
    const int row = i / (VW / 4), c4 = (i % (VW / 4)) * 4;
    const float4 x = zero_start ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(gstate + (int64_t)row * VDIM + c4);
    *reinterpret_cast<float4*>(&sm.S32[row][c4]) = x;
    uint2 pk;
    pk.x = pack_bf16x2(x.x, x.y);
    pk.y = pack_bf16x2(x.z, x.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(sm.Sb) + tile_off(128, row, c4)) = pk;
  }
  __syncthreads();
  const int base = sm.base;
  const int n_chunks = (t1 - t0 + CH - 1) / CH;
  // requests chunk c's operands into buffer b: the slot's W, P, U half and decays are plain copies (the
  // slot holds shared-memory images), the q, k, z rows are swizzled as they land; rows >= n are zero
  auto fetch = [&](int c, int b) {
    StateBuf& B = sm.buf[b];
    const uint8_t* slot = scratch + ((size_t)(base + c) * heads + head) * kSlotBytes;
    const int tb = t0 + c * CH;
    const int n = min(CH, t1 - tb);
    const uint32_t Wb_a = smem_u32(B.Wb), Pb_a = smem_u32(B.Pb), U_a = smem_u32(B.U32), C_a = smem_u32(B.cg), Qt_a = smem_u32(B.Qt),
                   Kt_a = smem_u32(B.Kt), Zt_a = smem_u32(B.Zt);
    for (int i = tid; i < 1024; i += kThreads) {
      cp_async16(Wb_a + i * 16, slot + kOffW + i * 16);
      cp_async16(U_a + i * 16, slot + kOffU + part * (CH * VW * 4) + i * 16);
    }
    for (int i = tid; i < 512; i += kThreads) cp_async16(Pb_a + i * 16, slot + kOffP + i * 16);
    if (tid < 32) cp_async16(C_a + tid * 16, slot + kOffC + tid * 16);  // cg and gam are adjacent in both places
    for (int i = tid; i < CH * 16; i += kThreads) {
      const int row = i >> 4, piece = i & 15;
      const uint32_t off = taddr<256>(0u, row, piece);
      if (row < n) {
        const int64_t src = (int64_t)(tb + row) * qkv_stride + head * KD + piece * 8;
        cp_async16(Kt_a + off, k + src);
        cp_async16(Qt_a + off, q + src);
      } else {
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(B.Kt) + off) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(B.Qt) + off) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    if (z) {
      for (int i = tid; i < CH * 8; i += kThreads) {
        const int row = i >> 3, piece = i & 7;
        if (row < n) cp_async16(Zt_a + taddr<128>(0u, row, piece), z + (int64_t)(tb + row) * qkv_stride + head * KD + part * VW + piece * 8);
      }
    }
    cp_async_commit();
  };
  fetch(0, 0);
  for (int c = 0; c < n_chunks; ++c) {
    const int b = c & 1;
    StateBuf& B = sm.buf[b];
    if (c + 1 < n_chunks) {
      fetch(c + 1, b ^ 1);  // that buffer's last readers passed the barrier that ended chunk c - 1
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int tb = t0 + c * CH;
    const int n = min(CH, t1 - tb);
    const uint32_t Wb_a = smem_u32(B.Wb), Pb_a = smem_u32(B.Pb), Qt_a = smem_u32(B.Qt), Kt_a = smem_u32(B.Kt);
    // ---- dV = U - W S  (warp: 16 token rows x 32 value columns)
    const int r0 = (warp & 3) * 16, p0 = (warp >> 2) * 4;
    {
      uint32_t wf[KD / 16][4];
      load_a<256, KD / 16>(Wb_a, r0, lane, wf);
      float acc[4][4];
      zero_acc(acc);
      mma_ab<128, KD / 16, 4>(wf, Sb_a, p0, lane, acc);
      const int i0 = r0 + fg, i1 = i0 + 8;
      const float cl = B.cg[CH - 1];
      const float e0 = expf(cl - B.cg[i0]), e1 = expf(cl - B.cg[i1]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = 8 * (p0 + j) + 2 * fc;
        const float d00 = B.U32[i0][col] - acc[j][0], d01 = B.U32[i0][col + 1] - acc[j][1];
        const float d10 = B.U32[i1][col] - acc[j][2], d11 = B.U32[i1][col + 1] - acc[j][3];
        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(sm.dVb) + tile_off(128, i0, col)) = pack_bf16x2(d00, d01);
        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(sm.dVb) + tile_off(128, i1, col)) = pack_bf16x2(d10, d11);
        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(sm.dVs) + tile_off(128, i0, col)) = pack_bf16x2(d00 * e0, d01 * e0);
        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(sm.dVs) + tile_off(128, i1, col)) = pack_bf16x2(d10 * e1, d11 * e1);
      }
    }
    __syncthreads();
    // ---- O = scale (gamma_i (Q S) + P dV), output gate, store
    {
      uint32_t qf[KD / 16][4];
      load_a<256, KD / 16>(Qt_a, r0, lane, qf);
      float acc[4][4];
      zero_acc(acc);
      mma_ab<128, KD / 16, 4>(qf, Sb_a, p0, lane, acc);
      const int i0 = r0 + fg, i1 = i0 + 8;
      const float g0 = B.gam[i0], g1 = B.gam[i1];
#pragma unroll
      for (int j = 0; j < 4; ++j) { acc[j][0] *= g0; acc[j][1] *= g0; acc[j][2] *= g1; acc[j][3] *= g1; }
      uint32_t pf[CH / 16][4];
      load_a<128, CH / 16>(Pb_a, r0, lane, pf);
      mma_ab<128, CH / 16, 4>(pf, dVb_a, p0, lane, acc);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = 8 * (p0 + j) + 2 * fc;
        float o00 = acc[j][0] * scale, o01 = acc[j][1] * scale, o10 = acc[j][2] * scale, o11 = acc[j][3] * scale;
        if (z) {
          if (i0 < n) {
            const float2 z0 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(B.Zt) + tile_off(128, i0, col)));
            o00 *= z0.x / (1.0f + __expf(-z0.x)); o01 *= z0.y / (1.0f + __expf(-z0.y));
          }
          if (i1 < n) {
            const float2 z1 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(B.Zt) + tile_off(128, i1, col)));
            o10 *= z1.x / (1.0f + __expf(-z1.x)); o11 *= z1.y / (1.0f + __expf(-z1.y));
          }
        }
        const int64_t ocol = (int64_t)head * VDIM + part * VW + col;
        if (i0 < n) *reinterpret_cast<uint32_t*>(o + (int64_t)(tb + i0) * heads * VDIM + ocol) = pack_bf16x2(o00, o01);
        if (i1 < n) *reinterpret_cast<uint32_t*>(o + (int64_t)(tb + i1) * heads * VDIM + ocol) = pack_bf16x2(o10, o11);
      }
    }
    __syncthreads();  // every read of Sb for this chunk is done before it changes
    // ---- S = gamma_64 S + K^T (dV exp(c_64 - c_i))  (warp: 16 key rows x all 64 value columns)
    {
      const int m0 = warp * 16;
      uint32_t kf[CH / 16][4];
      load_at<256, CH / 16>(Kt_a, m0, lane, kf);
      float acc[VW / 8][4];
      zero_acc(acc);
      mma_ab<128, CH / 16, VW / 8>(kf, dVs_a, 0, lane, acc);
      const float gl = B.gam[CH - 1];
      const int k0 = m0 + fg, k1 = k0 + 8;
#pragma unroll
      for (int j = 0; j < VW / 8; ++j) {
        const int col = 8 * j + 2 * fc;
        float2 s0 = *reinterpret_cast<float2*>(&sm.S32[k0][col]), s1 = *reinterpret_cast<float2*>(&sm.S32[k1][col]);
        s0.x = gl * s0.x + acc[j][0]; s0.y = gl * s0.y + acc[j][1];
        s1.x = gl * s1.x + acc[j][2]; s1.y = gl * s1.y + acc[j][3];
        *reinterpret_cast<float2*>(&sm.S32[k0][col]) = s0;
        *reinterpret_cast<float2*>(&sm.S32[k1][col]) = s1;
        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(sm.Sb) + tile_off(128, k0, col)) = pack_bf16x2(s0.x, s0.y);
        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(sm.Sb) + tile_off(128, k1, col)) = pack_bf16x2(s1.x, s1.y);
      }
    }
    __syncthreads();  // the chunk's buffer is free for the fetch after next; the state copies are complete
  }
  for (int i = tid; i < KD * VW / 4; i += kThreads) {
    const int row = i / (VW / 4), c4 = (i % (VW / 4)) * 4;
    *reinterpret_cast<float4*>(gstate + (int64_t)row * VDIM + c4) = *reinterpret_cast<const float4*>(&sm.S32[row][c4]);
  }
}

}  // namespace

extern "C" size_t logismos_gdn_chunked_scratch_bytes(int32_t n_tokens, int32_t n_seqs, int32_t heads) {
  if (n_tokens < 0 || n_seqs < 0 || heads <= 0) return 0;
  return ((size_t)n_tokens / CH + (size_t)n_seqs) * (size_t)heads * kSlotBytes;  // every sequence may end in a partial chunk
}

extern "C" uint32_t logismos_launch_gdn_chunked(void* state, const void* q, const void* k, const void* v, const void* g,
                                                const void* beta, void* o, const void* gate_z, const void* cu_seqlens,
                                                const void* state_slots, const void* fresh, int32_t n_seqs, int32_t heads,
                                                int32_t qkv_stride, float scale, void* scratch, int32_t n_tokens, void* stream) {
  lg::LaunchScope launch_scope_;
  if (n_seqs < 0 || heads <= 0 || qkv_stride < heads * KD || (qkv_stride % 8)) return lg::kInvalidValue;
  if (n_seqs == 0) return 0;
  if (((uintptr_t)state & 15) || ((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15) || ((uintptr_t)gate_z & 15) ||
      ((uintptr_t)o & 3))
    return lg::kInvalidValue;
  const int64_t ctas = (int64_t)n_seqs * heads * 2;
  if (ctas > 2147483647ll) return lg::kInvalidValue;
  if (scratch) {
    // two launches: the state-independent part of every chunk at once, then the chains over the chunks
    if (n_tokens < 0 || ((uintptr_t)scratch & 127) || heads > 65535) return lg::kInvalidValue;
    const int64_t max_chunks = (int64_t)n_tokens / CH + n_seqs;
    if (max_chunks > 2147483647ll) return lg::kInvalidValue;
    const int smem_a = (int)sizeof(IntraSmem) + 128, smem_b = (int)sizeof(StateSmem) + 128;
    cudaError_t e = cudaFuncSetAttribute(gdn_chunk_intra_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_a);
    if (e != cudaSuccess) return (uint32_t)e;
    e = cudaFuncSetAttribute(gdn_chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_b);
    if (e != cudaSuccess) return (uint32_t)e;
    lg::launch(gdn_chunk_intra_kernel, dim3((unsigned)max_chunks, (unsigned)heads), dim3(kThreads), smem_a, (cudaStream_t)stream,
               (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const float*)g, (const float*)beta,
               (const int*)cu_seqlens, n_seqs, heads, (int64_t)qkv_stride, (uint8_t*)scratch);
    uint32_t rc = lg::launch_status();
    if (rc) return rc;
    lg::launch(gdn_chunk_state_kernel, dim3((unsigned)ctas), dim3(kThreads), smem_b, (cudaStream_t)stream, (float*)state,
               (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (__nv_bfloat16*)o, (const __nv_bfloat16*)gate_z, (const int*)cu_seqlens,
               (const int*)state_slots, (const uint8_t*)fresh, heads, (int64_t)qkv_stride, scale, (const uint8_t*)scratch);
    return lg::launch_status();
  }
  const int smem = (int)sizeof(Smem) + 128;
  cudaError_t e = cudaFuncSetAttribute(gdn_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (uint32_t)e;
  lg::launch(gdn_chunk_kernel, dim3((unsigned)ctas), dim3(kThreads), smem, (cudaStream_t)stream, 
      (float*)state, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const float*)g, (const float*)beta,
      (__nv_bfloat16*)o, (const __nv_bfloat16*)gate_z, (const int*)cu_seqlens, (const int*)state_slots, (const uint8_t*)fresh, heads,
      (int64_t)qkv_stride, scale);
  return lg::launch_status();
}
