// int4 group-32 dequant GEMV / skinny GEMM:  y[b,n] = sum_g s[n,g] * sum_{k in g} q[n,k] * x[b,k]
//
// Weight layout (anchored on the reference's Turbo4Block nibble order, crates/quant/src/lib.rs
// :272-301): codes [N, K/2] bytes, value k of a row in byte k/2, low nibble for even k, stored as
// a two's-complement 4-bit integer; scales [N, K/32] fp16. Activations x [B, K] bf16, output
// y [B, N] bf16, fp32 accumulation. The weight matrix stays [N, K] like the reference's
// linear_t (crates/kernels/src/cpu_f32/mod.rs:271-345).
//
// The kernel is bound by HBM traffic of the codes (0.5625 B per weight incl. scales), so the
// design goal is to keep CUDA-core work per weight minimal:
//   - a warp owns 16 weight rows; lane (g = lane/4, c = lane%4) reads, for rows g and g+8, the
//     32-bit word c of four consecutive groups, i.e. the warp touches 64 contiguous bytes of
//     each of its 16 rows per step;
//   - nibbles become 16-bit floats with one LOP3 per pair and one shift per 32-bit word: the low
//     nibble of each byte, (w & 0x000f000f) ^ 0x0008 | 0x4300, is the bf16 number 136 + q (q the
//     signed code); the high nibble is used IN PLACE, (w & 0x00f000f0) ^ 0x0080 | 0x6400, which is
//     the fp16 number 1152 + 16 q; both exact;
//   - the multiply-accumulate runs on the tensor cores (mma.sync m16n8k16, fp32 accumulate, exact
//     products): one bf16 instruction for the low nibbles against x, one fp16 instruction for the
//     high nibbles against x/16, all 16 k-slots of an instruction taken from ONE quantisation
//     group, so the group scale is applied afterwards in fp32:
//       acc += s * (sum_lo (136+q) x + sum_hi (1152+16q) x/16 - 136 sum_lo x - 72 sum_hi x).
//     The correction term is computed once per CTA while x is staged. x/16 is held in fp16, whose
//     range is narrow, so every batch row is first scaled by a power of two that brings its largest
//     magnitude into [2^13, 2^14) (exact in bf16 and fp16; undone exactly on the fp32 result): rows
//     of any magnitude, 1e-6 or 1e6, keep full precision, and only elements more than 2^-24 below
//     their row's maximum fall into fp16's subnormals;
//   - x is staged in shared memory in the slot order the fragments want (per 8 values:
//     bf16 [x0,x4,x2,x6] then fp16 [x1,x5,x3,x7]/16), so a lane fetches the B fragments of both
//     instructions of a group with one 128-bit load.
#include "common.cuh"
#include "logismos_kernels.h"

namespace {

using namespace lg;

constexpr int kGroup = 32;
constexpr int kIterK = 128;  // k covered by one warp step (4 groups)

LG_DEVINL uint32_t nib_pair_bf16(uint32_t w) {
  uint32_t r;
  // (w & 0x000f000f) ^ 0x43084308 : LUT (a & b) ^ c = 0x6a
  asm("lop3.b32 %0, %1, %2, %3, 0x6a;\n" : "=r"(r) : "r"(w), "r"(0x000f000fu), "r"(0x43084308u));
  return r;
}

LG_DEVINL uint32_t nib_pair_f16_hi(uint32_t w) {
  uint32_t r;
  // (w & 0x00f000f0) ^ 0x64806480 : the high nibble of each byte, in place, as fp16 1152 + 16 q
  asm("lop3.b32 %0, %1, %2, %3, 0x6a;\n" : "=r"(r) : "r"(w), "r"(0x00f000f0u), "r"(0x64806480u));
  return r;
}

LG_DEVINL void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2], const float (&c)[4]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// One 16-byte unit of staged activations from 8 consecutive bf16 values x0..x7 of one batch row:
// bf16 (x0,x4) (x2,x6) for the low-nibble instruction, fp16 (x1,x5)/16 (x3,x7)/16 for the
// high-nibble instruction. Returns the unit's share of the group correction.
LG_DEVINL float stage_unit(uint4 raw, float f, uint4& out) {
  float2 v01 = unpack_bf16x2(raw.x), v23 = unpack_bf16x2(raw.y);
  float2 v45 = unpack_bf16x2(raw.z), v67 = unpack_bf16x2(raw.w);
  v01.x *= f; v01.y *= f; v23.x *= f; v23.y *= f; v45.x *= f; v45.y *= f; v67.x *= f; v67.y *= f;  // power of two: exact
  out.x = pack_bf16x2(v01.x, v45.x);  // (x0, x4) bf16
  out.y = pack_bf16x2(v23.x, v67.x);  // (x2, x6) bf16
  const __half2 h15 = __floats2half2_rn(v01.y * 0.0625f, v45.y * 0.0625f);
  const __half2 h37 = __floats2half2_rn(v23.y * 0.0625f, v67.y * 0.0625f);
  out.z = *reinterpret_cast<const uint32_t*>(&h15);
  out.w = *reinterpret_cast<const uint32_t*>(&h37);
  const float2 f15 = __half22float2(h15), f37 = __half22float2(h37);
  const float lo = (v01.x + v45.x) + (v23.x + v67.x);
  const float hi = (f15.x + f15.y) + (f37.x + f37.y);  // sum of x/16 as the tensor core will see it
  return 136.0f * lo + 1152.0f * hi;
}

// Per batch row, the power of two f that brings the row's largest magnitude into [2^13, 2^14) and its
// inverse (both exact); an all-zero or non-finite row keeps f = 1. maxbits, fscale, finv: shared
// memory arrays of `rows` entries. Ends with a block-wide barrier.
LG_DEVINL void row_prescale(const __nv_bfloat16* __restrict__ x, int batch, int K, int rows, uint32_t* maxbits, float* fscale,
                            float* finv) {
  for (int n = threadIdx.x; n < rows; n += blockDim.x) maxbits[n] = 0u;
  __syncthreads();
  const int units_row = K / 8;
  for (int u = threadIdx.x; u < rows * units_row; u += blockDim.x) {
    const int n = u / units_row;
    if (n >= batch) break;
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + (size_t)n * K + (size_t)(u % units_row) * 8));
    uint32_t m = 0;
    const uint32_t w[4] = {raw.x & 0x7fff7fffu, raw.y & 0x7fff7fffu, raw.z & 0x7fff7fffu, raw.w & 0x7fff7fffu};
#pragma unroll
    for (int i = 0; i < 4; ++i) m = max(m, max(w[i] & 0xffffu, w[i] >> 16));  // |bf16| orders like its bits
    if (m > (maxbits[n] >> 16)) atomicMax(&maxbits[n], m << 16);
  }
  __syncthreads();
  for (int n = threadIdx.x; n < rows; n += blockDim.x) {
    const uint32_t b = maxbits[n];
    const int e = (int)((b >> 23) & 0xffu);  // biased exponent of the row maximum
    float f = 1.0f, fi = 1.0f;
    if (e > 0 && e < 255) {
      const int fe = min(max(127 + 13 - (e - 127), 2), 252);
      f = __uint_as_float((uint32_t)fe << 23);
      fi = __uint_as_float((uint32_t)(254 - fe) << 23);
    }
    fscale[n] = f;
    finv[n] = fi;
  }
  __syncthreads();
}

// y is bf16 [batch, N], or fp32 when the caller keeps full precision up to an argmax
LG_DEVINL void store_y(void* y, int out_f32, size_t idx, float v) {
  if (out_f32) reinterpret_cast<float*>(y)[idx] = v;
  else reinterpret_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(v);
}

struct Frag {
  uint32_t w0[4], w1[4];  // word c of groups G0..G0+3 for rows g and g+8
  uint2 s0, s1;           // 4 fp16 scales each
};

LG_DEVINL void load_frag(Frag& f, const uint8_t* p0, const uint8_t* p1, const __half* sp0,
                         const __half* sp1) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f.w0[j] = __ldg(reinterpret_cast<const uint32_t*>(p0 + j * 16));
    f.w1[j] = __ldg(reinterpret_cast<const uint32_t*>(p1 + j * 16));
  }
  f.s0 = __ldg(reinterpret_cast<const uint2*>(sp0));
  f.s1 = __ldg(reinterpret_cast<const uint2*>(sp1));
}

// NT = number of 8-wide batch tiles. Block = 32 * rt * ks threads.
template <int NT>
__global__ void __launch_bounds__(256)
gemv_int4_g32_kernel(const uint8_t* __restrict__ codes, const __half* __restrict__ scales,
                     const __nv_bfloat16* __restrict__ x, void* __restrict__ y, int out_f32, int batch,
                     int N, int K, int kc, int rt, int ks) {
  lg::pdl_prologue();
  extern __shared__ __align__(16) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int rt_idx = warp / ks, ks_idx = warp % ks;
  const int groups_kc = kc / kGroup;
  const int xrow_stride = groups_kc * 64 + 64;  // bytes; +64 keeps 128-bit fragment loads conflict free
  uint8_t* xs = smem;
  float* negcorr = reinterpret_cast<float*>(smem + (size_t)NT * 8 * xrow_stride);
  float* fscale = negcorr + (size_t)groups_kc * NT * 8;
  float* finv = fscale + NT * 8;
  row_prescale(x, batch, K, NT * 8, reinterpret_cast<uint32_t*>(finv + NT * 8), fscale, finv);

  const int row_base = (blockIdx.x * rt + rt_idx) * 16;
  const int r0 = min(row_base + g, N - 1), r1 = min(row_base + g + 8, N - 1);
  const int groups_row = K / kGroup;
  const uint8_t* wp0 = codes + (size_t)r0 * (K / 2) + c * 4;
  const uint8_t* wp1 = codes + (size_t)r1 * (K / 2) + c * 4;
  const __half* sp0 = scales + (size_t)r0 * groups_row;
  const __half* sp1 = scales + (size_t)r1 * groups_row;

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += kc) {
    const int kcur = min(kc, K - k0);
    const int iters = kcur / kIterK;
    // first weight fragment of this chunk goes in flight before x is staged
    Frag cur;
    int it = ks_idx;
    if (it < iters)
      load_frag(cur, wp0 + (k0 >> 1) + it * 64, wp1 + (k0 >> 1) + it * 64,
                sp0 + k0 / kGroup + it * 4, sp1 + k0 / kGroup + it * 4);

    if (k0 > 0) __syncthreads();  // previous chunk fully consumed
    {
      const int units_row = kcur / 8;
      const int total = NT * 8 * units_row;  // multiple of 128: whole warps are in or out
      for (int u = tid; u < total; u += blockDim.x) {
        const int n = u / units_row, kk = u % units_row;
        const int G = kk >> 2, cc = kk & 3;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (n < batch) raw = __ldg(reinterpret_cast<const uint4*>(x + (size_t)n * K + k0 + kk * 8));
        uint4 perm;
        float s = stage_unit(raw, fscale[n], perm);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        *reinterpret_cast<uint4*>(xs + (size_t)n * xrow_stride + G * 64 + cc * 16) = perm;
        if (cc == 0) negcorr[G * (NT * 8) + n] = -s;
      }
    }
    __syncthreads();

    while (it < iters) {
      const int nit = it + ks;
      Frag nxt;
      if (nit < iters)
        load_frag(nxt, wp0 + (k0 >> 1) + nit * 64, wp1 + (k0 >> 1) + nit * 64,
                  sp0 + k0 / kGroup + nit * 4, sp1 + k0 / kGroup + nit * 4);
      const __half2 s0a = *reinterpret_cast<const __half2*>(&cur.s0.x);
      const __half2 s0b = *reinterpret_cast<const __half2*>(&cur.s0.y);
      const __half2 s1a = *reinterpret_cast<const __half2*>(&cur.s1.x);
      const __half2 s1b = *reinterpret_cast<const __half2*>(&cur.s1.y);
      const float sc0[4] = {__low2float(s0a), __high2float(s0a), __low2float(s0b), __high2float(s0b)};
      const float sc1[4] = {__low2float(s1a), __high2float(s1a), __low2float(s1b), __high2float(s1b)};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int G = it * 4 + j;
        const uint32_t w0 = cur.w0[j], w1 = cur.w1[j];
        const uint32_t w0s = w0 >> 8, w1s = w1 >> 8;
        const uint32_t a_lo[4] = {nib_pair_bf16(w0), nib_pair_bf16(w1), nib_pair_bf16(w0s), nib_pair_bf16(w1s)};
        const uint32_t a_hi[4] = {nib_pair_f16_hi(w0), nib_pair_f16_hi(w1), nib_pair_f16_hi(w0s), nib_pair_f16_hi(w1s)};
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint4 bx = *reinterpret_cast<const uint4*>(xs + (size_t)(nt * 8 + g) * xrow_stride +
                                                           G * 64 + c * 16);
          const float2 nc = *reinterpret_cast<const float2*>(negcorr + G * (NT * 8) + nt * 8 + 2 * c);
          float d[4] = {nc.x, nc.y, nc.x, nc.y};
          const uint32_t b_lo[2] = {bx.x, bx.y}, b_hi[2] = {bx.z, bx.w};
          mma_bf16_16816(d, a_lo, b_lo, d);
          mma_f16_16816(d, a_hi, b_hi, d);
          acc[nt][0] = fmaf(sc0[j], d[0], acc[nt][0]);
          acc[nt][1] = fmaf(sc0[j], d[1], acc[nt][1]);
          acc[nt][2] = fmaf(sc1[j], d[2], acc[nt][2]);
          acc[nt][3] = fmaf(sc1[j], d[3], acc[nt][3]);
        }
      }
      cur = nxt;
      it = nit;
    }
  }

  // the rows' scales back out of shared memory before the reduction buffer takes its place
  float iv[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) { iv[nt][0] = finv[nt * 8 + 2 * c]; iv[nt][1] = finv[nt * 8 + 2 * c + 1]; }
  // reduce the ks partial sums of each row tile through shared memory, then store
  __syncthreads();
  float* red = reinterpret_cast<float*>(smem);  // [warp][NT][4][32]
  if (ks > 1) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) red[((warp * NT + nt) * 4 + i) * 32 + lane] = acc[nt][i];
    __syncthreads();
  }
  if (ks_idx == 0) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float v[4] = {acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]};
      for (int s = 1; s < ks; ++s)
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] += red[(((warp + s) * NT + nt) * 4 + i) * 32 + lane];
      const int b0 = nt * 8 + 2 * c;
      const int ra = row_base + g, rb = row_base + g + 8;
      if (ra < N) {
        if (b0 < batch) store_y(y, out_f32, (size_t)b0 * N + ra, v[0] * iv[nt][0]);
        if (b0 + 1 < batch) store_y(y, out_f32, (size_t)(b0 + 1) * N + ra, v[1] * iv[nt][1]);
      }
      if (rb < N) {
        if (b0 < batch) store_y(y, out_f32, (size_t)b0 * N + rb, v[2] * iv[nt][0]);
        if (b0 + 1 < batch) store_y(y, out_f32, (size_t)(b0 + 1) * N + rb, v[3] * iv[nt][1]);
      }
    }
  }
}


// ---- streaming variant ---------------------------------------------------------------------------
// For tall weight matrices (many 16-row tiles per SM) the kernel above spends most of its
// instructions re-staging x and reducing across warps. Here a CTA stages x ONCE (all of K) and every
// warp then streams whole row tiles on its own: the weights of one step (16 rows x 64 B) and their
// scales (16 rows x 8 B) travel global -> shared with cp.async through a per-warp ring of STAGES
// slots that runs ahead across row-tile boundaries; ldmatrix.x4 hands lane (g, c) exactly "word c of
// groups 0..3 of row g"; no block-wide barrier and no cross-warp reduction in the loop.
constexpr int kWPitch = 80;  // row pitch of a staged weight step: conflict-free ldmatrix
// One ring slot holds one warp step: RT row tiles of 16 rows x (64 B of codes at kWPitch, 4 fp16
// scales, the same 4 scales widened to fp32).
__host__ __device__ constexpr int slot_bytes(int rt) { return rt * (16 * kWPitch + 16 * 8 + 16 * 16); }

// RT = 16-row tiles a warp carries side by side (1 or 2). With two, the activation fragments and the
// group corrections fetched from shared memory, the ring bookkeeping and the copy addressing are paid
// once for twice the weights, which is what bounds this kernel at batch <= 16: issue slots, not HBM.
template <int NT, int STAGES, int RT>
__global__ void __launch_bounds__(STAGES == 8 ? 256 : (RT == 2 ? 384 : (NT <= 2 ? 768 : 512)))
gemv_int4_g32_stream_kernel(const uint8_t* __restrict__ codes, const __half* __restrict__ scales,
                            const __nv_bfloat16* __restrict__ x, void* __restrict__ y, int out_f32, int batch,
                            int N, int K) {
  lg::pdl_prologue();
  extern __shared__ __align__(16) uint8_t smem[];
  constexpr int kSlot = slot_bytes(RT);
  constexpr int kRows = 16 * RT;
  constexpr uint32_t kScaleH = kRows * kWPitch;      // fp16 scales of the slot
  constexpr uint32_t kScaleF = kScaleH + kRows * 8;  // fp32 scales of the slot, [row][4]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int groups = K / kGroup, iters = K / kIterK;
  const int xrow_stride = groups * 64 + 64;
  uint8_t* xs = smem;
  float* negcorr = reinterpret_cast<float*>(smem + (size_t)NT * 8 * xrow_stride);
  float* fscale = negcorr + (size_t)groups * NT * 8;
  float* finv = fscale + NT * 8;
  uint8_t* ring_gen = smem + (size_t)NT * 8 * xrow_stride + (size_t)groups * NT * 8 * 4 + (size_t)NT * 8 * 12 + (size_t)warp * STAGES * kSlot;
  const uint32_t ring = smem_u32(ring_gen);

  // stage x (bf16, fragment order, every row scaled by its power of two) and the per-group corrections, once
  row_prescale(x, batch, K, NT * 8, reinterpret_cast<uint32_t*>(finv + NT * 8), fscale, finv);
  {
    const int units_row = K / 8;
    const int total = NT * 8 * units_row;
    for (int u = tid; u < total; u += blockDim.x) {
      const int n = u / units_row, kk = u % units_row;
      const int G = kk >> 2, cc = kk & 3;
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (n < batch) raw = __ldg(reinterpret_cast<const uint4*>(x + (size_t)n * K + kk * 8));
      uint4 perm;
      float s = stage_unit(raw, fscale[n], perm);
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      *reinterpret_cast<uint4*>(xs + (size_t)n * xrow_stride + G * 64 + cc * 16) = perm;
      if (cc == 0) negcorr[G * (NT * 8) + n] = -s;
    }
  }
  __syncthreads();

  const int row_tiles = (N + kRows - 1) / kRows;
  const int tile_stride = gridDim.x * nwarps;
  const int first_tile = blockIdx.x * nwarps + warp;
  const int my_tiles = first_tile < row_tiles ? (row_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
  const int total_steps = my_tiles * iters;
  const uint32_t ring_end = ring + STAGES * kSlot;

  // ---- producer: runs STAGES-1 steps ahead of the consumer, across row-tile boundaries. All
  // addresses advance by constants inside a tile; they are rebuilt only when the tile changes.
  int p_left = total_steps, p_it = 0, p_tile = first_tile;
  uint32_t p_slot = ring;
  const uint8_t* pw[2 * RT];
  const __half* ps;
  auto producer_tile = [&](int tile) {
    const int rb = tile * kRows;
#pragma unroll
    for (int h = 0; h < 2 * RT; ++h) pw[h] = codes + (size_t)min(rb + g + 8 * h, N - 1) * (K / 2) + c * 16;
    ps = scales + (size_t)min(rb + (lane & (kRows - 1)), N - 1) * groups;
  };
  producer_tile(p_tile);
  const uint32_t dst_w = (uint32_t)(g * kWPitch + c * 16), dst_s = kScaleH + (uint32_t)((lane & (kRows - 1)) * 8);
  auto issue = [&]() {
    if (p_left > 0) {
#pragma unroll
      for (int h = 0; h < 2 * RT; ++h) {
        cp_async16(p_slot + dst_w + h * 8 * kWPitch, pw[h]);
        pw[h] += 64;
      }
      if (lane < kRows) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(p_slot + dst_s), "l"(ps));
      ps += 4;
      p_slot += kSlot;
      if (p_slot == ring_end) p_slot = ring;
      --p_left;
      if (++p_it == iters) { p_it = 0; p_tile += tile_stride; producer_tile(p_tile); }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) issue();

  // ---- consumer
  const int mat = lane >> 3, mr = lane & 7;  // ldmatrix: lanes 8j..8j+7 address the rows of matrix j (= group j)
  const uint32_t ld_off = (uint32_t)(mr * kWPitch + mat * 16);
  const uint32_t sc_off = kScaleF + (uint32_t)(g * 16);
  const uint32_t xs_a = smem_u32(xs) + (uint32_t)(g * xrow_stride + c * 16);
  const uint32_t nc_a = smem_u32(negcorr) + (uint32_t)(2 * c * 4);
  uint32_t c_slot = ring;
  int c_tile = first_tile;
  for (int t = 0; t < my_tiles; ++t, c_tile += tile_stride) {
    float acc[RT][NT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[r][nt][i] = 0.0f;
    uint32_t xa = xs_a, na = nc_a;
    for (int it = 0; it < iters; ++it) {
      issue();
      cp_async_wait<STAGES - 1>();
      __syncwarp();
      uint32_t w[2 * RT][4];  // [2r] rows g, [2r+1] rows g+8 of row tile r: word c of groups 0..3
#pragma unroll
      for (int h = 0; h < 2 * RT; ++h) ldmatrix_x4(w[h], c_slot + ld_off + h * 8 * kWPitch);
      // each lane widens 2*RT of the step's 64*RT scales to fp32 (instead of every lane widening 8*RT)
      if constexpr (RT == 1) {
        uint32_t sh;
        asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(sh) : "r"(c_slot + kScaleH + (uint32_t)(lane * 4)));
        const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&sh));
        asm volatile("st.shared.v2.f32 [%0], {%1, %2};\n" ::"r"(c_slot + kScaleF + (uint32_t)(lane * 8)), "f"(sf.x), "f"(sf.y));
      } else {
        uint32_t sh0, sh1;
        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];\n" : "=r"(sh0), "=r"(sh1) : "r"(c_slot + kScaleH + (uint32_t)(lane * 8)));
        const float2 sa = __half22float2(*reinterpret_cast<const __half2*>(&sh0));
        const float2 sb = __half22float2(*reinterpret_cast<const __half2*>(&sh1));
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"r"(c_slot + kScaleF + (uint32_t)(lane * 16)), "f"(sa.x), "f"(sa.y), "f"(sb.x), "f"(sb.y));
      }
      __syncwarp();
      float sc[2 * RT][4];
#pragma unroll
      for (int h = 0; h < 2 * RT; ++h)
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];\n"
                     : "=f"(sc[h][0]), "=f"(sc[h][1]), "=f"(sc[h][2]), "=f"(sc[h][3])
                     : "r"(c_slot + sc_off + h * 128));
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t a_lo[RT][4], a_hi[RT][4];
#pragma unroll
        for (int r = 0; r < RT; ++r) {
          const uint32_t w0 = w[2 * r][j], w1 = w[2 * r + 1][j];
          const uint32_t w0s = w0 >> 8, w1s = w1 >> 8;
          a_lo[r][0] = nib_pair_bf16(w0); a_lo[r][1] = nib_pair_bf16(w1);
          a_lo[r][2] = nib_pair_bf16(w0s); a_lo[r][3] = nib_pair_bf16(w1s);
          a_hi[r][0] = nib_pair_f16_hi(w0); a_hi[r][1] = nib_pair_f16_hi(w1);
          a_hi[r][2] = nib_pair_f16_hi(w0s); a_hi[r][3] = nib_pair_f16_hi(w1s);
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          uint32_t b_lo[2], b_hi[2];
          float nc[2];
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n"
                       : "=r"(b_lo[0]), "=r"(b_lo[1]), "=r"(b_hi[0]), "=r"(b_hi[1])
                       : "r"(xa + (uint32_t)(nt * 8 * xrow_stride + j * 64)));
          asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];\n" : "=f"(nc[0]), "=f"(nc[1]) : "r"(na + (uint32_t)((j * NT * 8 + nt * 8) * 4)));
#pragma unroll
          for (int r = 0; r < RT; ++r) {
            float d[4] = {nc[0], nc[1], nc[0], nc[1]};
            mma_bf16_16816(d, a_lo[r], b_lo, d);
            mma_f16_16816(d, a_hi[r], b_hi, d);
            acc[r][nt][0] = fmaf(sc[2 * r][j], d[0], acc[r][nt][0]);
            acc[r][nt][1] = fmaf(sc[2 * r][j], d[1], acc[r][nt][1]);
            acc[r][nt][2] = fmaf(sc[2 * r + 1][j], d[2], acc[r][nt][2]);
            acc[r][nt][3] = fmaf(sc[2 * r + 1][j], d[3], acc[r][nt][3]);
          }
        }
      }
      __syncwarp();  // every lane is done with the slot before a later issue() refills it
      c_slot += kSlot;
      if (c_slot == ring_end) c_slot = ring;
      xa += 4 * 64;
      na += 4 * NT * 8 * 4;
    }
#pragma unroll
    for (int r = 0; r < RT; ++r) {
      const int ra = c_tile * kRows + r * 16 + g, rb = ra + 8;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int b0 = nt * 8 + 2 * c;
        const float i0 = finv[b0], i1 = finv[b0 + 1];
        if (ra < N) {
          if (b0 < batch) store_y(y, out_f32, (size_t)b0 * N + ra, acc[r][nt][0] * i0);
          if (b0 + 1 < batch) store_y(y, out_f32, (size_t)(b0 + 1) * N + ra, acc[r][nt][1] * i1);
        }
        if (rb < N) {
          if (b0 < batch) store_y(y, out_f32, (size_t)b0 * N + rb, acc[r][nt][2] * i0);
          if (b0 + 1 < batch) store_y(y, out_f32, (size_t)(b0 + 1) * N + rb, acc[r][nt][3] * i1);
        }
      }
    }
  }
  cp_async_wait<0>();
}

// ---- wide-slot streaming variant ------------------------------------------------------------------
// For the tallest matrices at batch <= 16 whose rows lie a multiple of 1 KB apart: a warp carries two 16-row tiles side by side, and a ring slot
// holds TWO k steps of them: 32 rows x 128 B of codes (whole 128-byte lines, four per copy instruction)
// and 32 rows x 8 fp16 scales (16 B per row, one copy per lane). Against the narrow slot this halves
// the copy rounds, waits and ring bookkeeping, requests whole lines from L2, and stops fetching every
// 32-byte sector of scales four times. Lanes read their scales as fp16 straight from the slot.
template <int KS> struct Wide {
  static constexpr int kPitch = KS * 64 + 16;            // codes of KS k steps + 16: conflict-free ldmatrix
  static constexpr int kSPitch = KS == 2 ? 16 : 48;      // KS * 4 fp16 scales per row (+16 at KS = 4: conflict-free)
  static constexpr int kSlot = 32 * kPitch + 32 * kSPitch;
};

template <int NT, int STAGES, int KS>
__global__ void __launch_bounds__(384)
gemv_int4_g32_wide_kernel(const uint8_t* __restrict__ codes, const __half* __restrict__ scales,
                          const __nv_bfloat16* __restrict__ x, void* __restrict__ y, int out_f32, int batch,
                          int N, int K) {
  lg::pdl_prologue();
  extern __shared__ __align__(16) uint8_t smem[];
  constexpr int kWidePitch = Wide<KS>::kPitch, kSPitch = Wide<KS>::kSPitch, kWideSlot = Wide<KS>::kSlot;
  constexpr uint32_t kScaleOff = 32 * kWidePitch;
  constexpr int kCh = 4 * KS;          // 16-byte chunks per row per slot
  constexpr int kRowsPer = 32 / kCh;  // rows one copy instruction covers
  constexpr int kCopies = 32 / kRowsPer;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int groups = K / kGroup, iters2 = K / (KS * kIterK);  // slots per row tile
  const int xrow_stride = groups * 64 + 64;
  uint8_t* xs = smem;
  float* negcorr = reinterpret_cast<float*>(smem + (size_t)NT * 8 * xrow_stride);
  float* fscale = negcorr + (size_t)groups * NT * 8;
  float* finv = fscale + NT * 8;
  uint8_t* ring_gen = smem + (size_t)NT * 8 * xrow_stride + (size_t)groups * NT * 8 * 4 + (size_t)NT * 8 * 12 + (size_t)warp * STAGES * kWideSlot;
  const uint32_t ring = smem_u32(ring_gen);

  // stage x (bf16, fragment order, every row scaled by its power of two) and the per-group corrections, once
  row_prescale(x, batch, K, NT * 8, reinterpret_cast<uint32_t*>(finv + NT * 8), fscale, finv);
  {
    const int units_row = K / 8;
    const int total = NT * 8 * units_row;
    for (int u = tid; u < total; u += blockDim.x) {
      const int n = u / units_row, kk = u % units_row;
      const int G = kk >> 2, cc = kk & 3;
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (n < batch) raw = __ldg(reinterpret_cast<const uint4*>(x + (size_t)n * K + kk * 8));
      uint4 perm;
      float s = stage_unit(raw, fscale[n], perm);
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      *reinterpret_cast<uint4*>(xs + (size_t)n * xrow_stride + G * 64 + cc * 16) = perm;
      if (cc == 0) negcorr[G * (NT * 8) + n] = -s;
    }
  }
  __syncthreads();

  const int row_tiles = (N + 31) / 32;
  const int tile_stride = gridDim.x * nwarps;
  const int first_tile = blockIdx.x * nwarps + warp;
  const int my_tiles = first_tile < row_tiles ? (row_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
  const int total_slots = my_tiles * iters2;
  const uint32_t ring_end = ring + STAGES * kWideSlot;

  // ---- producer: lane (r4 = lane / 8, ch = lane % 8) copies chunk ch of rows r4, r4 + 4, ... of the
  // tile, so one instruction moves four whole 128-byte lines; lane L also copies row L's scales.
  const int r4 = lane / kCh, ch = lane % kCh;
  const size_t row_bytes = (size_t)(K / 2);
  int p_left = total_slots, p_it = 0, p_tile = first_tile;
  uint32_t p_slot = ring;
  const uint8_t* pw;   // codes of row (tile * 32 + r4), chunk ch, current slot
  const __half* ps;    // scales of row (tile * 32 + lane), current slot
  bool p_full;         // all 32 rows of the producer's tile exist
  auto producer_tile = [&](int tile) {
    const int rb = tile * 32;
    p_full = rb + 32 <= N;
    pw = codes + (size_t)min(rb + r4, N - 1) * row_bytes + ch * 16;
    ps = scales + (size_t)min(rb + lane, N - 1) * groups;
  };
  producer_tile(p_tile);
  const uint32_t dst_w = (uint32_t)(r4 * kWidePitch + ch * 16), dst_s = kScaleOff + (uint32_t)(lane * kSPitch);
  auto issue = [&]() {
    if (p_left > 0) {
      if (p_full) {
#pragma unroll
        for (int i = 0; i < kCopies; ++i) cp_async16(p_slot + dst_w + i * kRowsPer * kWidePitch, pw + (size_t)(kRowsPer * i) * row_bytes);
      } else {  // last tile of a ragged matrix: rows past the end re-read the last row (never stored)
        const int rb = p_tile * 32;
        const size_t koff = (size_t)p_it * (KS * 64) + ch * 16;
#pragma unroll
        for (int i = 0; i < kCopies; ++i)
          cp_async16(p_slot + dst_w + i * kRowsPer * kWidePitch, codes + (size_t)min(rb + r4 + kRowsPer * i, N - 1) * row_bytes + koff);
      }
#pragma unroll
      for (int i = 0; i < KS / 2; ++i) cp_async16(p_slot + dst_s + i * 16, ps + i * 8);
      pw += KS * 64; ps += KS * 4;
      p_slot += kWideSlot;
      if (p_slot == ring_end) p_slot = ring;
      --p_left;
      if (++p_it == iters2) { p_it = 0; p_tile += tile_stride; producer_tile(p_tile); }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) issue();

  // ---- consumer
  const int mat = lane >> 3, mr = lane & 7;  // ldmatrix: lanes 8j..8j+7 address the rows of matrix j (= group j)
  const uint32_t ld_off = (uint32_t)(mr * kWidePitch + mat * 16);
  const uint32_t sc_off = kScaleOff + (uint32_t)(g * kSPitch);
  const uint32_t xs_a = smem_u32(xs) + (uint32_t)(g * xrow_stride + c * 16);
  const uint32_t nc_a = smem_u32(negcorr) + (uint32_t)(2 * c * 4);
  uint32_t c_slot = ring;
  int c_tile = first_tile;
  for (int t = 0; t < my_tiles; ++t, c_tile += tile_stride) {
    float acc[2][NT][4];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[r][nt][i] = 0.0f;
    uint32_t xa = xs_a, na = nc_a;
    for (int it = 0; it < iters2; ++it) {
      issue();
      cp_async_wait<STAGES - 1>();
      __syncwarp();
      uint32_t sraw[4][2 * KS];  // [h]: the 4 * KS fp16 scales (KS k steps x four groups) of row g + 8h
#pragma unroll
      for (int h = 0; h < 4; ++h)
#pragma unroll
        for (int i = 0; i < KS / 2; ++i)
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n"
                       : "=r"(sraw[h][4 * i]), "=r"(sraw[h][4 * i + 1]), "=r"(sraw[h][4 * i + 2]), "=r"(sraw[h][4 * i + 3])
                       : "r"(c_slot + sc_off + h * 8 * kSPitch + i * 16));
#pragma unroll
      for (int half = 0; half < KS; ++half) {
        uint32_t w[4][4];  // [2r] rows g, [2r+1] rows g+8 of row tile r: word c of groups 0..3 of this k step
#pragma unroll
        for (int h = 0; h < 4; ++h) ldmatrix_x4(w[h], c_slot + ld_off + h * 8 * kWidePitch + half * 64);
        float sc[4][4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sraw[h][2 * half]));
          const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sraw[h][2 * half + 1]));
          sc[h][0] = s01.x; sc[h][1] = s01.y; sc[h][2] = s23.x; sc[h][3] = s23.y;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t a_lo[2][4], a_hi[2][4];
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const uint32_t w0 = w[2 * r][j], w1 = w[2 * r + 1][j];
            const uint32_t w0s = w0 >> 8, w1s = w1 >> 8;
            a_lo[r][0] = nib_pair_bf16(w0); a_lo[r][1] = nib_pair_bf16(w1);
            a_lo[r][2] = nib_pair_bf16(w0s); a_lo[r][3] = nib_pair_bf16(w1s);
            a_hi[r][0] = nib_pair_f16_hi(w0); a_hi[r][1] = nib_pair_f16_hi(w1);
            a_hi[r][2] = nib_pair_f16_hi(w0s); a_hi[r][3] = nib_pair_f16_hi(w1s);
          }
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            uint32_t b_lo[2], b_hi[2];
            float nc[2];
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n"
                         : "=r"(b_lo[0]), "=r"(b_lo[1]), "=r"(b_hi[0]), "=r"(b_hi[1])
                         : "r"(xa + (uint32_t)(nt * 8 * xrow_stride + j * 64)));
            asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];\n" : "=f"(nc[0]), "=f"(nc[1]) : "r"(na + (uint32_t)((j * NT * 8 + nt * 8) * 4)));
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              float d[4] = {nc[0], nc[1], nc[0], nc[1]};
              mma_bf16_16816(d, a_lo[r], b_lo, d);
              mma_f16_16816(d, a_hi[r], b_hi, d);
              acc[r][nt][0] = fmaf(sc[2 * r][j], d[0], acc[r][nt][0]);
              acc[r][nt][1] = fmaf(sc[2 * r][j], d[1], acc[r][nt][1]);
              acc[r][nt][2] = fmaf(sc[2 * r + 1][j], d[2], acc[r][nt][2]);
              acc[r][nt][3] = fmaf(sc[2 * r + 1][j], d[3], acc[r][nt][3]);
            }
          }
        }
        xa += 4 * 64;
        na += 4 * NT * 8 * 4;
      }
      __syncwarp();  // every lane is done with the slot before a later issue() refills it
      c_slot += kWideSlot;
      if (c_slot == ring_end) c_slot = ring;
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int ra = c_tile * 32 + r * 16 + g, rb = ra + 8;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int b0 = nt * 8 + 2 * c;
        const float i0 = finv[b0], i1 = finv[b0 + 1];
        if (ra < N) {
          if (b0 < batch) store_y(y, out_f32, (size_t)b0 * N + ra, acc[r][nt][0] * i0);
          if (b0 + 1 < batch) store_y(y, out_f32, (size_t)(b0 + 1) * N + ra, acc[r][nt][1] * i1);
        }
        if (rb < N) {
          if (b0 < batch) store_y(y, out_f32, (size_t)b0 * N + rb, acc[r][nt][2] * i0);
          if (b0 + 1 < batch) store_y(y, out_f32, (size_t)(b0 + 1) * N + rb, acc[r][nt][3] * i1);
        }
      }
    }
  }
  cp_async_wait<0>();
}

int gemv_sm_count() {
  static int n = 0;
  if (n) return n;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (n <= 0) n = 148;
  return n;
}

template <int NT, int STAGES, int RT>
uint32_t launch_stream(const void* codes, const void* scales, const void* x, void* y, int out_f32, int batch, int N, int K,
                       int grid, int warps, size_t smem, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(gemv_int4_g32_stream_kernel<NT, STAGES, RT>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (uint32_t)e;
  // ordered launches for the GEMV kernels: back-to-back independent GEMVs measured slower with
  // programmatic dependent launch (8960 x 1536: 8.1 -> 9.0 us, 1536 x 8960: 19.6 -> 25.0 us), and a model
  // step has one GEMV (the lm_head), so there is nothing to gain from it here
  lg::launch_ordered(gemv_int4_g32_stream_kernel<NT, STAGES, RT>, grid, dim3(warps * 32), smem, stream, 
      (const uint8_t*)codes, (const __half*)scales, (const __nv_bfloat16*)x, y, out_f32, batch, N, K);
  return lg::launch_status();
}

// Among warp counts lo..hi, the one that leaves the least idle tail: every warp gets floor or ceil of
// tiles / (sms * warps) row tiles, and the kernel ends with the slowest warp.
int best_warp_count(int row_tiles, int sms, int lo, int hi) {
  double best_eff = -1.0;
  int best_w = hi;
  for (int wv = hi; wv >= lo; --wv) {
    const long slots = (long)sms * wv;
    const long per = (row_tiles + slots - 1) / slots;
    const double eff = (double)row_tiles / (double)(per * slots);
    if (eff > best_eff + 1e-9) { best_eff = eff; best_w = wv; }
  }
  return best_w;
}

// Returns true (and the status in *rc) when the streaming variant applies and was launched.
template <int NT>
bool try_launch_stream(const void* codes, const void* scales, const void* x, void* y, int out_f32, int batch, int N, int K,
                       cudaStream_t stream, uint32_t* rc) {
  const int sms = gemv_sm_count();
  const int row_tiles = (N + 15) / 16;
  if (row_tiles < 2 * sms) return false;  // too few row tiles per SM: the k-split kernel spreads better
  const int groups = K / kGroup;
  const size_t xbytes = (size_t)NT * 8 * (groups * 64 + 64) + (size_t)groups * NT * 8 * 4 + (size_t)NT * 8 * 12;
  const size_t budget = 200 * 1024;
  if (xbytes + 2 * 8 * slot_bytes(1) > budget) return false;  // x does not fit: chunked kernel
  int warps = (row_tiles + sms - 1) / sms;
  if (warps <= 8) {  // short matrix: few warps, each with a deep ring
    warps = warps < 2 ? 2 : warps;
    while (xbytes + (size_t)warps * 8 * slot_bytes(1) > budget) --warps;
    const int grid = (row_tiles + warps - 1) / warps < sms ? (row_tiles + warps - 1) / warps : sms;
    *rc = launch_stream<NT, 8, 1>(codes, scales, x, y, out_f32, batch, N, K, grid, warps, xbytes + (size_t)warps * 8 * slot_bytes(1), stream);
    return true;
  }
  // Up to 16 batch rows a warp carries two row tiles side by side (fewer instructions per weight);
  // the warp counts are the measured optimum on 148 SMs for a 151936-row matrix: 11 with one batch
  // tile, 7 with two (more warps there lose to shared-memory pressure from the fragment loads).
  const int rt = (NT <= 2 && row_tiles >= 32 * sms) ? 2 : 1;  // two tiles only when every warp gets several
  const int max_warps = (int)((budget - xbytes) / (4 * slot_bytes(rt)));
  const int tiles = (N + 16 * rt - 1) / (16 * rt);
  int hi = rt == 1 ? 16 : (NT == 1 ? 12 : 8), lo = rt == 1 ? 10 : (NT == 1 ? 8 : 6);
  if (hi > max_warps) hi = max_warps;
  if (lo > hi) lo = hi;
  warps = best_warp_count(tiles, sms, lo, hi);
  if constexpr (NT <= 2) {
    // Wide slots where the narrow ones measured slower: rows a multiple of 1 KB apart (K = 2048:
    // 38.3 against 41.2 us for 151936 rows; at K = 1536 the narrow slots win, 28.6 against 29.1 us).
    const size_t wsmem = xbytes + (size_t)warps * 2 * Wide<2>::kSlot;
    if (rt == 2 && K % 2048 == 0 && wsmem <= budget) {
      auto kern = gemv_int4_g32_wide_kernel<NT, 2, 2>;
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wsmem);
      if (e != cudaSuccess) { *rc = (uint32_t)e; return true; }
      lg::launch_ordered(kern, dim3(sms), dim3(warps * 32), wsmem, stream, (const uint8_t*)codes, (const __half*)scales, (const __nv_bfloat16*)x,
                                               y, out_f32, batch, N, K);
      *rc = lg::launch_status();
      return true;
    }
  }
  const size_t smem = xbytes + (size_t)warps * 4 * slot_bytes(rt);
  if constexpr (NT <= 2) {
    if (rt == 2) {
      // three ring slots measured best with two tiles per warp (28.6 us against 28.9 with four, 29.9 with two)
      *rc = launch_stream<NT, 3, 2>(codes, scales, x, y, out_f32, batch, N, K, sms, warps, xbytes + (size_t)warps * 3 * slot_bytes(2), stream);
      return true;
    }
  }
  *rc = launch_stream<NT, 4, 1>(codes, scales, x, y, out_f32, batch, N, K, sms, warps, smem, stream);
  return true;
}

template <int NT>
uint32_t launch_nt(const void* codes, const void* scales, const void* x, void* y, int out_f32, int batch, int N,
                   int K, cudaStream_t stream) {
  uint32_t src = 0;
  if (try_launch_stream<NT>(codes, scales, x, y, out_f32, batch, N, K, stream, &src)) return src;
  const int iters_k = K / kIterK;
  int kc = 4096 / NT;  // x chunk staged per pass: NT * 8 rows * kc * 2 B  (<= 64 KB)
  if (kc > K) kc = K;
  const int iters_c = kc / kIterK;
  int ks = 8;  // warps splitting the k range of one 16-row tile; each should get >= 2 steps
  while (ks > 1 && (iters_c < 2 * ks || iters_k < 2 * ks)) ks >>= 1;
  const int row_tiles = (N + 15) / 16;
  int rt = 8 / ks;  // row tiles per CTA: 8 warps unless that leaves fewer than two CTAs per SM
  while (rt > 1 && row_tiles / rt < 2 * 148) rt >>= 1;
  const int threads = 32 * rt * ks;
  const int groups_kc = kc / kGroup;
  size_t smem = (size_t)NT * 8 * (groups_kc * 64 + 64) + (size_t)groups_kc * NT * 8 * 4 + (size_t)NT * 8 * 12;
  const size_t red = (size_t)(threads / 32) * NT * 4 * 32 * 4;
  if (red > smem) smem = red;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(gemv_int4_g32_kernel<NT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (uint32_t)e;
  }
  const int grid = (row_tiles + rt - 1) / rt;
  lg::launch_ordered(gemv_int4_g32_kernel<NT>, grid, dim3(threads), smem, stream, 
      (const uint8_t*)codes, (const __half*)scales, (const __nv_bfloat16*)x, y, out_f32,
      batch, N, K, kc, rt, ks);
  return lg::launch_status();
}

}  // namespace

static uint32_t launch_gemv(const void* codes, const void* scales_f16, const void* x_bf16, void* y, int out_f32, int32_t batch,
                            int32_t n, int32_t k, void* stream) {
  if (batch <= 0 || batch > 64 || n <= 0 || k <= 0 || (k % kIterK) != 0) return lg::kInvalidValue;
  if (((uintptr_t)codes & 15) || ((uintptr_t)scales_f16 & 7) || ((uintptr_t)x_bf16 & 15))
    return lg::kInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  const int nt = (batch + 7) / 8;
  if (nt == 1) return launch_nt<1>(codes, scales_f16, x_bf16, y, out_f32, batch, n, k, s);
  if (nt == 2) return launch_nt<2>(codes, scales_f16, x_bf16, y, out_f32, batch, n, k, s);
  if (nt <= 4) return launch_nt<4>(codes, scales_f16, x_bf16, y, out_f32, batch, n, k, s);
  return launch_nt<8>(codes, scales_f16, x_bf16, y, out_f32, batch, n, k, s);
}

extern "C" uint32_t logismos_launch_gemv_int4_g32_bf16(const void* codes, const void* scales_f16,
                                                       const void* x_bf16, void* y_bf16,
                                                       int32_t batch, int32_t n, int32_t k,
                                                       void* stream) {
  lg::LaunchScope launch_scope_;
  return launch_gemv(codes, scales_f16, x_bf16, y_bf16, 0, batch, n, k, stream);
}

extern "C" uint32_t logismos_launch_gemv_int4_g32_f32(const void* codes, const void* scales_f16,
                                                      const void* x_bf16, void* y_f32, int32_t batch,
                                                      int32_t n, int32_t k, void* stream) {
  lg::LaunchScope launch_scope_;
  return launch_gemv(codes, scales_f16, x_bf16, y_f32, 1, batch, n, k, stream);
}

// The same product for any batch up to 64 with the route chosen by shape and row count: the streaming
// GEMV above, or the fused-dequant tensor-core kernel (qgemm_tcgen05.cu), whose fp32 sums go through
// `workspace` and are rounded to bf16 by its finishing kernel. The mma.sync GEMV re-reads the activation
// fragments from shared memory for every 16 weight rows (at 64 batch rows that costs several times the
// weight stream) and walks k serially per row tile, so few long rows leave most SMs idle; the
// tensor-core kernel keeps the activations in one operand tile and splits k over the CTAs. Measured
// crossovers (time per launch, weights from HBM): above 16 rows always; k >= 3 n at every batch
// (1536 x 8960: 10.9 against 19.9 us at one row, 58 us at 16); 8 to 16 rows up to n = 16384 (7.8 against
// 9.1 / 18.6 us for 1536 x 1536). The vocabulary-sized matrices stay on the GEMV up to 16 rows (55
// against 67 us).
extern "C" int32_t logismos_skinny_int4_route(int32_t batch, int32_t n, int32_t k) {
  if ((k % 256) != 0 || (n % 4) != 0 || batch < 1 || batch > 64) return 0;
  if (batch > 16) return 1;
  if ((int64_t)k >= 3 * (int64_t)n) return 1;
  return batch >= 8 && n <= 16384 ? 1 : 0;
}

extern "C" uint32_t logismos_launch_skinny_int4_g32_bf16(const void* codes, const void* scales_f16, const void* x_bf16, void* y_bf16,
                                                         int32_t batch, int32_t n, int32_t k, void* workspace_f32, void* status_i32,
                                                         void* stream) {
  lg::LaunchScope launch_scope_;
  if (workspace_f32 == nullptr || !logismos_skinny_int4_route(batch, n, k))
    return launch_gemv(codes, scales_f16, x_bf16, y_bf16, 0, batch, n, k, stream);
  if ((uintptr_t)workspace_f32 & 15) return lg::kInvalidValue;
  const uint32_t rc = logismos_launch_qlinear_int4_g32_acc_f32(x_bf16, codes, scales_f16, workspace_f32, batch, n, k, k, n, status_i32, stream);
  if (rc) return rc;
  return logismos_launch_qlinear_finish_bf16(workspace_f32, nullptr, y_bf16, batch, n, n, n, 0, stream);
}
