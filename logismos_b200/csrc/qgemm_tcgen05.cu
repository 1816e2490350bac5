// acc[m, n] += A[m, k] * dequant(W)[n, k]^T with int4 group-32 weights, for the small token counts of
// decode and mixed steps (m <= 256), on the 5th-generation tensor cores with the dequantisation
// fused into the operand pipeline: the GPU form of cpu_f32::linear_t (crates/kernels/src/cpu_f32/
// mod.rs:271-345) applied to the dequantised matrix, which is the definition of the int4 linear
// (the reference has no quantised linear; the weight storage is its Turbo4Block nibble order,
// crates/quant/src/kv_codec.rs:70-77).
//
// The weights, not the tokens, fill the 128 rows of the MMA (D[128 weight rows, NT tokens]), so the
// tensor work scales with the real token count and the kernel stays bound by the int4 stream up to
// about 64 tokens. The work is cut into units (128 weight rows x 256 values of k); persistent CTAs
// (two per SM up to 64 tokens) each take a contiguous, equal span of units, and consecutive units of
// one weight tile form one accumulation with one epilogue. 16 warps:
//   warp 0      TMA producer of the raw int4 tiles: codes [128 rows x 128 B] (128-byte swizzle) and
//               fp16 scales [128 rows x 8] per 256 values of k, ring of 2
//   warp 1      TMA producer of the activation tiles [NT x 64] bf16 (128-byte swizzle), ring of 3
//   warp 2      allocates TMEM, issues tcgen05.mma (cta_group::1, kind::f16, M=128, N=NT, K=16)
//               with fp32 accumulators in TMEM, two accumulator buffers
//   warps 4-11  dequantise: thread = (weight row, 32-value group); nibble pairs -> bf16 by byte
//               permute + one logic op (exact 136 + q), minus 136, times the group scale in bf16x2,
//               written as the 128-byte-swizzled K-major tile the MMA descriptor expects
//   warps 12-15 epilogue: read the accumulator from TMEM (lane = weight row, column = token) and add
//               it to acc with fire-and-forget fp32 reductions, one coalesced 128-byte row segment
//               per instruction, while the other accumulator buffer is being filled
// Spans that split a weight tile meet in the fp32 reductions; the order of those additions, and
// therefore the last bits of acc, can differ between runs. Every mbarrier wait is bounded; on expiry the kernel raises an error word, lets copies in
// flight land, frees its TMEM and returns. No cluster launch and no multicast.
#include <cuda.h>

#include "common.cuh"
#include "logismos_kernels.h"
#include "tcgen05.cuh"

namespace {

using namespace lg;
using namespace lg::tc;

constexpr int kWRows = 128;        // weight rows per CTA = MMA M
constexpr int kKB = 64;            // k per MMA stage (one 128-byte swizzle row of bf16)
constexpr int kRawK = 256;         // k per raw stage: 128 B of codes, 8 scales per row
constexpr int kRawStages = 2;
constexpr int kMmaStages = 3;
constexpr int kRawCodes = kWRows * 128;           // 16 KB
constexpr int kRawScales = kWRows * 16;           // 2 KB
constexpr int kRawStage = kRawCodes + kRawScales; // 18 KB (codes first: 1024-aligned)
constexpr int kWdStage = kWRows * 128;            // 16 KB dequantised tile
constexpr int kDqWarps = 8;
constexpr int kEpiWarps = 4;
constexpr int kQThreads = 32 * (4 + kDqWarps + kEpiWarps);  // 512

template <int NT>
struct QCfg {
  static constexpr int kAStage = NT * 128;
  static constexpr int kMmaStage = kWdStage + kAStage;
  static constexpr int kBarBytes = 256;
  static constexpr size_t kSmem = (size_t)kRawStages * kRawStage + (size_t)kMmaStages * kMmaStage + 1024 + kBarBytes;
  static constexpr int kCtasPerSm = kSmem <= 113 * 1024 ? 2 : 1;
};

// two nibbles of one byte (k even in the low nibble) -> bf16x2 {136 + q_even, 136 + q_odd}
LG_DEVINL uint32_t nib_pair_136(uint32_t lo, uint32_t hi, uint32_t sel) {
  uint32_t t;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(t) : "r"(lo), "r"(hi), "r"(sel));
  // bytes 1 and 3 hold data of other pairs: keep the nibbles, flip their sign bit, or in 0x4300
  return (t & 0x000f000fu) ^ 0x43084308u;
}

LG_DEVINL uint32_t bf16x2_sub_mul(uint32_t v, uint32_t c136, uint32_t s2) {
  __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&v);
  const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(&c136);
  const __nv_bfloat162 s = *reinterpret_cast<const __nv_bfloat162*>(&s2);
  a = __hmul2(__hsub2(a, c), s);
  return *reinterpret_cast<uint32_t*>(&a);
}

template <int NT>
__global__ void __launch_bounds__(kQThreads, QCfg<NT>::kCtasPerSm)
qlinear_int4_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_codes,
                            const __grid_constant__ CUtensorMap map_scales, float* __restrict__ acc, int M, int N, int ldc,
                            int n_raw, int total_units, int* __restrict__ status) {
  using C = QCfg<NT>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t raw_base = smem_base;
  const uint32_t mma_base = smem_base + kRawStages * kRawStage;   // kRawStage is a multiple of 1024
  const uint32_t bars = mma_base + kMmaStages * C::kMmaStage;
  uint8_t* bars_gen = smem_gen + kRawStages * kRawStage + kMmaStages * C::kMmaStage;
  auto raw_full = [&](int s) { return bars + 8u * s; };
  auto raw_empty = [&](int s) { return bars + 8u * (kRawStages + s); };
  auto a_full = [&](int s) { return bars + 8u * (2 * kRawStages + s); };
  auto wd_full = [&](int s) { return bars + 8u * (2 * kRawStages + kMmaStages + s); };
  auto mma_empty = [&](int s) { return bars + 8u * (2 * kRawStages + 2 * kMmaStages + s); };
  auto tfull = [&](int b) { return bars + 8u * (2 * kRawStages + 3 * kMmaStages + b); };
  auto tempty = [&](int b) { return bars + 8u * (2 * kRawStages + 3 * kMmaStages + 2 + b); };
  constexpr int kNumBars = 2 * kRawStages + 3 * kMmaStages + 4;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_gen + 8 * kNumBars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // this CTA's contiguous span of units; unit u = (weight tile u / n_raw, raw block u % n_raw). Units of
  // one tile that fall into one span are one accumulation ("segment") with one epilogue.
  const int u0 = (int)((long long)total_units * blockIdx.x / gridDim.x);
  const int u1 = (int)((long long)total_units * (blockIdx.x + 1) / gridDim.x);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRawStages; ++s) { mbar_init(raw_full(s), 1); mbar_init(raw_empty(s), kDqWarps); }
    for (int s = 0; s < kMmaStages; ++s) { mbar_init(a_full(s), 1); mbar_init(wd_full(s), kDqWarps); mbar_init(mma_empty(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull(b), 1); mbar_init(tempty(b), kEpiWarps); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32((const void*)tmem_slot)), "r"((uint32_t)(2 * NT)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- raw int4 producer ----------------
    if (lane == 0) {
      int rs = 0;
      uint32_t rphase = 0;
      for (int u = u0; u < u1; ++u) {
        const int tile = u / n_raw, kk = (u % n_raw) * kRawK;
        if (!mbar_wait(raw_empty(rs), rphase ^ 1u, abort_flag)) break;
        mbar_expect_tx(raw_full(rs), (uint32_t)kRawStage);
        const uint32_t dst = raw_base + rs * kRawStage;
        tma_load_2d(dst, &map_codes, raw_full(rs), kk / 2, tile * kWRows);
        tma_load_2d(dst + kRawCodes, &map_scales, raw_full(rs), kk / 32, tile * kWRows);
        if (++rs == kRawStages) { rs = 0; rphase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ---------------- activation producer ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = u0; u < u1 && ok; ++u) {
        const int kk = (u % n_raw) * kRawK;
        for (int j = 0; j < kRawK / kKB; ++j) {
          if (!mbar_wait(mma_empty(s), phase ^ 1u, abort_flag)) { ok = false; break; }
          mbar_expect_tx(a_full(s), (uint32_t)C::kAStage);
          tma_load_2d(mma_base + s * C::kMmaStage + kWdStage, &map_a, a_full(s), kk + j * kKB, 0);
          if (++s == kMmaStages) { s = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 2) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc<NT>();
      int s = 0, seg = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = u0; u < u1 && ok; ++u) {
        const int rb = u % n_raw;
        const bool seg_start = (u == u0) || rb == 0, seg_end = (u + 1 == u1) || rb == n_raw - 1;
        const int buf = seg & 1;
        if (seg_start) {
          if (!mbar_wait(tempty(buf), (((uint32_t)seg >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
        }
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * NT);
        for (int j = 0; j < kRawK / kKB; ++j) {
          if (!mbar_wait(wd_full(s), phase, abort_flag) || !mbar_wait(a_full(s), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sw = mma_base + s * C::kMmaStage;
          const uint64_t dw = make_smem_desc(sw), da = make_smem_desc(sw + kWdStage);
#pragma unroll
          for (int k = 0; k < kKB / 16; ++k)
            tc_mma_bf16(d_tmem, dw + (uint64_t)(2 * k), da + (uint64_t)(2 * k), idesc, (!seg_start || j || k) ? 1u : 0u);
          tc_commit(mma_empty(s));
          if (++s == kMmaStages) { s = 0; phase ^= 1u; }
        }
        if (ok && seg_end) { tc_commit(tfull(buf)); ++seg; }
      }
    }
  } else if (warp >= 4 && warp < 4 + kDqWarps) {
    // ---------------- dequantise ----------------
    const int wd = warp - 4;
    const int row = (wd & 3) * 32 + lane;   // weight row of the tile
    const int half = wd >> 2;                // which 32-value group of a 64-wide k block
    int rs = 0, s = 0;
    uint32_t rphase = 0, phase = 0;
    bool ok = true;
    const uint32_t c136 = 0x43084308u;
    for (int u = u0; u < u1 && ok; ++u) {
      if (!mbar_wait(raw_full(rs), rphase, abort_flag)) { ok = false; break; }
      const uint8_t* raw = smem_gen + rs * kRawStage;
      const uint16_t* sc = reinterpret_cast<const uint16_t*>(raw + kRawCodes) + row * 8;
#pragma unroll 1
      for (int j = 0; j < kRawK / kKB; ++j) {
        const int g = 2 * j + half;  // group inside the raw block = 16-byte chunk of the row's codes
        const uint4 cw = *reinterpret_cast<const uint4*>(raw + row * 128 + ((g ^ (row & 7)) << 4));
        const float sf = __half2float(__ushort_as_half(sc[g]));
        const __nv_bfloat16 sb = __float2bfloat16_rn(sf);
        const __nv_bfloat162 sb2 = __halves2bfloat162(sb, sb);
        const uint32_t s2 = *reinterpret_cast<const uint32_t*>(&sb2);
        uint4 o[4];
        const uint32_t words[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t lo = words[i] & 0x0f0f0f0fu, hi = (words[i] >> 4) & 0x0f0f0f0fu;
          o[i].x = bf16x2_sub_mul(nib_pair_136(lo, hi, 0x0400u), c136, s2);  // bytes {lo.b0, x, hi.b0, x}
          o[i].y = bf16x2_sub_mul(nib_pair_136(lo, hi, 0x0501u), c136, s2);
          o[i].z = bf16x2_sub_mul(nib_pair_136(lo, hi, 0x0602u), c136, s2);
          o[i].w = bf16x2_sub_mul(nib_pair_136(lo, hi, 0x0703u), c136, s2);
        }
        if (!mbar_wait(mma_empty(s), phase ^ 1u, abort_flag)) { ok = false; break; }
        uint8_t* wt = smem_gen + kRawStages * kRawStage + s * C::kMmaStage + row * 128;
#pragma unroll
        for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(wt + (((half * 4 + i) ^ (row & 7)) << 4)) = o[i];
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(wd_full(s));
        if (++s == kMmaStages) { s = 0; phase ^= 1u; }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(raw_empty(rs));
      if (++rs == kRawStages) { rs = 0; rphase ^= 1u; }
    }
  } else if (warp >= 4 + kDqWarps) {
    // ---------------- epilogue: TMEM (lane = weight row, column = token) -> fp32 reductions ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int seg = 0;
    bool ok = true;
    for (int u = u0; u < u1 && ok; ++u) {
      const int rb = u % n_raw;
      if (!((u + 1 == u1) || rb == n_raw - 1)) continue;  // not the end of a segment
      const int buf = seg & 1;
      if (!mbar_wait(tfull(buf), ((uint32_t)seg >> 1) & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int f = (u / n_raw) * kWRows + q * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < NT; c += 32) {
        if (c >= M) break;
        uint32_t r[32];
        tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * NT + c), r);
        tc_wait_ld();
        if (f < N) {
          float* dst = acc + (size_t)c * ldc + f;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c + j < M) atomicAdd(dst + (size_t)j * ldc, __uint_as_float(r[j]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty(buf));
      ++seg;
    }
  }

  // ---------------- teardown ----------------
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && status) atomicExch(status, 2);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)(2 * NT)) : "memory");
  }
}

// acc fp32 [m, n] -> bf16 (+ bias), or SwiGLU over rows interleaved in blocks of 32 (32 gate columns
// then the 32 matching up columns); acc is left zeroed for the next accumulation.
__global__ void qlinear_finish_kernel(float* __restrict__ acc, const float* __restrict__ bias, __nv_bfloat16* __restrict__ out,
                                      int m, int n, int ld_acc, int ldc, int swiglu) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  if (!swiglu) {
    const int per_row = n / 4;
    if (idx >= (int64_t)m * per_row) return;
    const int t = (int)(idx / per_row), c = (int)(idx % per_row) * 4;
    float4* p = reinterpret_cast<float4*>(acc + (size_t)t * ld_acc + c);
    float4 v = *p;
    *p = zero;
    if (bias) { v.x += bias[c]; v.y += bias[c + 1]; v.z += bias[c + 2]; v.w += bias[c + 3]; }
    uint2 pk;
    pk.x = pack_bf16x2(v.x, v.y);
    pk.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(out + (size_t)t * ldc + c) = pk;
  } else {
    const int inter = n / 2, per_row = inter / 4;
    if (idx >= (int64_t)m * per_row) return;
    const int t = (int)(idx / per_row), oc = (int)(idx % per_row) * 4;
    const int gc = (oc >> 5) * 64 + (oc & 31);
    float4* pg = reinterpret_cast<float4*>(acc + (size_t)t * ld_acc + gc);
    float4* pu = reinterpret_cast<float4*>(acc + (size_t)t * ld_acc + gc + 32);
    float4 g = *pg, u = *pu;
    *pg = zero;
    *pu = zero;
    if (bias) {
      g.x += bias[gc]; g.y += bias[gc + 1]; g.z += bias[gc + 2]; g.w += bias[gc + 3];
      u.x += bias[gc + 32]; u.y += bias[gc + 33]; u.z += bias[gc + 34]; u.w += bias[gc + 35];
    }
    auto silu = [](float x) { return x / (1.0f + __expf(-x)); };
    uint2 pk;
    pk.x = pack_bf16x2(silu(g.x) * u.x, silu(g.y) * u.y);
    pk.y = pack_bf16x2(silu(g.z) * u.z, silu(g.w) * u.w);
    *reinterpret_cast<uint2*>(out + (size_t)t * ldc + oc) = pk;
  }
}

bool make_map_generic(CUtensorMap* map, CUtensorMapDataType dt, uint64_t esz, const void* ptr, uint64_t rows, uint64_t cols,
                      uint64_t ld, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * esz};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NT>
uint32_t launch_q(const void* a, const void* codes, const void* scales, float* acc, int m, int n, int k, int lda, int ldc,
                  int* status, cudaStream_t stream) {
  CUtensorMap ma, mc, ms;
  if (!make_map(&ma, a, (uint64_t)m, (uint64_t)k, (uint64_t)lda, NT)) return lg::kInvalidValue;
  if (!make_map_generic(&mc, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, codes, (uint64_t)n, (uint64_t)k / 2, (uint64_t)k / 2, 128, kWRows,
                        CU_TENSOR_MAP_SWIZZLE_128B))
    return lg::kInvalidValue;
  if (!make_map_generic(&ms, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, scales, (uint64_t)n, (uint64_t)k / 32, (uint64_t)k / 32, 8, kWRows,
                        CU_TENSOR_MAP_SWIZZLE_NONE))
    return lg::kInvalidValue;
  auto kern = qlinear_int4_tcgen05_kernel<NT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)QCfg<NT>::kSmem);
  if (e != cudaSuccess) return (uint32_t)e;
  // persistent CTAs, each with a contiguous, equal share of the (weight tile, raw block) units
  const int n_tiles = (n + kWRows - 1) / kWRows, n_raw = k / kRawK;
  const long total = (long)n_tiles * n_raw;
  if (total > 2147483647l) return lg::kInvalidValue;
  const int slots = sm_count() * QCfg<NT>::kCtasPerSm;
  const int grid = total < slots ? (int)total : slots;
  kern<<<grid, kQThreads, QCfg<NT>::kSmem, stream>>>(ma, mc, ms, acc, m, n, ldc, n_raw, (int)total, status);
  return lg::launch_status();
}

}  // namespace

extern "C" {

uint32_t logismos_launch_qlinear_int4_g32_acc_f32(const void* a, const void* codes, const void* scales, void* acc, int32_t m,
                                                  int32_t n, int32_t k, int32_t lda, int32_t ldc, void* status_i32,
                                                  void* stream) {
  lg::LaunchScope launch_scope_;
  if (m <= 0 || m > 256 || n <= 0 || k <= 0 || (k % kRawK) || (lda % 8) || lda < k || ldc < n) return lg::kInvalidValue;
  if (((uintptr_t)a & 15) || ((uintptr_t)codes & 15) || ((uintptr_t)scales & 15) || ((uintptr_t)acc & 3)) return lg::kInvalidValue;
  if ((k / 2) % 16 || ((k / 32) * 2) % 16) return lg::kInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  int* st = (int*)status_i32;
  float* o = (float*)acc;
  if (m <= 64) return launch_q<64>(a, codes, scales, o, m, n, k, lda, ldc, st, s);
  if (m <= 128) return launch_q<128>(a, codes, scales, o, m, n, k, lda, ldc, st, s);
  return launch_q<256>(a, codes, scales, o, m, n, k, lda, ldc, st, s);
}

uint32_t logismos_launch_qlinear_finish_bf16(void* acc, const void* bias, void* out, int32_t m, int32_t n, int32_t ld_acc,
                                             int32_t ldc, int32_t swiglu, void* stream) {
  lg::LaunchScope launch_scope_;
  if (m < 0 || n <= 0 || (n % (swiglu ? 64 : 4)) || ld_acc < n || (ld_acc % 4) || (ldc % 4) || ldc < (swiglu ? n / 2 : n))
    return lg::kInvalidValue;
  if (((uintptr_t)acc & 15) || ((uintptr_t)out & 7)) return lg::kInvalidValue;
  if (m == 0) return 0;
  const int64_t total = (int64_t)m * ((swiglu ? n / 2 : n) / 4);
  qlinear_finish_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (float*)acc, (const float*)bias, (__nv_bfloat16*)out, m, n, ld_acc, ldc, swiglu);
  return lg::launch_status();
}

}  // extern "C"
