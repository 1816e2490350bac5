// C = A W^T (+ bias) on the 5th-generation tensor cores: the GPU form of cpu_f32::linear_t
// (crates/kernels/src/cpu_f32/mod.rs:271-345) for the encoder / prefill GEMMs, which are the
// only dense contractions on the path.
//
// Design (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor 2-D tiles of A [128 x 64] and W [BN x 64]
//               (bf16, 128-byte swizzle) into a ring of shared-memory stages
//   warp 1      allocates TMEM and issues tcgen05.mma (cta_group::1, kind::f16, M=128, N=BN,
//               K=16; four per 64-wide stage) with fp32 accumulators in TMEM; two accumulator
//               buffers so the epilogue of tile i overlaps the main loop of tile i+1
//   warps 2..5  epilogue: tcgen05.ld 32 lanes x 32 columns per warp step; bf16 outputs (bias,
//               SwiGLU fused in registers) go out as 64-byte-per-thread vector stores; the fp32
//               residual update x += acc is staged as 32 x 32 slabs in shared memory (128-byte
//               swizzle) and applied by a TMA bulk tensor reduce-add, so x is never read into the SM
// Synchronisation is by mbarriers only: full/empty per stage (TMA complete_tx, tcgen05.commit)
// and full/empty per accumulator buffer. Every wait is bounded; on expiry the kernel raises an
// error word, lets outstanding copies land, frees its TMEM and returns.
// No cluster launch and no multicast is used: each CTA fetches its own tiles.
#include <cuda.h>

#include "common.cuh"
#include "logismos_kernels.h"
#include "tcgen05.cuh"

namespace {

using namespace lg;
using namespace lg::tc;

constexpr int BM = 128;
constexpr int BK = 64;            // 64 bf16 = 128 B = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;

template <int BN>
struct Cfg {
  static constexpr int kStageA = BM * BK * 2;
  static constexpr int kStageB = BN * BK * 2;
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = (192 * 1024) / kStage;  // 256->4, 192->4, 128->6
  static constexpr int kTmemCols = (2 * BN <= 256) ? 256 : 512;
  static constexpr int kEpiBytes = 4 * 2 * 4096;  // 4 epilogue warps x 2 staging slabs of 32 rows x 128 B
  static constexpr size_t kSmem = (size_t)kStages * kStage + kEpiBytes + 1024 /*align*/ + 256 /*barriers*/;
};

LG_DEVINL float silu_f(float x) { return x / (1.0f + __expf(-x)); }

template <int BN, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
linear_t_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                        const __grid_constant__ CUtensorMap map_out, const float* __restrict__ bias,
                        void* __restrict__ out, int M, int N, int K, int ldc, int splits, int w_static,
                        int* __restrict__ status) {
  using C = Cfg<BN>;
  lg::pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: required by the 128-byte swizzle atoms the descriptors assume
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t epi_base = smem_base + C::kStages * C::kStage;  // 8 staging slabs of 4 KB (1024-aligned)
  const uint32_t bars = epi_base + C::kEpiBytes;  // full[S], empty[S], tfull[2], tempty[2]
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::kStages + s); };
  auto tfull_bar = [&](int b) { return bars + 8u * (2 * C::kStages + b); };
  auto tempty_bar = [&](int b) { return bars + 8u * (2 * C::kStages + 2 + b); };
  uint8_t* bars_gen = smem_gen + C::kStages * C::kStage + C::kEpiBytes;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * (2 * C::kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_gen + 8 * (2 * C::kStages + 4) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  // a work item is (k slice, output tile); slices of k exist only for the accumulating epilogue, whose
  // reduce-add makes them meet in the output
  const int out_tiles = m_tiles * n_tiles;
  const int total_tiles = out_tiles * splits;
  const int all_kb = K / BK;
  const int kb_per = (all_kb + splits - 1) / splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  // w_static: nothing still in flight writes the weights, so the weight halves of the first stages of
  // this CTA's first tile are requested before the dependency wait (they land while the preceding
  // kernel drains); each stage's barrier already expects the bytes of both halves
  int pre_w = 0;
  if (w_static && threadIdx.x == 0 && (int)blockIdx.x < total_tiles) {
    const int ot = (int)blockIdx.x % out_tiles, sp = (int)blockIdx.x / out_tiles;
    const int n_blk = ot / m_tiles;
    const int kb0 = sp * kb_per, kb1 = min(all_kb, kb0 + kb_per);
    for (int kb = kb0; kb < kb1 && pre_w < C::kStages; ++kb, ++pre_w) {
      mbar_expect_tx(full_bar(pre_w), (uint32_t)C::kStage);
      tma_load_2d(smem_base + pre_w * C::kStage + C::kStageA, &map_w, full_bar(pre_w), kb * BK, n_blk * BN);
    }
  }
  lg::pdl_wait();  // everything before this touched shared memory or read the static weights only
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32((const void*)tmem_slot)), "r"((uint32_t)C::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int ot = tile % out_tiles, sp = tile / out_tiles;
        const int m_blk = ot % m_tiles, n_blk = ot / m_tiles;
        const int kb0 = sp * kb_per, kb1 = min(all_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
          const bool have_w = pre_w > 0;  // requested before the dependency wait (first stages of the first tile)
          if (!have_w) mbar_expect_tx(full_bar(stage), (uint32_t)C::kStage);
          const uint32_t sa = smem_base + stage * C::kStage;
          tma_load_2d(sa, &map_a, full_bar(stage), kb * BK, m_blk * BM);
          if (!have_w) tma_load_2d(sa + C::kStageA, &map_w, full_bar(stage), kb * BK, n_blk * BN);
          else --pre_w;
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc<BN>();
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
        const int buf = it & 1;
        const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
        if (!mbar_wait(tempty_bar(buf), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        const int sp = tile / out_tiles;
        const int kb0 = sp * kb_per, kb1 = min(all_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * C::kStage;
          const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + C::kStageA);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing 16 bf16 along K inside the swizzle row = +32 B = +2 in the encoded address
            tc_mma_bf16(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, ((kb - kb0) | k) ? 1u : 0u);
          }
          tc_commit(empty_bar(stage));  // stage reusable once these MMAs have read it
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) tc_commit(tfull_bar(buf));  // accumulator complete
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    uint8_t* slabs = smem_gen + C::kStages * C::kStage + q * 2 * 4096;
    const uint32_t slabs_a = epi_base + q * 2 * 4096;
    int it = 0, n_store = 0;
    bool ok = true;
    // hands the slab just written to the TMA engine; the slab used two stores ago must have been read
    auto slab_acquire = [&]() -> int {
      const int b = n_store & 1;
      if (lane == 0) bulk_wait_read<1>();
      __syncwarp();
      return b;
    };
    auto slab_release = [&](int b, int x, int y, bool in_range) {
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        if (in_range) {
          if (EPI == LG_EPI_RESID_F32) tma_reduce_add_2d(&map_out, slabs_a + b * 4096, x, y);
          else tma_store_2d(&map_out, slabs_a + b * 4096, x, y);
        }
        bulk_commit();
      }
      ++n_store;
    };
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
      const int ot = tile % out_tiles;
      const int m_blk = ot % m_tiles, n_blk = ot / m_tiles;
      const bool first_slice = tile < out_tiles;  // the bias joins once
      const int buf = it & 1;
      const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
      if (!mbar_wait_warp(tfull_bar(buf), acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row0 = m_blk * BM + q * 32;  // first output row of this warp's slab
      const int row = row0 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
      if (EPI == LG_EPI_RESID_F32) {
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tc_ld32(t_row + c, r);
          tc_wait_ld();
          const int ncol = n_blk * BN + c;
          const int b = slab_acquire();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float a0 = __uint_as_float(r[4 * j]), a1 = __uint_as_float(r[4 * j + 1]);
            float a2 = __uint_as_float(r[4 * j + 2]), a3 = __uint_as_float(r[4 * j + 3]);
            if (bias && first_slice && ncol + 4 * j < N) { a0 += bias[ncol + 4 * j]; a1 += bias[ncol + 4 * j + 1]; a2 += bias[ncol + 4 * j + 2]; a3 += bias[ncol + 4 * j + 3]; }
            slab_write(slabs + b * 4096, lane, j, make_uint4(__float_as_uint(a0), __float_as_uint(a1), __float_as_uint(a2), __float_as_uint(a3)));
          }
          slab_release(b, ncol, row0, ncol < N && row0 < M);
        }
      } else if (EPI == LG_EPI_BF16) {
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tc_ld32(t_row + c, r);
          tc_wait_ld();
          const int ncol = n_blk * BN + c;
          if (row < M) {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * ldc + ncol;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (ncol + j * 8 < N) {
                  uint32_t w[4];
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    const int e = j * 8 + i * 2;
                    float a = __uint_as_float(r[e]), b = __uint_as_float(r[e + 1]);
                    if (bias) { a += bias[ncol + e]; b += bias[ncol + e + 1]; }
                    w[i] = pack_bf16x2(a, b);
                  }
                  *reinterpret_cast<uint4*>(dst + j * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                }
              }
          }
        }
      } else {  // LG_EPI_SWIGLU
        // W rows interleave 32 gate rows with the 32 matching up rows
        for (int c = 0; c < BN; c += 64) {
          uint32_t g[32], u[32];
          tc_ld32(t_row + c, g);
          tc_ld32(t_row + c + 32, u);
          tc_wait_ld();
          const int ncol = n_blk * BN + c;        // column of the gate block in W-row space
          const int ocol = ncol >> 1;             // output column
          if (row < M && ncol < N) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * ldc + ocol;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t w[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int e = j * 8 + i * 2;
                float g0 = __uint_as_float(g[e]), g1 = __uint_as_float(g[e + 1]);
                float u0 = __uint_as_float(u[e]), u1 = __uint_as_float(u[e + 1]);
                if (bias) { g0 += bias[ncol + e]; g1 += bias[ncol + e + 1]; u0 += bias[ncol + 32 + e]; u1 += bias[ncol + 32 + e + 1]; }
                w[i] = pack_bf16x2(silu_f(g0) * u0, silu_f(g1) * u1);
              }
              *reinterpret_cast<uint4*>(dst + j * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
    }
    if (lane == 0) bulk_wait_all();  // every slab has left shared memory and landed before the CTA retires
  }

  // ---------------- teardown ----------------
  __syncwarp();
  if (*abort_flag) {
    // a wait expired somewhere: give copies that may still be in flight time to land before the
    // shared memory and TMEM are released, and report
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && status) atomicExch(status, 2 | (1 << 8));  // low byte 2: a bounded wait expired; next byte: which kernel family
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols) : "memory");
  }
}

// One thread per output element, ascending-k fp32 accumulation: the correctness anchor.
__global__ void linear_t_naive_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w,
                                      const float* __restrict__ bias, void* __restrict__ out, int M, int N,
                                      int K, int lda, int ldc, int epi) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  const int row = blockIdx.y * blockDim.y + threadIdx.y;
  if (row >= M || col >= N) return;
  float acc = 0.0f;
  const __nv_bfloat16* ar = a + (size_t)row * lda;
  const __nv_bfloat16* wr = w + (size_t)col * K;
  for (int k = 0; k < K; ++k) acc += __bfloat162float(ar[k]) * __bfloat162float(wr[k]);
  if (bias) acc += bias[col];
  if (epi == LG_EPI_BF16)
    reinterpret_cast<__nv_bfloat16*>(out)[(size_t)row * ldc + col] = __float2bfloat16_rn(acc);
  else
    reinterpret_cast<float*>(out)[(size_t)row * ldc + col] += acc;
}

// ---- host side ------------------------------------------------------------------------------------

template <int BN, int EPI>
uint32_t launch_cfg(const void* a, const void* w, const float* bias, void* out, int m, int n, int k, int lda,
                    int ldc, int w_static, int* status, cudaStream_t stream) {
  CUtensorMap ma, mw, mo;
  if (!make_map(&ma, a, (uint64_t)m, (uint64_t)k, (uint64_t)lda, BM)) return lg::kInvalidValue;
  if (!make_map(&mw, w, (uint64_t)n, (uint64_t)k, (uint64_t)k, BN)) return lg::kInvalidValue;
  if (EPI == LG_EPI_RESID_F32) {  // fp32 [m, n] in 32 x 32 boxes for the reduce-add epilogue
    if (!make_map(&mo, out, (uint64_t)m, (uint64_t)n, (uint64_t)ldc, 32, true)) return lg::kInvalidValue;
  } else {
    mo = ma;  // unused by the direct-store epilogues
  }
  auto kern = linear_t_tcgen05_kernel<BN, EPI>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<BN>::kSmem);
  if (e != cudaSuccess) return (uint32_t)e;
  const int tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
  // few output tiles and a long reduction (the output projections of a small step): the accumulating
  // epilogue lets slices of k run on otherwise idle SMs; every slice gets at least four k blocks
  int splits = 1;
  if (EPI == LG_EPI_RESID_F32 && !lg::deterministic()) {
    const int all_kb = k / BK;
    if (tiles * 2 <= sm_count() && all_kb >= 8) {
      const int want = sm_count() / tiles;
      int kb_per = (all_kb + want - 1) / want;
      if (kb_per < 4) kb_per = 4;
      splits = (all_kb + kb_per - 1) / kb_per;
    }
  }
  const int items = tiles * splits;
  const int grid = items < sm_count() ? items : sm_count();
  lg::launch(kern, dim3(grid), dim3(kThreads), Cfg<BN>::kSmem, stream, ma, mw, mo, bias, out, m, n, k, ldc, splits, w_static, status);
  return lg::launch_status();
}

template <int EPI>
uint32_t launch_epi(const void* a, const void* w, const float* bias, void* out, int m, int n, int k, int lda,
                    int ldc, int w_static, int* status, cudaStream_t stream) {
  // tile width by wave quantisation: time ~ waves(BN) * BN; ties go to the wider tile
  const int sms = sm_count();
  const int mt = (m + BM - 1) / BM;
  int best_bn = 256;
  long best_cost = -1;
  const int cands[3] = {256, 192, 128};
  for (int i = 0; i < 3; ++i) {
    const int bn = cands[i];
    const long tiles = (long)mt * ((n + bn - 1) / bn);
    const long waves = (tiles + sms - 1) / sms;
    const long cost = waves * bn;
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_bn = bn; }
  }
  if (best_bn == 256) return launch_cfg<256, EPI>(a, w, bias, out, m, n, k, lda, ldc, w_static, status, stream);
  if (best_bn == 192) return launch_cfg<192, EPI>(a, w, bias, out, m, n, k, lda, ldc, w_static, status, stream);
  return launch_cfg<128, EPI>(a, w, bias, out, m, n, k, lda, ldc, w_static, status, stream);
}

}  // namespace

extern "C" {

uint32_t logismos_launch_linear_t_bf16(const void* a, const void* w, const void* bias, void* out, int32_t m,
                                       int32_t n, int32_t k, int32_t lda, int32_t ldc, int32_t epilogue,
                                       void* status_i32, void* stream) {
  lg::LaunchScope launch_scope_;
  const int w_static = (epilogue & LG_EPI_STATIC_W) ? 1 : 0;
  epilogue &= ~LG_EPI_STATIC_W;
  if (m <= 0 || n <= 0 || k <= 0 || (k % BK) || (n % 16) || (lda % 8) || lda < k) return lg::kInvalidValue;
  if (((uintptr_t)a & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15)) return lg::kInvalidValue;
  if (epilogue == LG_EPI_SWIGLU && (n % 64)) return lg::kInvalidValue;
  const int out_cols = epilogue == LG_EPI_SWIGLU ? n / 2 : n;
  if (ldc < out_cols || (ldc % (epilogue == LG_EPI_RESID_F32 ? 4 : 8))) return lg::kInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  const float* b = (const float*)bias;
  int* st = (int*)status_i32;
  switch (epilogue) {
    case LG_EPI_BF16: return launch_epi<LG_EPI_BF16>(a, w, b, out, m, n, k, lda, ldc, w_static, st, s);
    case LG_EPI_RESID_F32: return launch_epi<LG_EPI_RESID_F32>(a, w, b, out, m, n, k, lda, ldc, w_static, st, s);
    case LG_EPI_SWIGLU: return launch_epi<LG_EPI_SWIGLU>(a, w, b, out, m, n, k, lda, ldc, w_static, st, s);
    default: return lg::kInvalidValue;
  }
}

uint32_t logismos_launch_linear_t_naive_bf16(const void* a, const void* w, const void* bias, void* out,
                                             int32_t m, int32_t n, int32_t k, int32_t lda, int32_t ldc,
                                             int32_t epilogue, void* stream) {
  lg::LaunchScope launch_scope_;
  if (m <= 0 || n <= 0 || k <= 0 || lda < k || ldc < n) return lg::kInvalidValue;
  if (epilogue != LG_EPI_BF16 && epilogue != LG_EPI_RESID_F32) return lg::kInvalidValue;
  dim3 block(32, 8), grid((n + 31) / 32, (m + 7) / 8);
  linear_t_naive_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (const float*)bias, out, m, n, k, lda, ldc, epilogue);
  return lg::launch_status();
}

}  // extern "C"
