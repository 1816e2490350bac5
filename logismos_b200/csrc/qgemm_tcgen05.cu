// acc[m, n] += A[m, k] * dequant(W)[n, k]^T with int4 group-32 weights, for the small token counts of
// decode and mixed steps (m <= 256), on the 5th-generation tensor cores with the dequantisation
// fused into the operand pipeline: the GPU form of cpu_f32::linear_t (crates/kernels/src/cpu_f32/
// mod.rs:271-345) applied to the dequantised matrix, which is the definition of the int4 linear
// (the reference has no quantised linear; the weight storage is its Turbo4Block nibble order,
// crates/quant/src/kv_codec.rs:70-77).
//
// The weights, not the tokens, fill the 128 rows of the MMA (D[128 weight rows, NT tokens]), so the
// tensor work scales with the real token count and the kernel stays bound by the int4 stream up to
// about 64 tokens. The work is cut into units (128 weight rows x 256 values of k); one persistent
// CTA per SM takes a contiguous, equal span of units, and consecutive units of one weight tile form
// one accumulation with one epilogue. 30 warps:
//   warp 0      TMA producer of the raw int4 tiles: codes [128 rows x 128 B] (128-byte swizzle) and
//               fp16 scales [128 rows x 8] per 256 values of k, ring of 3
//   warp 1      TMA producer of the activation tiles [NT x 64] bf16 (128-byte swizzle), its own ring
//               of three 32 KB stages so that their L2 latency stays off the critical path
//   warps 2, 3, 28, 29  one thread each issues tcgen05.mma (cta_group::1, kind::f16, M=128, N=NT, K=16)
//               for one of the four k blocks of every unit (two each, from warps 2 and 3 only, above 64
//               tokens), the weight operand read from TMEM and the activations from shared memory,
//               into its own fp32 accumulators in TMEM (warp 2 also allocates the tensor memory)
//   warps 4-19  dequantise: four groups of four warps, group g owns k block g of every unit; thread =
//               one weight row x 64 values; the raw stage is released as soon as it is in registers;
//               nibble pairs -> bf16 by byte permute + one logic op (exact 136 + q), minus 136, times
//               the group scale in bf16x2, stored with one tcgen05.st into the tensor-memory tile the
//               MMA reads as its row operand (lane = weight row, column = two values of k), so the
//               expanded weights never pass through shared memory
//   warps 20-27 epilogue (two per lane quarter, half of the token columns each): read the accumulator from TMEM (lane = weight row, column = token) and add
//               it to acc with fire-and-forget fp32 reductions, one coalesced 128-byte row segment
//               per instruction, while the other accumulator buffer is being filled
// Spans that split a weight tile meet in the fp32 reductions; the order of those additions, and
// therefore the last bits of acc, can differ between runs. Every mbarrier wait is bounded; on expiry the kernel raises an error word, lets copies in
// flight land, frees its TMEM and returns. No cluster launch and no multicast.
#include <cuda.h>

#include "common.cuh"
#include "logismos_kernels.h"
#include "tcgen05.cuh"
#include "int4_dequant.cuh"

// Development aid: built with -DLG_QTRACE the first CTA records, per unit, the clock at the points of
// the hand-offs between its roles into a global buffer (logismos_qtrace_buffer); never defined in the
// library build.
#ifdef LG_QTRACE
__device__ long long g_qtrace[4096 * 12];
#define QTRACE(unit, slot) do { if (blockIdx.x == 0 && (unit) < 4096) g_qtrace[(unit) * 12 + (slot)] = clock64(); } while (0)
extern "C" void* logismos_qtrace_buffer() { void* p = nullptr; cudaGetSymbolAddress(&p, g_qtrace); return p; }
#else
#define QTRACE(unit, slot) do { } while (0)
#endif

namespace {

using namespace lg;
using namespace lg::tc;

constexpr int kWRows = 128;        // weight rows per CTA = MMA M
constexpr int kKB = 64;            // k per MMA stage (one 128-byte swizzle row of bf16)
constexpr int kRawK = 256;         // k per raw stage: 128 B of codes, 8 scales per row
constexpr int kGroups = kRawK / kKB;  // 4 k blocks per raw block = 4 MMA stages = 4 dequantising warp groups
constexpr int kRawStages = 5;
constexpr int kRawCodes = kWRows * 128;           // 16 KB
constexpr int kRawScales = kWRows * 16;           // 2 KB
constexpr int kRawStage = kRawCodes + kRawScales; // 18 KB (codes first: 1024-aligned)
constexpr int kWdCols = kKB / 2;                  // TMEM columns of one dequantised k block: 128 lanes x 32 columns x 2 bf16
constexpr int kDqWarps = 4 * kGroups;             // 16
constexpr int kMaxIssuers = 4;                    // MMA-issuing threads: warps 2, 3 and (up to 64 tokens) 28, 29, one per scheduler
constexpr int kEpiWarps = 8;                      // two per TMEM lane quarter, half of the token columns each
constexpr int kQThreads = 32 * (4 + kDqWarps + kEpiWarps + 2);  // 960

template <int NT>
struct QCfg {
  static constexpr int kABlock = NT * 128;             // activation tile of one k block
  static constexpr int kABlocksPerStage = NT <= 64 ? 4 : 2;  // activation stage: a whole unit (NT <= 64) or half of one
  static constexpr int kAStage = kABlocksPerStage * kABlock;
  static constexpr int kAStages = 3;
  static constexpr int kBarBytes = 512;
  static constexpr size_t kSmem = (size_t)kRawStages * kRawStage + (size_t)kAStages * kAStage + 1024 + kBarBytes;
  // TMEM: two buffers of dequantised weight tiles (four k blocks each; operand A of the MMA), then two
  // accumulators. One CTA per SM, so the whole tensor memory is this CTA's.
  static constexpr int kWBufCols = kGroups * kWdCols;  // 128
  static constexpr int kAccCol = 2 * kWBufCols;
  // An issuing thread spends on the order of a hundred cycles per tcgen05.mma whatever the tile width
  // (traced: 8 MMAs and their waits took 1100-1600 of the 2500 cycles a unit cost with two issuers), so
  // up to 64 tokens every k block of a unit has its own issuing thread and its own accumulator.
  static constexpr int kIssuers = NT <= 64 ? 4 : 2;
  static constexpr int kAccBufs = NT <= 32 ? 2 : 1;   // accumulator buffers per issuing thread
  static constexpr int kTmemCols = 512;
  static_assert(kAccCol + kIssuers * kAccBufs * NT <= 512, "tensor memory budget");
};

// Waits of roles that are idle most of the time (producers, epilogue) poll rarely, so that their
// polling does not take issue slots from the dequantising warps. Bounded like mbar_wait.
LG_DEVINL bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    __nanosleep(i < 8 ? 100 : 400);
  }
  *abort_flag = 1;
  return false;
}

// D[tmem] (+)= A[tmem] * B[smem]^T: the weight operand is read from tensor memory, where the
// dequantising warps put it (lane = row, one 32-bit column = two consecutive values of k)
LG_DEVINL void tc_mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// registers -> tensor memory: the 32 lanes of this warp's quarter, 32 consecutive columns
LG_DEVINL void tc_st32(uint32_t taddr, const uint4 (&v)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr), "r"(v[0].x), "r"(v[0].y), "r"(v[0].z), "r"(v[0].w), "r"(v[1].x), "r"(v[1].y), "r"(v[1].z), "r"(v[1].w),
        "r"(v[2].x), "r"(v[2].y), "r"(v[2].z), "r"(v[2].w), "r"(v[3].x), "r"(v[3].y), "r"(v[3].z), "r"(v[3].w),
        "r"(v[4].x), "r"(v[4].y), "r"(v[4].z), "r"(v[4].w), "r"(v[5].x), "r"(v[5].y), "r"(v[5].z), "r"(v[5].w),
        "r"(v[6].x), "r"(v[6].y), "r"(v[6].z), "r"(v[6].w), "r"(v[7].x), "r"(v[7].y), "r"(v[7].z), "r"(v[7].w)
      : "memory");
}
LG_DEVINL void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

template <int NT>
__global__ void __launch_bounds__(kQThreads, 1)
qlinear_int4_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_codes,
                            const __grid_constant__ CUtensorMap map_scales, float* __restrict__ acc, int M, int N, int ldc,
                            int n_raw, int total_units, int whole_tiles, int w_static, int* __restrict__ status) {
  using C = QCfg<NT>;
  lg::pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t raw_base = smem_base;
  const uint32_t a_base = smem_base + kRawStages * kRawStage;   // kRawStage is a multiple of 1024
  constexpr int kTileBytes = kRawStages * kRawStage + C::kAStages * C::kAStage;
  const uint32_t bars = smem_base + kTileBytes;
  uint8_t* bars_gen = smem_gen + kTileBytes;
  auto raw_full = [&](int s) { return bars + 8u * s; };
  auto raw_empty = [&](int s) { return bars + 8u * (kRawStages + s); };
  auto wd_full = [&](int wb, int g) { return bars + 8u * (2 * kRawStages + wb * kGroups + g); };
  auto wd_empty = [&](int wb) { return bars + 8u * (2 * kRawStages + 2 * kGroups + wb); };
  auto tfull = [&](int is, int b) { return bars + 8u * (2 * kRawStages + 2 * kGroups + 2 + is * 2 + b); };
  auto tempty = [&](int b) { return bars + 8u * (2 * kRawStages + 2 * kGroups + 2 + 2 * kMaxIssuers + b); };
  auto a_full = [&](int s) { return bars + 8u * (2 * kRawStages + 2 * kGroups + 4 + 2 * kMaxIssuers + s); };
  auto a_empty = [&](int s) { return bars + 8u * (2 * kRawStages + 2 * kGroups + 4 + 2 * kMaxIssuers + C::kAStages + s); };
  constexpr int kNumBars = 2 * kRawStages + 2 * kGroups + 4 + 2 * kMaxIssuers + 2 * C::kAStages;
  constexpr int kIssuers = C::kIssuers;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_gen + 8 * kNumBars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // this CTA's contiguous span of units; unit u = (weight tile u / n_raw, raw block u % n_raw). Units of
  // one tile that fall into one span are one accumulation ("segment") with one epilogue. The weight
  // tiles of a unit go to tensor-memory buffer (unit count & 1).
  // whole_tiles: spans end at tile boundaries, so every output element is added exactly once (no
  // reduction between CTAs: bit-identical results from run to run, at the price of uneven spans)
  const int n_tiles_all = total_units / n_raw;
  const int u0 = whole_tiles ? (int)((long long)n_tiles_all * blockIdx.x / gridDim.x) * n_raw
                             : (int)((long long)total_units * blockIdx.x / gridDim.x);
  const int u1 = whole_tiles ? (int)((long long)n_tiles_all * (blockIdx.x + 1) / gridDim.x) * n_raw
                             : (int)((long long)total_units * (blockIdx.x + 1) / gridDim.x);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRawStages; ++s) { mbar_init(raw_full(s), 1); mbar_init(raw_empty(s), kDqWarps); }
    for (int wb = 0; wb < 2; ++wb) {
      for (int g = 0; g < kGroups; ++g) mbar_init(wd_full(wb, g), 4);
      mbar_init(wd_empty(wb), kIssuers);
    }
    // an activation stage of a whole unit is read by both issuing threads, one of half a unit by one
    for (int s = 0; s < C::kAStages; ++s) { mbar_init(a_full(s), 1); mbar_init(a_empty(s), C::kABlocksPerStage == kGroups ? kIssuers : 1); }
    for (int b = 0; b < 2; ++b) {
      for (int is = 0; is < kMaxIssuers; ++is) mbar_init(tfull(is, b), 1);
      mbar_init(tempty(b), kEpiWarps);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  // the raw-weight producer's position in its span; thread 0 carries it across the dependency wait
  int p_rs = 0, p_u = u0, p_tile = u0 / n_raw, p_rb = u0 % n_raw;
  uint32_t p_phase = 0;
  auto issue_raw = [&]() {  // requests unit p_u's codes and scales into ring slot p_rs and advances
    mbar_expect_tx(raw_full(p_rs), (uint32_t)kRawStage);
    const uint32_t dst = raw_base + p_rs * kRawStage;
    const int kk = p_rb * kRawK;
    tma_load_2d(dst, &map_codes, raw_full(p_rs), kk / 2, p_tile * kWRows);
    tma_load_2d(dst + kRawCodes, &map_scales, raw_full(p_rs), kk / 32, p_tile * kWRows);
    if (++p_rs == kRawStages) { p_rs = 0; p_phase ^= 1u; }
    if (++p_rb == n_raw) { p_rb = 0; ++p_tile; }
    ++p_u;
  };
  // w_static: nothing still in flight writes the weights, so the ring is filled before the dependency
  // wait (the first slots are free by construction) and lands while the preceding kernel drains
  // Only in the configurations of up to 64 tokens: with 128-token tiles (two issuing threads, activation
  // stages of half a unit) an early-filled ring made about one launch in a few hundred run into an
  // expired wait in a stress test (vocabulary-sized matrix, back-to-back launches); the cause is not
  // understood, and without the early fill 12000 such launches passed.
  if (w_static && NT <= 64 && threadIdx.x == 0)
    while (p_u < u1 && p_u - u0 < kRawStages) issue_raw();
  lg::pdl_wait();  // everything before this touched shared memory or read the static weights only
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32((const void*)tmem_slot)), "r"((uint32_t)C::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- raw int4 producer ----------------
    if (lane == 0) {
      while (p_u < u1) {
        if (!mbar_wait_sleep(raw_empty(p_rs), p_phase ^ 1u, abort_flag, 100)) break;
        QTRACE(p_u - u0, 0);
        issue_raw();
      }
    }
  } else if (warp == 1) {
    // ---------------- activation producer: its own ring of 32 KB stages (one barrier per stage), so
    // that the L2 latency of the activations stays off the critical path ----------------
    if (lane == 0) {
      int as = 0;
      uint32_t aphase = 0;
      bool ok = true;
      int rb = u0 % n_raw;
      for (int u = u0; u < u1 && ok; ++u) {
        const int kk = rb * kRawK;
        if (++rb == n_raw) rb = 0;
#pragma unroll
        for (int h = 0; h < kGroups / C::kABlocksPerStage; ++h) {
          if (!mbar_wait_sleep(a_empty(as), aphase ^ 1u, abort_flag, 100)) { ok = false; break; }
          if (h == 0) QTRACE(u - u0, 10);
          mbar_expect_tx(a_full(as), (uint32_t)C::kAStage);
#pragma unroll
          for (int b = 0; b < C::kABlocksPerStage; ++b)
            tma_load_2d(a_base + as * C::kAStage + b * C::kABlock, &map_a, a_full(as), kk + (h * C::kABlocksPerStage + b) * kKB, 0);
          if (++as == C::kAStages) { as = 0; aphase ^= 1u; }
        }
      }
    }
  } else if (warp == 2 || warp == 3 || ((warp == 28 || warp == 29) && kIssuers == 4)) {
    // ---------------- MMA issuers: thread `is` takes kGroups / kIssuers k blocks of every unit into its
    // own accumulators (the epilogue adds them up). Issuing an MMA or a commit costs a thread on the
    // order of a hundred cycles whatever the tile size, so the k blocks of a unit are issued in
    // parallel by threads on different schedulers; descriptors are built from constants and one add.
    if (lane == 0) {
      const int is = warp < 4 ? warp - 2 : warp - 26;
      constexpr uint32_t idesc = make_idesc<NT>();
      constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024 B, version 1, 128-byte swizzle
      constexpr int per = C::kABlocksPerStage;          // k blocks per activation stage: 4 or 2
      constexpr int kMine = kGroups / kIssuers;         // 2
      const uint32_t a_lo0 = ((a_base & 0x3ffffu) >> 4) | (1u << 16);
      int seg = 0, n_unit = 0;
      // activation stages in the order this thread meets them: every stage (per == 4) or every second one
      int ai = per == kGroups ? 0 : is;
      bool ok = true;
      int rb_next = u0 % n_raw;
      for (int u = u0; u < u1 && ok; ++u, ++n_unit) {
        const int rb = rb_next;
        if (++rb_next == n_raw) rb_next = 0;
        const bool seg_start = (u == u0) || rb == 0, seg_end = (u + 1 == u1) || rb == n_raw - 1;
        const int buf = seg % C::kAccBufs, wb = n_unit & 1;
        const uint32_t tphase = (uint32_t)(seg / C::kAccBufs) & 1u;
        const uint32_t wphase = ((uint32_t)n_unit >> 1) & 1u;
        if (seg_start) {
          if (!mbar_wait(tempty(buf), tphase ^ 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
        }
        if (is == 0) QTRACE(u - u0, 11);
        const uint32_t d_tmem = tmem_base + (uint32_t)(C::kAccCol + (is * C::kAccBufs + buf) * NT);
        const int as = ai % C::kAStages;
        if (!mbar_wait(a_full(as), (uint32_t)(ai / C::kAStages) & 1u, abort_flag)) { ok = false; break; }
        if (is == 0) QTRACE(u - u0, 6);
#pragma unroll
        for (int j = 0; j < kMine; ++j) {
          const int g = is * kMine + j;
          if (!mbar_wait(wd_full(wb, g), wphase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          if (is == 0 && j == 0) QTRACE(u - u0, 7);
          const uint32_t w_tmem = tmem_base + (uint32_t)(wb * C::kWBufCols + g * kWdCols);  // 8 columns per 16 values of k
          const uint32_t a_lo = a_lo0 + (uint32_t)(as * (C::kAStage >> 4) + (g % per) * (C::kABlock >> 4));
#pragma unroll
          for (int k = 0; k < kKB / 16; ++k)
            tc_mma_bf16_ts(d_tmem, w_tmem + 8u * k, ((uint64_t)desc_hi << 32) | (a_lo + 2u * k), idesc, (!seg_start || j || k) ? 1u : 0u);
        }
        if (!ok) break;
        if (is == 0) QTRACE(u - u0, 8);
        tc_commit(a_empty(as));
        tc_commit(wd_empty(wb));
        if (is == 0) QTRACE(u - u0, 9);
        ai += per == kGroups ? 1 : kIssuers;
        if (seg_end) { tc_commit(tfull(is, buf)); ++seg; }
      }
    }
  } else if (warp >= 4 && warp < 4 + kDqWarps) {
    // ---------------- dequantise: warp group g owns k block g of every unit ----------------
    const int wd = warp - 4;
    const int g = wd >> 2;
    const int row = (wd & 3) * 32 + lane;   // weight row of the tile
    int rs = 0, n_unit = 0;
    uint32_t rphase = 0;
    bool ok = true;
    const uint32_t wt0 = tmem_base + ((uint32_t)((wd & 3) * 32) << 16) + (uint32_t)(g * kWdCols);  // this warp's lane quarter
    for (int u = u0; u < u1 && ok; ++u, ++n_unit) {
      const int wb = n_unit & 1;
      const uint32_t wphase = ((uint32_t)n_unit >> 1) & 1u;
      if (wd == 0 && lane == 0) QTRACE(u - u0, 1);
      if (!mbar_wait_sleep_warp(raw_full(rs), rphase, abort_flag)) { ok = false; break; }
      if (wd == 0 && lane == 0) QTRACE(u - u0, 2);
      const uint8_t* raw = smem_gen + rs * kRawStage;
      // this row's 64 codes of k block g (two 16-byte chunks, swizzled by the TMA) and their two scales
      const uint4 c0 = *reinterpret_cast<const uint4*>(raw + row * 128 + (((2 * g) ^ (row & 7)) << 4));
      const uint4 c1 = *reinterpret_cast<const uint4*>(raw + row * 128 + (((2 * g + 1) ^ (row & 7)) << 4));
      const uint32_t sc = *reinterpret_cast<const uint32_t*>(raw + kRawCodes + row * 16 + g * 4);
      __syncwarp();
      if (lane == 0) mbar_arrive(raw_empty(rs));  // the raw stage is in registers: hand it back
      if (++rs == kRawStages) { rs = 0; rphase ^= 1u; }
      const uint32_t s0 = scale_bf16x2(sc, 0), s1 = scale_bf16x2(sc, 1);
      uint4 o[8];
      o[0] = dequant_word(c0.x, s0); o[1] = dequant_word(c0.y, s0); o[2] = dequant_word(c0.z, s0); o[3] = dequant_word(c0.w, s0);
      o[4] = dequant_word(c1.x, s1); o[5] = dequant_word(c1.y, s1); o[6] = dequant_word(c1.z, s1); o[7] = dequant_word(c1.w, s1);
      if (wd == 0 && lane == 0) QTRACE(u - u0, 3);
      if (!mbar_wait_sleep_warp(wd_empty(wb), wphase ^ 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      if (wd == 0 && lane == 0) QTRACE(u - u0, 4);
      tc_st32(wt0 + (uint32_t)(wb * C::kWBufCols), o);  // lane = weight row, 32 columns = its 64 bf16 in k order
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(wd_full(wb, g));
      if (wd == 0 && lane == 0) QTRACE(u - u0, 5);
    }
  } else if (warp >= 4 + kDqWarps && warp < 4 + kDqWarps + kEpiWarps) {
    // ---------------- epilogue: TMEM (lane = weight row, column = token) -> fp32 reductions ----------------
    const int q = warp & 3;                       // TMEM lane quarter this warp may access
    const int chalf = (warp - 4 - kDqWarps) >> 2;  // which half of the token columns
    int seg = 0;
    bool ok = true;
    // segment ends: the last unit of every weight tile in the span, and the span's last unit
    for (int u = u0 + (n_raw - 1 - u0 % n_raw); ok && u0 < u1; u += n_raw) {
      if (u >= u1 - 1) u = u1 - 1;
      const int buf = seg % C::kAccBufs;
      const uint32_t tphase = (uint32_t)(seg / C::kAccBufs) & 1u;
#pragma unroll
      for (int is = 0; is < kIssuers; ++is)
        if (ok && !mbar_wait_relaxed(tfull(is, buf), tphase, abort_flag)) ok = false;
      ok = __all_sync(0xffffffffu, ok) != 0;  // one outcome for the warp, and the lanes back together before the tensor-memory loads
      if (!ok) break;
      tc_fence_after();
      const int f = (u / n_raw) * kWRows + q * 32 + lane;
#pragma unroll 1
      for (int c = chalf * (NT / 2); c < (chalf + 1) * (NT / 2); c += 16) {
        if (c >= M) break;
        float sum[16];
#pragma unroll
        for (int is = 0; is < kIssuers; ++is) {
          uint32_t r[16];
          tc_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(C::kAccCol + (is * C::kAccBufs + buf) * NT + c), r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) sum[j] = is ? sum[j] + __uint_as_float(r[j]) : __uint_as_float(r[j]);
        }
        if (f < N) {
          float* dst = acc + (size_t)c * ldc + f;
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c + j < M) atomicAdd(dst + (size_t)j * ldc, sum[j]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty(buf));
      ++seg;
      if (u == u1 - 1) break;
    }
  }

  // ---------------- teardown ----------------
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && status) atomicExch(status, 2 | (2 << 8));  // low byte 2: a bounded wait expired; next byte: which kernel family
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols) : "memory");
  }
}

// acc fp32 [m, n] -> bf16 (+ bias), or SwiGLU over rows interleaved in blocks of 32 (32 gate columns
// then the 32 matching up columns); acc is left zeroed for the next accumulation.
__global__ void qlinear_finish_kernel(float* __restrict__ acc, const float* __restrict__ bias, __nv_bfloat16* __restrict__ out,
                                      int m, int n, int ld_acc, int ldc, int swiglu) {
  lg::pdl_prologue();
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
                  int w_static, int* status, cudaStream_t stream) {
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
  const int slots = sm_count();
  // spans that end at tile boundaries leave no fp32 reductions in flight for the next kernel to wait on.
  // Above 32 rows that is worth more than the even split when the tiles still spread over the SMs
  // (a 64-row decode step of the hybrid model: 4.77 against 4.89 ms); at up to 32 rows and for matrices
  // of a few tiles or of many waves the even split wins
  const int whole = (lg::deterministic() || (m > 32 && n_tiles >= 32 && n_tiles <= 4 * slots)) ? 1 : 0;
  const long work = whole ? (long)n_tiles : total;
  const int grid = work < slots ? (int)work : slots;
  lg::launch(kern, grid, dim3(kQThreads), QCfg<NT>::kSmem, stream, ma, mc, ms, acc, m, n, ldc, n_raw, (int)total, whole, w_static, status);
  return lg::launch_status();
}

}  // namespace

extern "C" {

static uint32_t qlinear_acc(const void* a, const void* codes, const void* scales, void* acc, int32_t m, int32_t n, int32_t k,
                            int32_t lda, int32_t ldc, int w_static, void* status_i32, void* stream) {
  lg::LaunchScope launch_scope_;
  if (m <= 0 || m > 256 || n <= 0 || k <= 0 || (k % kRawK) || (lda % 8) || lda < k || ldc < n) return lg::kInvalidValue;
  if (((uintptr_t)a & 15) || ((uintptr_t)codes & 15) || ((uintptr_t)scales & 15) || ((uintptr_t)acc & 3)) return lg::kInvalidValue;
  if ((k / 2) % 16 || ((k / 32) * 2) % 16) return lg::kInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  int* st = (int*)status_i32;
  // token tiles of at most 128: beyond that the weights are streamed once per tile (the second pass
  // is served by L2 for the per-layer matrices)
  for (int t0 = 0; t0 < m; t0 += 128) {
    const int mt = m - t0 < 128 ? m - t0 : 128;
    const void* at = (const uint16_t*)a + (size_t)t0 * lda;
    float* o = (float*)acc + (size_t)t0 * ldc;
    const uint32_t rc = mt <= 32   ? launch_q<32>(at, codes, scales, o, mt, n, k, lda, ldc, w_static, st, s)
                        : mt <= 64 ? launch_q<64>(at, codes, scales, o, mt, n, k, lda, ldc, w_static, st, s)
                                   : launch_q<128>(at, codes, scales, o, mt, n, k, lda, ldc, w_static, st, s);
    if (rc) return rc;
  }
  return 0;
}

uint32_t logismos_launch_qlinear_int4_g32_acc_f32(const void* a, const void* codes, const void* scales, void* acc, int32_t m,
                                                  int32_t n, int32_t k, int32_t lda, int32_t ldc, void* status_i32,
                                                  void* stream) {
  return qlinear_acc(a, codes, scales, acc, m, n, k, lda, ldc, 0, status_i32, stream);
}

uint32_t logismos_launch_qlinear_int4_g32_acc_f32_static(const void* a, const void* codes, const void* scales, void* acc,
                                                         int32_t m, int32_t n, int32_t k, int32_t lda, int32_t ldc,
                                                         void* status_i32, void* stream) {
  return qlinear_acc(a, codes, scales, acc, m, n, k, lda, ldc, 1, status_i32, stream);
}

uint32_t logismos_launch_qlinear_finish_bf16(void* acc, const void* bias, void* out, int32_t m, int32_t n, int32_t ld_acc,
                                             int32_t ldc, int32_t swiglu, void* stream) {
  lg::LaunchScope launch_scope_;
  if (m < 0 || n <= 0 || (n % (swiglu ? 64 : 4)) || ld_acc < n || (ld_acc % 4) || (ldc % 4) || ldc < (swiglu ? n / 2 : n))
    return lg::kInvalidValue;
  if (((uintptr_t)acc & 15) || ((uintptr_t)out & 7)) return lg::kInvalidValue;
  if (m == 0) return 0;
  const int64_t total = (int64_t)m * ((swiglu ? n / 2 : n) / 4);
  lg::launch(qlinear_finish_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, 
      (float*)acc, (const float*)bias, (__nv_bfloat16*)out, m, n, ld_acc, ldc, swiglu);
  return lg::launch_status();
}

}  // extern "C"
