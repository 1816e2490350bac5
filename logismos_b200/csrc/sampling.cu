// The sampling chain on the device: the logit processors and the multinomial sampler of the
// reference's decode crate over fp32 logits [rows, n] (n = 151936 for the decoder configurations),
// in place, one launch per processor so that a chain keeps the reference's free ordering
// (crates/decode/src/chain.rs:33-76):
//   TemperatureScale    crates/decode/src/processors.rs:18-28
//   TopK                :50-82     (k-th largest by radix select on the float bits: exact)
//   TopP                :89-122    (smallest prefix by descending probability whose mass reaches p)
//   MinP                :130-146
//   RepetitionPenalty   :160-181
//   MultinomialSampler  crates/decode/src/sampler.rs:31-58  (the uniform draw is an input)
// The reference sorts the whole vocabulary per step for TopK / TopP; here a row is one CTA that finds
// the cut by a radix select over an order-preserving integer key of the logit, four bits per pass:
// every thread keeps its own 16 bins (count, probability mass) in shared memory (no atomics, a fixed
// summation order: results do not change between runs), the bins are reduced across the block, and one
// thread walks them from the top. Ties at the cut are kept in index order, as the reference's stable
// sort does.
#include "common.cuh"
#include "logismos_kernels.h"

namespace {

using namespace lg;

constexpr int kThreads = 1024;
constexpr int kBins = 16;
constexpr size_t kSelectSmem = (size_t)kBins * kThreads * 8 + 1024;

// larger float <-> larger key; NaN is ordered like -inf (TopK folds NaN to -inf before its sort)
LG_DEVINL uint32_t order_key(float v) {
  if (v != v) v = -INFINITY;
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__global__ void temperature_kernel(float* __restrict__ logits, int64_t total, float t) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) logits[i] = logits[i] / t;  // a true division, as the reference does (not a reciprocal multiply)
}

// one thread per row walks the row's list in order: a token listed twice is penalised twice
__global__ void repetition_penalty_rows_kernel(float* __restrict__ logits, int rows, int n, const uint32_t* __restrict__ tokens,
                                               const int* __restrict__ counts, int max_tokens, float penalty) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  float* l = logits + (size_t)row * n;
  const int c = min(max(counts[row], 0), max_tokens);
  for (int j = 0; j < c; ++j) {
    const uint32_t t = tokens[(size_t)row * max_tokens + j];
    if (t >= (uint32_t)n) continue;
    const float v = l[t];
    l[t] = v > 0.0f ? v / penalty : v * penalty;
  }
}

// block-wide maximum and sum of exp(l - max); finite_only: non-finite logits carry no mass (the sampler)
LG_DEVINL void row_max_sum(const float* __restrict__ l, int n, bool finite_only, float* red, float& mx, float& sum) {
  float m = -INFINITY;
  for (int i = threadIdx.x; i < n; i += kThreads) m = fmaxf(m, l[i]);  // fmaxf ignores NaN, as f32::max does
  mx = block_max(m, red);
  float s = 0.0f;
  for (int i = threadIdx.x; i < n; i += kThreads) {
    const float v = l[i];
    const bool fin = fabsf(v) <= 3.402823466e38f;  // false for inf and NaN
    s += (finite_only && !fin) ? 0.0f : expf(v - mx);
  }
  sum = block_sum(s, red);
}

// Radix select shared by TopK (by count) and TopP (by probability mass). On return *key_out is the
// key at which the cut falls, *above_* what lies strictly above it, *ties the number of elements with
// exactly that key, *none is set when the target was never reached (everything is kept).
template <bool BY_MASS>
LG_DEVINL void radix_select(const float* __restrict__ l, int n, float mx, float inv_sum, float target_mass, uint32_t target_count,
                            uint8_t* smem, uint32_t& key_out, float& above_mass, uint32_t& above_count, uint32_t& ties, bool& none) {
  uint32_t* cnt = reinterpret_cast<uint32_t*>(smem);                       // [kBins][kThreads]
  float* mass = reinterpret_cast<float*>(smem + (size_t)kBins * kThreads * 4);  // [kBins][kThreads]
  __shared__ uint32_t s_prefix, s_cnt_above, s_ties;
  __shared__ float s_mass_above;
  __shared__ int s_none;
  __shared__ uint32_t r_cnt[kBins];
  __shared__ float r_mass[kBins];
  if (threadIdx.x == 0) { s_prefix = 0; s_cnt_above = 0; s_mass_above = 0.0f; s_none = 0; s_ties = 0; }
  __syncthreads();
  for (int shift = 28; shift >= 0; shift -= 4) {
    const uint32_t prefix = s_prefix;
    const uint32_t pmask = shift == 28 ? 0u : (0xffffffffu << (shift + 4));
#pragma unroll
    for (int d = 0; d < kBins; ++d) {
      cnt[d * kThreads + threadIdx.x] = 0;
      if (BY_MASS) mass[d * kThreads + threadIdx.x] = 0.0f;
    }
    for (int i = threadIdx.x; i < n; i += kThreads) {
      const float v = l[i];
      const uint32_t key = order_key(v);
      if ((key & pmask) != prefix) continue;
      const int d = (key >> shift) & 15;
      cnt[d * kThreads + threadIdx.x] += 1;
      if (BY_MASS) mass[d * kThreads + threadIdx.x] += expf(v - mx) * inv_sum;
    }
    __syncthreads();
    {  // two warps per bin, fixed order
      const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
      const int d = warp >> 1, half = warp & 1;
      uint32_t c = 0;
      float m = 0.0f;
      for (int j = 0; j < kThreads / 64; ++j) {
        const int t = half * (kThreads / 2) + j * 32 + lane;
        c += cnt[d * kThreads + t];
        if (BY_MASS) m += mass[d * kThreads + t];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        c += __shfl_xor_sync(0xffffffffu, c, o);
        if (BY_MASS) m += __shfl_xor_sync(0xffffffffu, m, o);
      }
      __syncthreads();
      if (lane == 0 && half == 0) { r_cnt[d] = c; r_mass[d] = m; }
      __syncthreads();
      if (lane == 0 && half == 1) { r_cnt[d] += c; r_mass[d] += m; }
      __syncthreads();
    }
    if (threadIdx.x == 0) {
      int sel = -1;
      uint32_t ca = s_cnt_above;
      float ma = s_mass_above;
      for (int d = kBins - 1; d >= 0; --d) {
        if (r_cnt[d] == 0) continue;
        const bool reached = BY_MASS ? (ma + r_mass[d] >= target_mass) : (ca + r_cnt[d] >= target_count);
        if (reached) { sel = d; break; }
        ca += r_cnt[d];
        ma += r_mass[d];
      }
      if (sel < 0) {
        // the target is beyond the total (p above the rounded total mass): everything is kept; at a later
        // level only rounding can bring us here: settle on the lowest occupied bin
        if (shift == 28) s_none = 1;
        ca = s_cnt_above; ma = s_mass_above;
        for (int d = kBins - 1; d >= 0; --d) {
          if (r_cnt[d] == 0) continue;
          sel = d;
        }
        for (int d = kBins - 1; d > sel; --d) { ca += r_cnt[d]; ma += r_mass[d]; }
        if (sel < 0) sel = 0;
      }
      s_cnt_above = ca;
      s_mass_above = ma;
      s_prefix = prefix | ((uint32_t)sel << shift);
      s_ties = r_cnt[sel];
    }
    __syncthreads();
    if (s_none) break;
  }
  key_out = s_prefix;
  above_mass = s_mass_above;
  above_count = s_cnt_above;
  ties = s_ties;
  none = s_none != 0;
}

// Elements with key == cut, in index order: the first `keep_ties` stay. Tiles of the block size, an
// ordered count across the block per tile.
LG_DEVINL void mask_below_cut(float* __restrict__ l, int n, uint32_t cut, uint32_t ties, uint32_t keep_ties, bool mask_nan) {
  if (keep_ties >= ties) {
    for (int i = threadIdx.x; i < n; i += kThreads) {
      const float v = l[i];
      if (order_key(v) < cut || (mask_nan && v != v)) l[i] = -INFINITY;
    }
    return;
  }
  __shared__ uint32_t s_warp[kThreads / 32];
  __shared__ uint32_t s_base;
  if (threadIdx.x == 0) s_base = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i0 = 0; i0 < n; i0 += kThreads) {
    const int i = i0 + threadIdx.x;
    const float v = i < n ? l[i] : 0.0f;
    const uint32_t key = i < n ? order_key(v) : 0u;
    const bool tie = i < n && key == cut;
    const uint32_t bal = __ballot_sync(0xffffffffu, tie);
    if (lane == 0) s_warp[warp] = __popc(bal);
    __syncthreads();
    uint32_t before = s_base;
    for (int w = 0; w < warp; ++w) before += s_warp[w];
    const uint32_t rank = before + __popc(bal & ((1u << lane) - 1u));
    if (i < n && (key < cut || (tie && rank >= keep_ties) || (mask_nan && v != v))) l[i] = -INFINITY;
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t t = 0;
      for (int w = 0; w < kThreads / 32; ++w) t += s_warp[w];
      s_base += t;
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kThreads)
top_k_kernel(float* __restrict__ logits, int n, int k) {
  extern __shared__ __align__(16) uint8_t smem[];
  float* l = logits + (size_t)blockIdx.x * n;
  uint32_t cut, above_c, ties;
  float above_m;
  bool none;
  radix_select<false>(l, n, 0.0f, 0.0f, 0.0f, (uint32_t)k, smem, cut, above_m, above_c, ties, none);
  // every element tied with the k-th largest survives (the reference masks only `l < threshold`)
  mask_below_cut(l, n, cut, ties, ties, true);
}

__global__ void __launch_bounds__(kThreads)
top_p_kernel(float* __restrict__ logits, int n, float p) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ float red[32];
  __shared__ uint32_t s_keep;
  float* l = logits + (size_t)blockIdx.x * n;
  float mx, sum;
  row_max_sum(l, n, false, red, mx, sum);
  const float inv = sum > 0.0f ? 1.0f / sum : 1.0f;
  uint32_t cut, above_c, ties;
  float above_m;
  bool none;
  radix_select<true>(l, n, mx, inv, p, 0u, smem, cut, above_m, above_c, ties, none);
  if (none) return;  // the mass never reaches p: the reference keeps everything
  if (threadIdx.x == 0) {
    // the tied elements share one probability; they are taken one by one until the mass reaches p
    float q = 0.0f;
    {
      const uint32_t b = (cut & 0x80000000u) ? (cut & 0x7fffffffu) : ~cut;
      q = expf(__uint_as_float(b) - mx) * inv;
    }
    float cum = above_m;
    uint32_t m = 0;
    do { cum += q; ++m; } while (cum < p && m < ties);
    s_keep = m;
  }
  __syncthreads();
  mask_below_cut(l, n, cut, ties, s_keep, false);
}

__global__ void __launch_bounds__(kThreads)
min_p_kernel(float* __restrict__ logits, int n, float p) {
  __shared__ float red[32];
  float* l = logits + (size_t)blockIdx.x * n;
  float mx, sum;
  row_max_sum(l, n, false, red, mx, sum);
  const bool norm = sum > 0.0f;
  const float max_p = norm ? 1.0f / sum : 1.0f;  // exp(0) over the sum
  const float threshold = p * max_p;
  for (int i = threadIdx.x; i < n; i += kThreads) {
    float pr = expf(l[i] - mx);
    if (norm) pr /= sum;
    if (pr < threshold) l[i] = -INFINITY;
  }
}

// MultinomialSampler::sample for a given uniform draw: thread t owns the contiguous slice
// [t c, (t + 1) c) of the row; slice masses are scanned across the block and the thread(s) whose slice
// can hold the draw walk it as the reference does (u < p_i returns i, else u -= p_i).
__global__ void __launch_bounds__(kThreads)
multinomial_kernel(const float* __restrict__ logits, int n, const float* __restrict__ uniforms, uint32_t* __restrict__ out) {
  __shared__ float red[32];
  __shared__ float s_scan[kThreads / 32];
  __shared__ unsigned int s_best;
  const float* l = logits + (size_t)blockIdx.x * n;
  float mx, sum;
  row_max_sum(l, n, true, red, mx, sum);
  if (!(sum > 0.0f)) {  // no mass anywhere: greedy (first strict maximum from -inf, index 0 if none)
    float bv = -INFINITY;
    unsigned int bi = 0xffffffffu;
    for (int i = threadIdx.x; i < n; i += kThreads)
      if (l[i] > bv) { bv = l[i]; bi = (unsigned int)i; }
    if (threadIdx.x == 0) s_best = 0xffffffffu;
    __syncthreads();
    const float m = block_max(bv, red);
    if (bi != 0xffffffffu && bv == m) atomicMin(&s_best, bi);
    __syncthreads();
    if (threadIdx.x == 0) out[blockIdx.x] = s_best == 0xffffffffu ? 0u : s_best;
    return;
  }
  const float u = uniforms[blockIdx.x];
  const int per = (n + kThreads - 1) / kThreads;
  const int i0 = min(threadIdx.x * per, n), i1 = min(i0 + per, n);
  auto prob = [&](int i) {
    const float v = l[i];
    return fabsf(v) <= 3.402823466e38f ? expf(v - mx) / sum : 0.0f;
  };
  float mine = 0.0f;
  for (int i = i0; i < i1; ++i) mine += prob(i);
  // exclusive scan of the slice masses in thread order
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) s_scan[warp] = incl;
  if (threadIdx.x == 0) s_best = 0xffffffffu;
  __syncthreads();
  float base = 0.0f;
  for (int w = 0; w < warp; ++w) base += s_scan[w];
  const float excl = base + incl - mine;
  if (u >= excl && i0 < i1) {
    float r = u - excl;
    bool found = false;
    for (int i = i0; i < i1; ++i) {
      const float pr = prob(i);
      if (r < pr) { atomicMin(&s_best, (unsigned int)i); found = true; break; }
      r -= pr;
    }
    // the scan and the walk round differently: a draw left a hair above this slice belongs to the
    // start of the next one even if that thread's own bound says otherwise
    if (!found && r <= 2e-6f && i1 < n) atomicMin(&s_best, (unsigned int)i1);
  }
  __syncthreads();
  if (threadIdx.x == 0) out[blockIdx.x] = s_best == 0xffffffffu ? (uint32_t)(n - 1) : s_best;
}

}  // namespace

extern "C" {

uint32_t logismos_launch_temperature_f32(void* logits, int32_t rows, int32_t n, float temperature, void* stream) {
  lg::LaunchScope launch_scope_;
  if (rows < 0 || n < 0 || !logits) return lg::kInvalidValue;
  const float t = fmaxf(temperature, 1e-6f);
  if (fabsf(t - 1.0f) < 1e-9f || rows == 0 || n == 0) return 0;
  const int64_t total = (int64_t)rows * n;
  temperature_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((float*)logits, total, t);
  return lg::launch_status();
}

uint32_t logismos_launch_top_k_f32(void* logits, int32_t rows, int32_t n, int32_t k, void* stream) {
  lg::LaunchScope launch_scope_;
  if (rows < 0 || n < 0 || k < 0 || !logits) return lg::kInvalidValue;
  if (k == 0 || k >= n || rows == 0) return 0;
  cudaError_t e = cudaFuncSetAttribute(top_k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSelectSmem);
  if (e != cudaSuccess) return (uint32_t)e;
  top_k_kernel<<<rows, kThreads, kSelectSmem, (cudaStream_t)stream>>>((float*)logits, n, k);
  return lg::launch_status();
}

uint32_t logismos_launch_top_p_f32(void* logits, int32_t rows, int32_t n, float p, void* stream) {
  lg::LaunchScope launch_scope_;
  if (rows < 0 || n < 0 || !logits) return lg::kInvalidValue;
  const float pc = fminf(fmaxf(p, 0.0f), 1.0f);
  if (pc >= 1.0f || rows == 0 || n == 0) return 0;
  cudaError_t e = cudaFuncSetAttribute(top_p_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSelectSmem);
  if (e != cudaSuccess) return (uint32_t)e;
  top_p_kernel<<<rows, kThreads, kSelectSmem, (cudaStream_t)stream>>>((float*)logits, n, pc);
  return lg::launch_status();
}

uint32_t logismos_launch_min_p_f32(void* logits, int32_t rows, int32_t n, float p, void* stream) {
  lg::LaunchScope launch_scope_;
  if (rows < 0 || n < 0 || !logits) return lg::kInvalidValue;
  const float pc = fminf(fmaxf(p, 0.0f), 1.0f);
  if (pc <= 0.0f || rows == 0 || n == 0) return 0;
  min_p_kernel<<<rows, kThreads, 0, (cudaStream_t)stream>>>((float*)logits, n, pc);
  return lg::launch_status();
}

uint32_t logismos_launch_repetition_penalty_f32(void* logits, int32_t rows, int32_t n, const void* tokens_u32,
                                                const void* counts_i32, int32_t max_tokens, float penalty, void* stream) {
  lg::LaunchScope launch_scope_;
  if (rows < 0 || n < 0 || max_tokens < 0 || !logits || (max_tokens > 0 && (!tokens_u32 || !counts_i32))) return lg::kInvalidValue;
  if (fabsf(penalty - 1.0f) < 1e-9f || rows == 0 || n == 0 || max_tokens == 0) return 0;
  repetition_penalty_rows_kernel<<<(rows + 63) / 64, 64, 0, (cudaStream_t)stream>>>((float*)logits, rows, n, (const uint32_t*)tokens_u32,
                                                                                     (const int*)counts_i32, max_tokens, penalty);
  return lg::launch_status();
}

uint32_t logismos_launch_multinomial_f32(const void* logits, int32_t rows, int32_t n, const void* uniforms_f32, void* out_u32,
                                         void* stream) {
  lg::LaunchScope launch_scope_;
  if (rows < 0 || n < 0 || !out_u32 || (rows > 0 && n > 0 && (!logits || !uniforms_f32))) return lg::kInvalidValue;
  if (rows == 0) return 0;
  if (n == 0) return (uint32_t)cudaMemsetAsync(out_u32, 0, (size_t)rows * 4, (cudaStream_t)stream);  // an empty slice samples 0
  multinomial_kernel<<<rows, kThreads, 0, (cudaStream_t)stream>>>((const float*)logits, n, (const float*)uniforms_f32, (uint32_t*)out_u32);
  return lg::launch_status();
}

}  // extern "C"
