// CPU oracle, part 1: the fp32 reference kernels.
// Test infrastructure only; see oracle.h for the parity status of each group.
//
// Every function restates crates/kernels/src/cpu_f32/mod.rs of the reference
// (line ranges cited per function), with the same operation order for every
// scalar loop. The GEMM is a blocked single-threaded SGEMM with the calling
// convention of `matrixmultiply::sgemm` (general row/column strides), which is
// what the reference calls at cpu_f32/mod.rs:224 and :318.
#include "oracle.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <vector>

namespace {

typedef float v8f __attribute__((vector_size(32), aligned(4)));

constexpr size_t MR = 6, NR = 16, KC = 256, MC = 96, NC = 2048;

// C[mr,nr] (+)= Apanel[kc][MR] * Bpanel[kc][NR]
inline void micro_kernel(size_t kc, const float* __restrict ap, const float* __restrict bp,
                         float* __restrict c, ptrdiff_t rsc, ptrdiff_t csc, size_t mr, size_t nr,
                         bool accumulate) {
  v8f acc[MR][2];
  for (size_t i = 0; i < MR; ++i) { acc[i][0] = v8f{}; acc[i][1] = v8f{}; }
  for (size_t p = 0; p < kc; ++p) {
    v8f b0, b1;
    std::memcpy(&b0, bp + p * NR, 32);
    std::memcpy(&b1, bp + p * NR + 8, 32);
    const float* a = ap + p * MR;
#pragma GCC unroll 6
    for (size_t i = 0; i < MR; ++i) {
      float ai = a[i];
      v8f av = {ai, ai, ai, ai, ai, ai, ai, ai};
      acc[i][0] += av * b0;
      acc[i][1] += av * b1;
    }
  }
  float tmp[MR][NR];
  for (size_t i = 0; i < MR; ++i) {
    std::memcpy(&tmp[i][0], &acc[i][0], 32);
    std::memcpy(&tmp[i][8], &acc[i][1], 32);
  }
  for (size_t i = 0; i < mr; ++i)
    for (size_t j = 0; j < nr; ++j) {
      float* dst = c + (ptrdiff_t)i * rsc + (ptrdiff_t)j * csc;
      *dst = accumulate ? (*dst + tmp[i][j]) : tmp[i][j];
    }
}

// General-stride single-threaded SGEMM, C = A(m x k) * B(k x n), beta = 0.
void sgemm(size_t m, size_t k, size_t n, const float* a, ptrdiff_t rsa, ptrdiff_t csa,
           const float* b, ptrdiff_t rsb, ptrdiff_t csb, float* c, ptrdiff_t rsc, ptrdiff_t csc) {
  if (m == 0 || n == 0) return;
  if (k == 0) {
    for (size_t i = 0; i < m; ++i)
      for (size_t j = 0; j < n; ++j) c[(ptrdiff_t)i * rsc + (ptrdiff_t)j * csc] = 0.0f;
    return;
  }
  std::vector<float> apack(((MC + MR - 1) / MR) * MR * KC);
  std::vector<float> bpack(((NC + NR - 1) / NR) * NR * KC);
  for (size_t jc = 0; jc < n; jc += NC) {
    size_t nc = std::min(NC, n - jc);
    for (size_t pc = 0; pc < k; pc += KC) {
      size_t kc = std::min(KC, k - pc);
      // pack B[pc:pc+kc, jc:jc+nc] into NR-wide column panels
      for (size_t jr = 0; jr < nc; jr += NR) {
        size_t nr = std::min(NR, nc - jr);
        float* dst = bpack.data() + (jr / NR) * NR * KC;
        for (size_t p = 0; p < kc; ++p) {
          const float* src = b + (ptrdiff_t)(pc + p) * rsb + (ptrdiff_t)(jc + jr) * csb;
          for (size_t j = 0; j < nr; ++j) dst[p * NR + j] = src[(ptrdiff_t)j * csb];
          for (size_t j = nr; j < NR; ++j) dst[p * NR + j] = 0.0f;
        }
      }
      for (size_t ic = 0; ic < m; ic += MC) {
        size_t mc = std::min(MC, m - ic);
        for (size_t ir = 0; ir < mc; ir += MR) {
          size_t mr = std::min(MR, mc - ir);
          float* dst = apack.data() + (ir / MR) * MR * KC;
          for (size_t p = 0; p < kc; ++p) {
            const float* src = a + (ptrdiff_t)(ic + ir) * rsa + (ptrdiff_t)(pc + p) * csa;
            for (size_t i = 0; i < mr; ++i) dst[p * MR + i] = src[(ptrdiff_t)i * rsa];
            for (size_t i = mr; i < MR; ++i) dst[p * MR + i] = 0.0f;
          }
        }
        for (size_t jr = 0; jr < nc; jr += NR) {
          size_t nr = std::min(NR, nc - jr);
          const float* bp = bpack.data() + (jr / NR) * NR * KC;
          for (size_t ir = 0; ir < mc; ir += MR) {
            size_t mr = std::min(MR, mc - ir);
            const float* ap = apack.data() + (ir / MR) * MR * KC;
            micro_kernel(kc, ap, bp, c + (ptrdiff_t)(ic + ir) * rsc + (ptrdiff_t)(jc + jr) * csc,
                         rsc, csc, mr, nr, pc != 0);
          }
        }
      }
    }
  }
}

// checked_shape_len (cpu_f32/mod.rs:60-79): an overflowing product saturates to SIZE_MAX
size_t checked_shape_len(size_t a, size_t b) {
  size_t r;
  if (__builtin_mul_overflow(a, b, &r)) return std::numeric_limits<size_t>::max();
  return r;
}

}  // namespace

extern "C" {

// cpu_f32/mod.rs:106-127. An id >= vocab leaves its row zero; it is not an error.
void orc_embed_lookup(const float* weight, size_t hidden, size_t vocab, const uint32_t* ids,
                      size_t n_ids, float* out) {
  std::memset(out, 0, n_ids * hidden * sizeof(float));
  for (size_t i = 0; i < n_ids; ++i) {
    size_t id = ids[i];
    if (id >= vocab) continue;
    std::memcpy(out + i * hidden, weight + id * hidden, hidden * sizeof(float));
  }
}

// cpu_f32/mod.rs:137-159. Sequential fp32 sum of squares, then x * inv * w.
void orc_rms_norm(const float* x, const float* w, size_t rows, size_t n, float eps, float* y) {
  for (size_t r = 0; r < rows; ++r) {
    const float* row = x + r * n;
    float sum_sq = 0.0f;
    for (size_t j = 0; j < n; ++j) sum_sq += row[j] * row[j];
    float inv = 1.0f / std::sqrt((sum_sq / (float)n) + eps);
    for (size_t j = 0; j < n; ++j) y[r * n + j] = row[j] * inv * w[j];
  }
}

// cpu_f32/mod.rs:183-249. a [m,k], b [k,n], bias [n] or absent. Returns:
// 1 a length mismatch, 2 b length mismatch, 3 bias length mismatch, 4 m*n overflows
// (the four conditions under which the reference panics).
int orc_linear(const float* a, size_t a_len, const float* b, size_t b_len, const float* bias,
               size_t bias_len, size_t m, size_t n, size_t k, float* c) {
  if (a_len != checked_shape_len(m, k)) return 1;
  if (b_len != checked_shape_len(k, n)) return 2;
  if (bias && bias_len != n) return 3;
  size_t mn;
  if (__builtin_mul_overflow(m, n, &mn)) return 4;
  sgemm(m, k, n, a, (ptrdiff_t)k, 1, b, (ptrdiff_t)n, 1, c, (ptrdiff_t)n, 1);
  if (bias)
    for (size_t i = 0; i < m; ++i)
      for (size_t j = 0; j < n; ++j) c[i * n + j] += bias[j];
  return 0;
}

// cpu_f32/mod.rs:271-345. a [m,k], b [n,k] (HF weight, untransposed): B^T expressed by strides.
int orc_linear_t(const float* a, size_t a_len, const float* b, size_t b_len, const float* bias,
                 size_t bias_len, size_t m, size_t n, size_t k, float* c) {
  if (a_len != checked_shape_len(m, k)) return 1;
  if (b_len != checked_shape_len(n, k)) return 2;
  if (bias && bias_len != n) return 3;
  size_t mn;
  if (__builtin_mul_overflow(m, n, &mn)) return 4;
  sgemm(m, k, n, a, (ptrdiff_t)k, 1, b, 1, (ptrdiff_t)k, c, (ptrdiff_t)n, 1);
  if (bias)
    for (size_t i = 0; i < m; ++i)
      for (size_t j = 0; j < n; ++j) c[i * n + j] += bias[j];
  return 0;
}

// cpu_f32/mod.rs:349-351
void orc_silu(const float* x, size_t n, float* y) {
  for (size_t i = 0; i < n; ++i) y[i] = x[i] / (1.0f + std::exp(-x[i]));
}

// cpu_f32/mod.rs:365-374. Mismatched lengths panic in the reference: returns 1.
int orc_hadamard(const float* a, size_t a_len, const float* b, size_t b_len, float* c) {
  if (a_len != b_len) return 1;
  for (size_t i = 0; i < a_len; ++i) c[i] = a[i] * b[i];
  return 0;
}

// cpu_f32/mod.rs:380-433. A row that is all -inf becomes uniform 1/n.
void orc_softmax_last_dim(const float* x, size_t rows, size_t n, float* y) {
  for (size_t r = 0; r < rows; ++r) {
    const float* row = x + r * n;
    float* out = y + r * n;
    float m = -INFINITY;
    for (size_t j = 0; j < n; ++j)
      if (row[j] > m) m = row[j];
    if (std::isinf(m) && m < 0) {
      float uniform = n == 0 ? 0.0f : 1.0f / (float)n;
      for (size_t j = 0; j < n; ++j) out[j] = uniform;
      continue;
    }
    float denom = 0.0f;
    for (size_t j = 0; j < n; ++j) {
      float e = std::exp(row[j] - m);
      out[j] = e;
      denom += e;
    }
    float inv = 1.0f / denom;
    for (size_t j = 0; j < n; ++j) out[j] *= inv;
  }
}

// cpu_f32/mod.rs:451-486. rows must be a whole multiple of mask_rows (returns 1 otherwise,
// where the reference panics); n == 0, rows == 0 or an empty mask is a no-op.
int orc_mask_additive_in_place(float* scores, size_t scores_len, const uint8_t* mask,
                               size_t mask_len, size_t rows, size_t n) {
  (void)scores_len;
  if (n == 0 || rows == 0 || mask_len == 0) return 0;
  size_t mask_rows = mask_len / n;
  if (mask_rows == 0) return 0;
  if (rows % mask_rows != 0) return 1;
  size_t repeat = rows / mask_rows;
  for (size_t mr = 0; mr < mask_rows; ++mr)
    for (size_t rep = 0; rep < repeat; ++rep) {
      size_t r = mr * repeat + rep;
      for (size_t j = 0; j < n; ++j)
        if (mask[mr * n + j] == 0) scores[r * n + j] = -INFINITY;
    }
  return 0;
}

// cpu_f32/mod.rs:502-547. Halves convention; cos/sin are per-row [rows, head_dim/2].
void orc_rope_halves_in_place(float* x, const float* cos, const float* sin, size_t rows,
                              size_t head_dim) {
  size_t half = head_dim / 2;
  for (size_t r = 0; r < rows; ++r) {
    float* row = x + r * head_dim;
    const float* cr = cos + r * half;
    const float* sr = sin + r * half;
    for (size_t i = 0; i < half; ++i) {
      float x0 = row[i], x1 = row[i + half];
      row[i] = x0 * cr[i] - x1 * sr[i];
      row[i + half] = x0 * sr[i] + x1 * cr[i];
    }
  }
}

// cpu_f32/mod.rs:599-619. inv_freq and the angle are evaluated in f64, then cast to f32.
void orc_build_rope_table_f32(size_t seq, size_t head_dim, double theta, float* cos, float* sin) {
  size_t half = head_dim / 2;
  for (size_t pos = 0; pos < seq; ++pos)
    for (size_t i = 0; i < half; ++i) {
      double e = (2.0 * (double)i) / (double)head_dim;
      double inv_freq = std::pow(theta, -e);
      double angle = (double)pos * inv_freq;
      cos[pos * half + i] = (float)std::cos(angle);
      sin[pos * half + i] = (float)std::sin(angle);
    }
}

// cpu_f32/mod.rs:553-577. Denominator 0 leaves the (zero) sums unscaled.
void orc_mean_pool_masked(const float* h, const uint8_t* mask, size_t seq, size_t hidden,
                          float* out) {
  for (size_t j = 0; j < hidden; ++j) out[j] = 0.0f;
  float den = 0.0f;
  for (size_t s = 0; s < seq; ++s) {
    if (mask[s] == 0) continue;
    den += 1.0f;
    for (size_t j = 0; j < hidden; ++j) out[j] += h[s * hidden + j];
  }
  float inv = den > 0.0f ? 1.0f / den : 1.0f;
  for (size_t j = 0; j < hidden; ++j) out[j] *= inv;
}

// cpu_f32/mod.rs:582-591. Norm clamped to 1e-12.
void orc_l2_normalize_in_place(float* v, size_t n) {
  float sq = 0.0f;
  for (size_t i = 0; i < n; ++i) sq += v[i] * v[i];
  float inv = 1.0f / std::max(std::sqrt(sq), 1e-12f);
  for (size_t i = 0; i < n; ++i) v[i] *= inv;
}

}  // extern "C"
