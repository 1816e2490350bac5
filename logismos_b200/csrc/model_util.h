// Helpers shared by the model executors: device buffers, int4 matrices on the device, error macro.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "logismos_kernels.h"
#include "logismos_model.h"

namespace lgm {

void set_error(const std::string& s);

inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

struct Buf {
  void* p = nullptr;
  bool alloc(size_t n) { return cudaMalloc(&p, n ? n : 1) == cudaSuccess; }
  bool upload(const void* src, size_t n) { return alloc(n) && cudaMemcpy(p, src, n, cudaMemcpyHostToDevice) == cudaSuccess; }
  void release() { if (p) cudaFree(p); p = nullptr; }
};

// an int4 matrix on the device; `dense` is its optional bf16 expansion [n, k], made once at load for
// the steps that are bound by tensor throughput rather than by the weight stream
struct QMat { Buf codes, scales, dense; int n = 0, k = 0; };

// expands q into q.dense (blocking); false on allocation or launch failure
inline bool make_dense_copy(QMat& q) {
  if (!q.dense.alloc((size_t)q.n * q.k * 2)) return false;
  if (logismos_launch_dequant_int4_g32_bf16(q.codes.p, q.scales.p, q.dense.p, q.n, q.k, nullptr) != 0) return false;
  return cudaDeviceSynchronize() == cudaSuccess;
}

// gate and up rows interleaved in blocks of 32 (32 gate rows, then the 32 matching up rows), the
// row order the fused SwiGLU epilogue of the GEMM expects
inline bool upload_q_gate_up(QMat& q, const lg_int4_matrix_t& gate, const lg_int4_matrix_t& up, int inter, int k) {
  const size_t cb = (size_t)32 * (k / 2), sb = (size_t)32 * (k / 32);
  std::vector<uint8_t> codes((size_t)2 * inter * (k / 2));
  std::vector<uint16_t> scales((size_t)2 * inter * (k / 32));
  for (int b = 0; b < inter / 32; ++b) {
    std::memcpy(codes.data() + (size_t)(2 * b) * cb, gate.codes + (size_t)b * cb, cb);
    std::memcpy(codes.data() + (size_t)(2 * b + 1) * cb, up.codes + (size_t)b * cb, cb);
    std::memcpy(scales.data() + (size_t)(2 * b) * sb, gate.scales + (size_t)b * sb, sb * 2);
    std::memcpy(scales.data() + (size_t)(2 * b + 1) * sb, up.scales + (size_t)b * sb, sb * 2);
  }
  q.n = 2 * inter;
  q.k = k;
  return q.codes.upload(codes.data(), codes.size()) && q.scales.upload(scales.data(), scales.size() * 2);
}

inline bool upload_q(QMat& q, const std::vector<const lg_int4_matrix_t*>& parts, const std::vector<int>& rows, int k) {
  size_t n = 0;
  for (int r : rows) n += (size_t)r;
  std::vector<uint8_t> codes(n * (k / 2));
  std::vector<uint16_t> scales(n * (k / 32));
  size_t o = 0;
  for (size_t i = 0; i < parts.size(); ++i) {
    std::memcpy(codes.data() + o * (k / 2), parts[i]->codes, (size_t)rows[i] * (k / 2));
    std::memcpy(scales.data() + o * (k / 32), parts[i]->scales, (size_t)rows[i] * (k / 32) * 2);
    o += (size_t)rows[i];
  }
  q.n = (int)n;
  q.k = k;
  return q.codes.upload(codes.data(), codes.size()) && q.scales.upload(scales.data(), scales.size() * 2);
}

// C = A W^T with int4 weights, epilogue as for logismos_launch_linear_t_bf16. Up to 128 rows the
// dequantisation is fused into the tensor-core kernel (fp32 accumulation into the residual stream
// itself, or into the zeroed workspace `accws` finished to bf16); above that the weights are
// expanded to bf16 (the matrix's persistent copy when it has one, else into `wscratch` on every
// call) and the dense GEMM runs with its fused epilogues. The
// crossover is measured: the fused kernel's fp32 reductions grow with rows x columns, and the kernel
// that reads the accumulation target next waits for them to drain (a finishing kernel of 4 us alone
// took 21 us behind a 256-row accumulation).
constexpr int kFusedDequantMaxRows = 128;
inline uint32_t qlinear_any(const void* a, const QMat& w, const void* bias, void* out, int T, int lda, int ldc, int epi,
                            void* wscratch, void* accws, void* status, int* launches, cudaStream_t s) {
  uint32_t rc;
  // with a persistent bf16 copy at hand the dense GEMM (split over k for the narrow output projections)
  // is as fast or faster above 32 rows (measured at 64 / 128 rows: 6.5 / 6.7 us against 6.7 / 8.2 us for
  // 2048 x 2048, 9.5 / 9.8 against 10.7 / 14.6 us for 2048 x 6144, 14-18 against 19-24 us for the wide
  // projections with their finishing pass); below that the int4 stream wins
  const bool fused_ok = T <= kFusedDequantMaxRows && w.k % 256 == 0 && (!w.dense.p || T <= 32);
  if (fused_ok) {
    if (epi == LG_EPI_RESID_F32 && !bias) {
      *launches += 1;
      return logismos_launch_qlinear_int4_g32_acc_f32_static(a, w.codes.p, w.scales.p, out, T, w.n, w.k, lda, ldc, status, s);
    }
    if (epi != LG_EPI_RESID_F32) {
      rc = logismos_launch_qlinear_int4_g32_acc_f32_static(a, w.codes.p, w.scales.p, accws, T, w.n, w.k, lda, w.n, status, s);
      if (rc) return rc;
      *launches += 2;
      return logismos_launch_qlinear_finish_bf16(accws, bias, out, T, w.n, w.n, ldc, epi == LG_EPI_SWIGLU ? 1 : 0, s);
    }
  }
  if (w.dense.p) {
    *launches += 1;
    return logismos_launch_linear_t_bf16(a, w.dense.p, bias, out, T, w.n, w.k, lda, ldc, epi | LG_EPI_STATIC_W, status, s);  // the copy is made once at load
  }
  rc = logismos_launch_dequant_int4_g32_bf16(w.codes.p, w.scales.p, wscratch, w.n, w.k, s);
  if (rc) return rc;
  *launches += 2;
  return logismos_launch_linear_t_bf16(a, wscratch, bias, out, T, w.n, w.k, lda, ldc, epi, status, s);
}

// logits = hidden W^T over the vocabulary and decode::greedy (crates/decode/src/lib.rs:73-83) on
// them. The logits stay fp32 up to the argmax on every route, as in the reference (greedy takes the
// first strict maximum of fp32 logits), so the emitted token does not depend on how many rows the
// step had: up to 16 rows the streaming int4 GEMV stores its fp32 accumulators; above that the
// fused-dequant tensor-core kernel accumulates into the zeroed buffer. `logits` must hold rows * vocab
// floats. *logits_f32 is always 1 (kept for the readers of the buffer).
inline uint32_t lm_head_and_greedy(const QMat& lm_head, const void* hidden_bf16, void* logits, void* tokens, int rows, int hidden,
                                   void* status, int* logits_f32, int* launches, cudaStream_t s) {
  uint32_t rc;
  const int vocab = lm_head.n;
  *logits_f32 = 1;
  if (rows > 16 && hidden % 256 == 0) {
    for (int b0 = 0; b0 < rows; b0 += kFusedDequantMaxRows) {
      const int nb = rows - b0 < kFusedDequantMaxRows ? rows - b0 : kFusedDequantMaxRows;
      float* dst = (float*)logits + (size_t)b0 * vocab;
      if (cudaMemsetAsync(dst, 0, (size_t)nb * vocab * 4, s) != cudaSuccess) return (uint32_t)cudaGetLastError();
      rc = logismos_launch_qlinear_int4_g32_acc_f32_static((const uint16_t*)hidden_bf16 + (size_t)b0 * hidden, lm_head.codes.p,
                                                    lm_head.scales.p, dst, nb, vocab, hidden, hidden, vocab, status, s);
      if (rc) return rc;
      *launches += 1;
    }
  } else {
    for (int b0 = 0; b0 < rows; b0 += 64) {  // the GEMV takes up to 64 rows per launch
      const int nb = rows - b0 < 64 ? rows - b0 : 64;
      rc = logismos_launch_gemv_int4_g32_f32(lm_head.codes.p, lm_head.scales.p, (const uint16_t*)hidden_bf16 + (size_t)b0 * hidden,
                                             (float*)logits + (size_t)b0 * vocab, nb, vocab, hidden, s);
      if (rc) return rc;
      *launches += 1;
    }
  }
  *launches += 1;
  return logismos_launch_greedy_argmax(logits, 1, tokens, rows, vocab, s);
}

}  // namespace lgm

#define LG_TRY(expr, what)                                                                         \
  do {                                                                                             \
    uint32_t rc_ = (uint32_t)(expr);                                                               \
    if (rc_ != 0) {                                                                                \
      char buf_[192];                                                                              \
      std::snprintf(buf_, sizeof(buf_), "%s failed: %s (code %u)", what, cudaGetErrorString((cudaError_t)rc_), rc_); \
      lgm::set_error(buf_);                                                                             \
      return LG_EMB_COMPUTE;                                                                       \
    }                                                                                              \
  } while (0)

