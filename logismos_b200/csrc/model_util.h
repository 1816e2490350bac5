// Helpers shared by the model executors: device buffers, int4 matrices on the device, error macro.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

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

struct QMat { Buf codes, scales; int n = 0, k = 0; };

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

