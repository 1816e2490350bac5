// The four fp16 launchers of the reference's GPU op stack, retargeted to CUDA / sm_100a with
// unchanged symbols and argument lists (crates/kernels/src/{matmul,rms_norm,softmax,rope}/mod.rs
// extern blocks). Launchers never allocate and never synchronise; they return the raw launch
// status, 0 on success (matmul_launchers.cpp:24-31).
#include <mma.h>

#include "common.cuh"
#include "logismos_kernels.h"

namespace {

using namespace lg;

// One thread per output element, fp32 accumulate in ascending k, 64-bit indexing: the
// correctness anchor (same contract as matmul_naive.hip:14-42).
__global__ void matmul_naive_fp16_kernel(const __half* __restrict__ a, const __half* __restrict__ b,
                                         __half* __restrict__ d, int m, int n, int k) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  const int row = blockIdx.y * blockDim.y + threadIdx.y;
  if (row >= m || col >= n) return;
  float acc = 0.0f;
  for (int kk = 0; kk < k; ++kk)
    acc += __half2float(a[(int64_t)row * k + kk]) * __half2float(b[(int64_t)kk * n + col]);
  d[(int64_t)row * n + col] = __float2half_rn(acc);
}

// Tensor-core variant for M, N, K multiples of 16 (the only case the op layer selects it for,
// crates/praxis/src/matmul.rs:113-117). Each warp owns a 16x16 output tile and walks K with
// mma.sync fragments; a CTA of 4 warps covers a 32x32 block.
__global__ void matmul_tc_fp16_kernel(const __half* __restrict__ a, const __half* __restrict__ b,
                                      __half* __restrict__ d, int m, int n, int k) {
  using namespace nvcuda;
  const int warp = threadIdx.x >> 5;
  const int tile_m = blockIdx.y * 2 + (warp >> 1);
  const int tile_n = blockIdx.x * 2 + (warp & 1);
  if (tile_m * 16 >= m || tile_n * 16 >= n) return;
  wmma::fragment<wmma::matrix_a, 16, 16, 16, __half, wmma::row_major> fa;
  wmma::fragment<wmma::matrix_b, 16, 16, 16, __half, wmma::row_major> fb;
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc;
  wmma::fill_fragment(acc, 0.0f);
  const __half* ap = a + (int64_t)tile_m * 16 * k;
  const __half* bp = b + (int64_t)tile_n * 16;
  for (int kk = 0; kk < k; kk += 16) {
    wmma::load_matrix_sync(fa, ap + kk, k);
    wmma::load_matrix_sync(fb, bp + (int64_t)kk * n, n);
    wmma::mma_sync(acc, fa, fb, acc);
  }
  wmma::fragment<wmma::accumulator, 16, 16, 16, __half> out;
  for (int i = 0; i < acc.num_elements; ++i) out.x[i] = __float2half_rn(acc.x[i]);
  wmma::store_matrix_sync(d + (int64_t)tile_m * 16 * n + tile_n * 16, out, n, wmma::mem_row_major);
}

// y = x * rsqrt(mean(x^2) + eps) * w per row, fp32 statistics (rms_norm.hip:6-56), with a
// warp-shuffle reduction instead of the reference's shared-memory tree.
__global__ void rms_norm_fp16_kernel(const __half* __restrict__ x, const __half* __restrict__ w,
                                     __half* __restrict__ y, int n, float eps) {
  __shared__ float red[32];
  const __half* row = x + (int64_t)blockIdx.x * n;
  __half* out = y + (int64_t)blockIdx.x * n;
  float ss = 0.0f;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    float f = __half2float(row[j]);
    ss += f * f;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)n + eps);
  for (int j = threadIdx.x; j < n; j += blockDim.x)
    out[j] = __float2half_rn(__half2float(row[j]) * inv * __half2float(w[j]));
}

// Row softmax, max-subtracted, fp32. A row that is entirely -inf becomes uniform 1/n, the
// behaviour of both CPU references (softmax/cpu.rs:40-59); the reference's HIP kernel divides
// by a zero sum there (softmax.hip:51-61).
__global__ void softmax_fp16_kernel(const __half* __restrict__ x, __half* __restrict__ y, int n) {
  __shared__ float red[32];
  const __half* row = x + (int64_t)blockIdx.x * n;
  __half* out = y + (int64_t)blockIdx.x * n;
  float mx = -INFINITY;
  for (int j = threadIdx.x; j < n; j += blockDim.x) mx = fmaxf(mx, __half2float(row[j]));
  mx = block_max(mx, red);
  if (mx == -INFINITY) {
    const __half u = __float2half_rn(1.0f / (float)n);
    for (int j = threadIdx.x; j < n; j += blockDim.x) out[j] = u;
    return;
  }
  float s = 0.0f;
  for (int j = threadIdx.x; j < n; j += blockDim.x) s += __expf(__half2float(row[j]) - mx);
  s = block_sum(s, red);
  const float inv = 1.0f / s;
  for (int j = threadIdx.x; j < n; j += blockDim.x)
    out[j] = __float2half_rn(__expf(__half2float(row[j]) - mx) * inv);
}

// In-place interleaved-pair RoPE on (B,S,H,D) fp16 with an fp32 (S,D) table of interleaved
// (cos, sin) pairs (rope.hip:8-43). One thread per pair.
__global__ void rope_fp16_kernel(__half* __restrict__ qk, const float* __restrict__ cs, int seq,
                                 int heads, int head_dim, int64_t total_pairs) {
  const int pairs = head_dim >> 1;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_pairs) return;
  const int i = (int)(idx % pairs);
  const int64_t row = idx / pairs;                // (b*seq + s)*heads + h
  const int s = (int)((row / heads) % seq);
  const float c = cs[(int64_t)s * head_dim + 2 * i], sn = cs[(int64_t)s * head_dim + 2 * i + 1];
  __half2* p = reinterpret_cast<__half2*>(qk + row * head_dim) + i;
  const float2 v = __half22float2(*p);
  *p = __floats2half2_rn(v.x * c - v.y * sn, v.x * sn + v.y * c);
}

// check_matmul_shape (crates/kernels/src/matmul/mod.rs:89-117): all positive and every
// pairwise product within i32.
bool matmul_shape_ok(int m, int n, int k) {
  if (m <= 0 || n <= 0 || k <= 0) return false;
  const int64_t lim = 2147483647ll;
  return (int64_t)m * k <= lim && (int64_t)k * n <= lim && (int64_t)m * n <= lim;
}

}  // namespace

extern "C" {

uint32_t logismos_launch_matmul_naive_fp16(const void* a, const void* b, void* d, int32_t m,
                                           int32_t n, int32_t k, void* stream) {
  lg::LaunchScope launch_scope_;
  if (!matmul_shape_ok(m, n, k)) return lg::kInvalidValue;
  dim3 block(16, 16), grid((n + 15) / 16, (m + 15) / 16);
  matmul_naive_fp16_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(
      (const __half*)a, (const __half*)b, (__half*)d, m, n, k);
  return lg::launch_status();
}

uint32_t logismos_launch_matmul_wmma_fp16(const void* a, const void* b, void* d, int32_t m,
                                          int32_t n, int32_t k, void* stream) {
  lg::LaunchScope launch_scope_;
  if (!matmul_shape_ok(m, n, k) || (m % 16) || (n % 16) || (k % 16)) return lg::kInvalidValue;
  dim3 block(128), grid((n + 31) / 32, (m + 31) / 32);
  matmul_tc_fp16_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(
      (const __half*)a, (const __half*)b, (__half*)d, m, n, k);
  return lg::launch_status();
}

uint32_t logismos_launch_rms_norm_fp16(const void* x, const void* w, void* y, int32_t m, int32_t n,
                                       float eps, void* stream) {
  lg::LaunchScope launch_scope_;
  if (m <= 0 || n <= 0) return lg::kInvalidValue;
  int bs = 32;
  while (bs < n && bs < 256) bs <<= 1;
  rms_norm_fp16_kernel<<<m, bs, 0, (cudaStream_t)stream>>>((const __half*)x, (const __half*)w,
                                                          (__half*)y, n, eps);
  return lg::launch_status();
}

uint32_t logismos_launch_softmax_fp16(const void* x, void* y, int32_t m, int32_t n, void* stream) {
  lg::LaunchScope launch_scope_;
  if (m <= 0 || n <= 0) return lg::kInvalidValue;
  int bs = 32;
  while (bs < n && bs < 256) bs <<= 1;
  softmax_fp16_kernel<<<m, bs, 0, (cudaStream_t)stream>>>((const __half*)x, (__half*)y, n);
  return lg::launch_status();
}

// check_rope_shape (crates/kernels/src/rope/mod.rs:79-132): all positive, the product of the
// four extents within i32 (overflow of the 64-bit product is a rejection, not a wrap).
uint32_t logismos_launch_rope_fp16(void* qk, const void* cos_sin, int32_t batch, int32_t seq,
                                   int32_t heads, int32_t head_dim, void* stream) {
  lg::LaunchScope launch_scope_;
  if (batch <= 0 || seq <= 0 || heads <= 0 || head_dim <= 0 || (head_dim & 1)) return lg::kInvalidValue;
  int64_t total = 1;
  const int32_t dims[4] = {batch, seq, heads, head_dim};
  for (int i = 0; i < 4; ++i)
    if (__builtin_mul_overflow(total, (int64_t)dims[i], &total)) return lg::kInvalidValue;
  if (total > 2147483647ll) return lg::kInvalidValue;
  const int64_t pairs = total / 2;
  const int bs = 256;
  rope_fp16_kernel<<<(unsigned)((pairs + bs - 1) / bs), bs, 0, (cudaStream_t)stream>>>(
      (__half*)qk, (const float*)cos_sin, seq, heads, head_dim, pairs);
  return lg::launch_status();
}

}  // extern "C"
