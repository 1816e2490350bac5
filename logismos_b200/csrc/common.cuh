// Shared device helpers for the sm_100a kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LG_DEVINL __device__ __forceinline__

namespace lg {

// Launch status convention of the reference launchers (matmul_launchers.cpp:31): the raw
// runtime status of the launch, read right after it.
inline uint32_t launch_status() { return (uint32_t)cudaGetLastError(); }

// The runtime keeps the status of the last failed call until someone reads it, whoever made that
// call (an earlier API call of this process that was allowed to fail, another library). A launcher
// reports only its own launch, so it drops such a leftover before launching.
struct LaunchScope {
  LaunchScope() { (void)cudaGetLastError(); }
};

// Process-wide switch (logismos_set_deterministic): when set, the launchers give up the k splits whose
// partial sums meet in unordered fp32 reductions, so results are bit-identical from run to run and do
// not depend on how many rows share a launch.
bool deterministic();

// Process-wide switch (logismos_set_dependent_launch, default on): kernels of the model steps are
// launched with programmatic stream serialisation, so that the next kernel of the stream is scheduled
// while the current one drains. The contract every kernel launched through lg::launch keeps:
// pdl_prologue() is the first statement of the kernel, before any access to global memory and before
// any tensor-memory allocation. It first lets the dependent grid be scheduled (its blocks then wait at
// their own prologue) and then blocks until every grid this one depends on has completed and its
// writes are visible. Because each kernel of a chain passes that wait before it can complete,
// completion of the direct predecessor implies completion of everything before it. Allocating tensor
// memory only after the wait matters: a dependent block that took tensor memory before a block of the
// running grid on the same SM had allocated its own would wait for a grid that waits for it.
bool dependent_launch();

LG_DEVINL void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
LG_DEVINL void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
LG_DEVINL void pdl_prologue() {
  pdl_trigger();
  pdl_wait();
}

// kern<<<grid, block, smem, stream>>>(args...) with the programmatic-serialisation attribute when the
// switch is on. The launch status is read by the caller with launch_status(), as after <<<>>>.
template <typename... P, typename... A>
inline void launch(void (*kern)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = dependent_launch() ? 1u : 0u;
  (void)cudaLaunchKernelEx(&cfg, kern, static_cast<P>(args)...);
}

// The same launch without the attribute: an ordinary stream-ordered launch, which starts only after
// everything before it on the stream has completed. The model steps begin with one (the embedding
// lookup), so a kernel of a step may read, ahead of its own dependency wait, anything that earlier
// steps wrote (recurrent states, cached keys and values) besides the static weights.
template <typename... P, typename... A>
inline void launch_ordered(void (*kern)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  (void)cudaLaunchKernelEx(&cfg, kern, static_cast<P>(args)...);
}

// Shape-guard failures are reported as cudaErrorInvalidValue (1) without launching.
constexpr uint32_t kInvalidValue = 1u;

LG_DEVINL float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
LG_DEVINL float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for blockDim.x a multiple of 32 (<= 1024); `red` holds 32 floats.
LG_DEVINL float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.0f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}
LG_DEVINL float block_max(float v, float* red) {
  v = warp_max(v);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  t = warp_max(t);
  __syncthreads();
  return t;
}

LG_DEVINL uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

LG_DEVINL uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
LG_DEVINL float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}

// 16-byte async copy global -> shared, bypassing L1 (data is streamed once).
LG_DEVINL void cp_async16(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gptr));
}
LG_DEVINL void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
LG_DEVINL void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// mma.sync m16n8k16, bf16 inputs, fp32 accumulate: D = A(16x16,row) * B(16x8,col) + C
LG_DEVINL void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2],
                              const float (&c)[4]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%10,%11,%12,%13};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "f"(c[0]), "f"(c[1]),
        "f"(c[2]), "f"(c[3]));
}

LG_DEVINL void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}
LG_DEVINL void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}

}  // namespace lg
