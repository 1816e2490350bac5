// Wrappers shared by the tcgen05 kernels: mbarriers with bounded waits, TMA tile copies, the
// tcgen05 MMA / TMEM instructions, the shared-memory and instruction descriptors, and the host-side
// tensor-map encoder.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace lg {
namespace tc {

// Polls of a bounded wait. A poll suspends for up to about 2 us (the hint of try_wait) or sleeps for
// 40-400 ns, so a wait gives up after 20 ms to 1 s; a legitimate wait inside these kernels lasts
// microseconds.
constexpr uint32_t kSpinLimit = 1u << 19;

// ---- mbarrier / TMA / tcgen05 wrappers --------------------------------------------------------

LG_DEVINL void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
LG_DEVINL void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes));
}
LG_DEVINL void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar));
}
// The suspend-time hint lets a waiting thread sleep in hardware until the phase completes (or the
// hint expires) instead of re-issuing the test, which would take issue slots from working warps.
LG_DEVINL bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(2000u)
      : "memory");
  return ok != 0;
}
// Bounded wait. Returns false when the limit expired or another role already gave up.
LG_DEVINL bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 64) {
      if (*abort_flag) return false;
      __nanosleep(40);
    }
  }
  *abort_flag = 1;
  return false;
}

// The wait of a role with slack: it sleeps between polls from the first miss on, so that many waiting
// warps do not take issue slots from the one thread that feeds the tensor core (a warp that spins on
// try_wait competes for its scheduler like a warp doing arithmetic: with sixteen dequantising warps
// spinning, an MMA-issuing thread was traced at ~100 cycles per instruction). Bounded like mbar_wait.
LG_DEVINL bool mbar_wait_sleep(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t ns = 64) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    __nanosleep(ns);
  }
  *abort_flag = 1;
  return false;
}

// The waits of a role in which the WHOLE warp takes part (all 32 lanes must call). Every lane polls; the
// vote then makes the outcome the same for all of them and, being a warp-wide operation, brings the
// lanes back together: lanes can leave the polling loop in different iterations, and the tensor-memory
// instructions that follow (.sync.aligned) must be executed by the converged warp.
LG_DEVINL bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)) != 0;
}
LG_DEVINL bool mbar_wait_sleep_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t ns = 64) {
  return __all_sync(0xffffffffu, mbar_wait_sleep(bar, parity, abort_flag, ns)) != 0;
}

LG_DEVINL void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      ::"r"(smem_dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// shared -> global bulk tensor store / reduce-add of one staged slab (box given by the tensor map)
LG_DEVINL void tma_store_2d(const CUtensorMap* map, uint32_t smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];\n" ::"l"(map), "r"(smem_src),
               "r"(x), "r"(y)
               : "memory");
}
LG_DEVINL void tma_reduce_add_2d(const CUtensorMap* map, uint32_t smem_src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];\n" ::"l"(map),
               "r"(smem_src), "r"(x), "r"(y)
               : "memory");
}
LG_DEVINL void bulk_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
template <int N>
LG_DEVINL void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(N) : "memory"); }
LG_DEVINL void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }
LG_DEVINL void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// One 32-row slab of 128 bytes per row in the 128-byte-swizzle layout the tensor map expects: the
// 16-byte chunk j of row r sits at chunk position j ^ (r & 7). `slab` is 1024-byte aligned.
LG_DEVINL void slab_write(uint8_t* slab, int row, int chunk, uint4 v) {
  *reinterpret_cast<uint4*>(slab + row * 128 + ((chunk ^ (row & 7)) << 4)) = v;
}

LG_DEVINL void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
LG_DEVINL void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

LG_DEVINL void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar)
               : "memory");
}

LG_DEVINL void tc_mma_bf16(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

LG_DEVINL void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
LG_DEVINL void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
LG_DEVINL void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows of 128 B, 8-row
// swizzle atoms 1024 B apart (stride byte offset), leading byte offset unused (encoded 1),
// descriptor version 1, layout type 2 (SWIZZLE_128B). Addresses are encoded >> 4.
LG_DEVINL uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor for kind::f16: D fp32, A and B bf16, both K-major, M=128, N=BN.
template <int BN>
__host__ __device__ constexpr uint32_t make_idesc() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// ---- host side ------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = (EncodeTiledFn)p;
  return fn;
}

// 2-D tensor [rows, cols] with row stride ld (elements); box = [box_rows, 128 bytes of columns],
// 128-byte swizzle. Operands are bf16 (64 columns per box row); the fp32 output map has 32.
inline bool make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
              bool f32 = false) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  const uint64_t esz = f32 ? 4 : 2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * esz};
  cuuint32_t box[2] = {(cuuint32_t)(128 / esz), box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims,
            strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

inline int sm_count() {
  static int n = 0;
  if (n) return n;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (n <= 0) n = 148;
  return n;
}

}  // namespace tc
}  // namespace lg
