// TurboQuant 3-bit K/V rows inside the paged cache: the GPU form of encode_turbo3_0_head /
// decode_turbo3_0_head (crates/quant/src/lib.rs:316-413) with fwht_128 (:90-114), the codebook of
// :73-82 and the 14-byte block layout of :130-172 (2-byte little-endian fp16 norm + 12 bytes of 3-bit
// indices, four blocks per 128-value head chunk, the norm repeated in each).
//
// A quantised pool row holds, for one token, `chunks` = n_kv_heads * head_dim / 128 head chunks of 56
// bytes each (against 256 bytes as bf16: 4.57 times smaller), at slot block * 16 + offset like the
// bf16 pools. One warp handles one (token, chunk) of K and of V; a lane holds values 4 lane .. 4 lane + 3.
// The arithmetic follows the reference operation by operation so that the bytes come out identical: the
// sum of squares is accumulated sequentially in index order with separate multiply and add (no fused
// multiply-add), values are divided by the norm, the butterflies of the transform are the reference's
// (lo' = lo + hi, hi' = lo - hi for h = 1, 2, ..., 64) and the nearest centroid is the first minimum.
#include "common.cuh"
#include "logismos_kernels.h"
#include "turbo3.cuh"

namespace {

using namespace lg;
using namespace lg::t3;

__global__ void __launch_bounds__(256)
turbo3_store_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v, int src_stride, uint8_t* __restrict__ kpool,
                    uint8_t* __restrict__ vpool, const int64_t* __restrict__ slots, int n_tokens, int chunks, int64_t n_slots,
                    int* __restrict__ status) {
  lg::pdl_prologue();
  __shared__ float sq[8][128];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t task = (int64_t)blockIdx.x * 8 + warp;  // (token, chunk, k-or-v)
  if (task >= (int64_t)n_tokens * chunks * 2) return;
  const int kv = (int)(task & 1);
  const int chunk = (int)((task >> 1) % chunks), t = (int)((task >> 1) / chunks);
  const int64_t slot = slots[t];
  if (slot < 0 || slot >= n_slots) {
    if (lane == 0 && chunk == 0 && kv == 0 && status) atomicExch(status, 1);
    return;
  }
  const __nv_bfloat16* src = (kv ? v : k) + (size_t)t * src_stride + chunk * 128 + lane * 4;
  const uint2 raw = __ldg(reinterpret_cast<const uint2*>(src));
  const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
  const float val[4] = {a.x, a.y, b.x, b.y};
  encode_chunk(val, (kv ? vpool : kpool) + ((size_t)slot * chunks + chunk) * kChunkBytes, sq[warp], lane);
}

__global__ void __launch_bounds__(256)
turbo3_gather_kernel(const uint8_t* __restrict__ kpool, const uint8_t* __restrict__ vpool, const int* __restrict__ table, int table_len,
                     int len, int chunks, int n_pool_blocks, __nv_bfloat16* __restrict__ kout, __nv_bfloat16* __restrict__ vout,
                     int* __restrict__ status) {
  lg::pdl_prologue();
  __shared__ uint32_t words[8][16];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t task = (int64_t)blockIdx.x * 8 + warp;
  if (task >= (int64_t)len * chunks * 2) return;
  const int kv = (int)(task & 1);
  const int chunk = (int)((task >> 1) % chunks), t = (int)((task >> 1) / chunks);
  const int bi = t >> 4;
  const int blk = bi < table_len ? table[bi] : -1;
  __nv_bfloat16* dst = (kv ? vout : kout) + ((size_t)t * chunks + chunk) * 128 + lane * 4;
  if (blk < 0 || blk >= n_pool_blocks) {
    if (lane == 0 && status) atomicExch(status, 1);
    *reinterpret_cast<uint2*>(dst) = make_uint2(0u, 0u);
    return;
  }
  float o[4];
  decode_chunk((kv ? vpool : kpool) + (((size_t)blk * 16 + (t & 15)) * chunks + chunk) * kChunkBytes, o, words[warp], lane);
  *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
}

}  // namespace

extern "C" {

size_t logismos_turbo3_row_bytes(int32_t row_elems) { return row_elems > 0 && row_elems % 128 == 0 ? (size_t)(row_elems / 128) * kChunkBytes : 0; }

uint32_t logismos_launch_paged_kv_store_turbo3(const void* k_bf16, const void* v_bf16, int32_t src_row_stride, void* k_pool_t3,
                                               void* v_pool_t3, const void* slot_mapping_i64, int32_t n_tokens, int32_t row_elems,
                                               int64_t n_pool_slots, void* status_i32, void* stream) {
  lg::LaunchScope launch_scope_;
  if (n_tokens < 0 || row_elems <= 0 || (row_elems % 128) || (src_row_stride % 4) || src_row_stride < row_elems ||
      ((uintptr_t)k_bf16 & 7) || ((uintptr_t)v_bf16 & 7) || ((uintptr_t)k_pool_t3 & 7) || ((uintptr_t)v_pool_t3 & 7))
    return lg::kInvalidValue;
  if (n_tokens == 0) return 0;
  const int chunks = row_elems / 128;
  const int64_t tasks = (int64_t)n_tokens * chunks * 2;
  lg::launch(turbo3_store_kernel, dim3((unsigned)((tasks + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, 
      (const __nv_bfloat16*)k_bf16, (const __nv_bfloat16*)v_bf16, src_row_stride, (uint8_t*)k_pool_t3, (uint8_t*)v_pool_t3,
      (const int64_t*)slot_mapping_i64, n_tokens, chunks, n_pool_slots, (int*)status_i32);
  return lg::launch_status();
}

uint32_t logismos_launch_paged_kv_gather_turbo3(const void* k_pool_t3, const void* v_pool_t3, const void* block_table_i32,
                                                int32_t table_len, int32_t len, int32_t row_elems, int32_t n_pool_blocks,
                                                void* k_out_bf16, void* v_out_bf16, void* status_i32, void* stream) {
  lg::LaunchScope launch_scope_;
  if (table_len < 0 || len < 0 || row_elems <= 0 || (row_elems % 128) || ((uintptr_t)k_pool_t3 & 7) || ((uintptr_t)v_pool_t3 & 7) ||
      ((uintptr_t)k_out_bf16 & 7) || ((uintptr_t)v_out_bf16 & 7))
    return lg::kInvalidValue;
  if (len == 0) return 0;
  const int chunks = row_elems / 128;
  const int64_t tasks = (int64_t)len * chunks * 2;
  lg::launch(turbo3_gather_kernel, dim3((unsigned)((tasks + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, 
      (const uint8_t*)k_pool_t3, (const uint8_t*)v_pool_t3, (const int*)block_table_i32, table_len, len, chunks, n_pool_blocks,
      (__nv_bfloat16*)k_out_bf16, (__nv_bfloat16*)v_out_bf16, (int*)status_i32);
  return lg::launch_status();
}

}  // extern "C"
