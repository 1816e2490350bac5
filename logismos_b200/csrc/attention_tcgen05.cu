// Ragged-batch attention at head_dim 128 on the 5th-generation tensor cores: the score / softmax / PV
// stage of QwenAttention::forward (crates/transformers/src/attention.rs:226-296, GQA mapping
// :366-382) without materialising scores, the same contract as the mma.sync kernel in attention.cu.
//
// CTA = (128 queries, one query head, one sequence), 6 warps:
//   warp 0      TMA producer: the query tile once, then per block of 128 keys the K tile and the V^T
//               tile (each two [128 x 64] bf16 tiles, 128-byte swizzle), one slot each: K(j+1) lands
//               while the softmax of block j runs, V(j+1) while S(j+1) is computed
//   warp 1      one thread issues tcgen05.mma (cta_group::1, kind::f16, M = 128, N = 128, K = 16):
//               S = Q K^T with both operands in shared memory into TMEM, and O += P V with P read from
//               TMEM (lane = query, one 32-bit column = two keys) and V^T from shared memory
//   warps 2-5   online softmax, thread = query row: tcgen05.ld of S, running maximum and sum in fp32,
//               P rounded to bf16 and written over S with tcgen05.st, O rescaled in TMEM only when a
//               row's maximum grew by more than 2^8; at the end O / l to global memory
// One CTA uses 97 KB of shared memory and 256 TMEM columns, so two CTAs share an SM: while one runs its
// softmax on the CUDA cores the other has the tensor cores.
// V is consumed as V^T [kv_head * 128 + d, key] so that the PV product sees a K-major operand like
// every other operand in this library; a small kernel transposes the V columns of qkv into a scratch
// buffer first, every sequence starting at a multiple of 8 keys (the 16-byte rule of TMA) with its
// padding zeroed.
// Every mbarrier wait is bounded; on expiry the kernel raises the status word, lets copies in flight
// land, frees its TMEM and returns. No cluster launch and no multicast.
#include <cuda.h>

#include "common.cuh"
#include "logismos_kernels.h"
#include "tcgen05.cuh"
#include "turbo3.cuh"

namespace {

using namespace lg;
using namespace lg::tc;

constexpr int kTileBytes = 128 * 128;        // one [128 rows x 64 bf16] tile
constexpr int kBars = 8;                     // q_full, k_full, k_empty, v_full, v_empty, s_full, p_full, o_done
constexpr uint32_t kColS = 0, kColO = 128;   // P replaces S in place; O takes HD columns after it

// HD = head_dim, 128 or 256. Q and K: HD / 64 tiles of [128 rows x 64]; V^T: two tiles of [HD rows x 64 keys].
template <int HD> struct Attn {
  static constexpr int kQBytes = (HD / 64) * kTileBytes;
  static constexpr int kKBytes = (HD / 64) * kTileBytes;
  static constexpr int kVTile = HD * 128;
  static constexpr int kVBytes = 2 * kVTile;
  static constexpr size_t kSmem = 1024 + kQBytes + kKBytes + kVBytes + 8 * kBars + 16;  // 97 KB (two CTAs per SM) or 193 KB
  static constexpr uint32_t kTmemCols = HD == 128 ? 256 : 512;
};

LG_DEVINL float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

LG_DEVINL void tc_mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

LG_DEVINL void tc_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
        "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
LG_DEVINL void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

LG_DEVINL int round8(int v) { return (v + 7) & ~7; }

// V columns of qkv -> vt [n_kv * 128, tp] (row = kv head * 128 + d, column = padded key index), and the
// padded start of every sequence -> pstart[n_seqs]. Grid (key blocks of 64, kv heads, sequences).
// Optional halves-RoPE on the q and k heads in the same launch (cpu_f32::rope_halves_in_place,
// crates/kernels/src/cpu_f32/mod.rs:502-547): the blocks after the transposing ones take one
// (token, head, 8 adjacent i) per thread with 128-bit accesses.
struct RopeArgs {
  __nv_bfloat16* qk;      // nullptr: no RoPE blocks
  const float* cosT;      // [max_pos, HD / 2]
  const float* sinT;
  const int* positions;   // [n_tokens]
  int n_tokens, n_rot_heads, max_pos;
  int* status;
};

template <int HD>
LG_DEVINL void rope_block(const RopeArgs& r, int row_stride, int64_t idx) {
  constexpr int half = HD / 2, octs = half / 8;
  const int64_t total = (int64_t)r.n_tokens * r.n_rot_heads * octs;
  if (idx >= total) return;
  const int p = (int)(idx % octs);
  const int h = (int)((idx / octs) % r.n_rot_heads);
  const int t = (int)(idx / ((int64_t)octs * r.n_rot_heads));
  const int pos = r.positions[t];
  if (pos < 0 || pos >= r.max_pos) {  // RopeTable::gather rejects it (rope.rs:57-66)
    if (r.status) atomicExch(r.status, 1);
    return;
  }
  __nv_bfloat16* base = r.qk + (size_t)t * row_stride + h * HD + 8 * p;
  const float4* cp = reinterpret_cast<const float4*>(r.cosT + (size_t)pos * half + 8 * p);
  const float4* sp = reinterpret_cast<const float4*>(r.sinT + (size_t)pos * half + 8 * p);
  const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
  const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  uint4* lo = reinterpret_cast<uint4*>(base);
  uint4* hi = reinterpret_cast<uint4*>(base + half);
  const uint4 a = *lo, b = *hi;
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
  uint32_t ow[4], pw[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x0 = unpack_bf16x2(aw[i]), x1 = unpack_bf16x2(bw[i]);
    ow[i] = pack_bf16x2(x0.x * c[2 * i] - x1.x * sn[2 * i], x0.y * c[2 * i + 1] - x1.y * sn[2 * i + 1]);
    pw[i] = pack_bf16x2(x0.x * sn[2 * i] + x1.x * c[2 * i], x0.y * sn[2 * i + 1] + x1.y * c[2 * i + 1]);
  }
  *lo = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  *hi = make_uint4(pw[0], pw[1], pw[2], pw[3]);
}

// Grid: tx * n_kv * n_seqs transposing blocks (key block of 64, kv head, sequence), then the RoPE blocks.
template <int HD>
__global__ void __launch_bounds__(256)
transpose_v_kernel(const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ cu, __nv_bfloat16* __restrict__ vt,
                   int* __restrict__ pstart, int n_seqs, int row_stride, int v_off, int tp, int tx, int n_kv, RopeArgs rope) {
  lg::pdl_prologue();
  __shared__ __align__(16) __nv_bfloat16 tile[64][HD + 8];
  constexpr int kParts = 256 / HD, kChunks = HD / 8;  // threads per d row; 16-byte chunks per token row
  __shared__ int p0_s;
  const int tid = threadIdx.x;
  const int t_blocks = tx * n_kv * n_seqs;
  if ((int)blockIdx.x >= t_blocks) {
    rope_block<HD>(rope, row_stride, (int64_t)((int)blockIdx.x - t_blocks) * 256 + tid);
    return;
  }
  const int tb = (int)blockIdx.x % tx, kvh = ((int)blockIdx.x / tx) % n_kv, s = (int)blockIdx.x / (tx * n_kv);
  if (tid < 32) {
    int part = 0;
    for (int i = tid; i < s; i += 32) part += round8(cu[i + 1] - cu[i]);
    part += __shfl_xor_sync(0xffffffffu, part, 16);
    part += __shfl_xor_sync(0xffffffffu, part, 8);
    part += __shfl_xor_sync(0xffffffffu, part, 4);
    part += __shfl_xor_sync(0xffffffffu, part, 2);
    part += __shfl_xor_sync(0xffffffffu, part, 1);
    if (tid == 0) p0_s = part;
  }
  __syncthreads();
  const int p0 = p0_s;
  const int t0 = cu[s], len = cu[s + 1] - t0, plen = round8(len);
  if (tb == 0 && kvh == 0 && tid == 0) pstart[s] = p0;
  if (tb == 0 && s == n_seqs - 1) {  // columns after the last sequence are read as padding by the last key block
    const int d = tid / kParts;
    for (int col = p0 + plen + (tid % kParts) * 8; col + 8 <= tp; col += 8 * kParts)
      *reinterpret_cast<uint4*>(vt + (size_t)(kvh * HD + d) * tp + col) = make_uint4(0u, 0u, 0u, 0u);
  }
  if (tb * 64 >= plen) return;
  for (int u = tid; u < 64 * kChunks; u += 256) {
    const int r = u / kChunks, ch = u % kChunks, t = tb * 64 + r;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (t < len) v = __ldg(reinterpret_cast<const uint4*>(qkv + (size_t)(t0 + t) * row_stride + v_off + kvh * HD + ch * 8));
    *reinterpret_cast<uint4*>(&tile[r][ch * 8]) = v;
  }
  __syncthreads();
  const int d = tid / kParts, half = tid % kParts;
#pragma unroll
  for (int g8 = 0; g8 < 8 / kParts; ++g8) {
    const int tl = half * (64 / kParts) + g8 * 8;
    if (tb * 64 + tl < plen) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint16_t lo = *reinterpret_cast<const uint16_t*>(&tile[tl + 2 * i][d]);
        const uint16_t hi = *reinterpret_cast<const uint16_t*>(&tile[tl + 2 * i + 1][d]);
        w[i] = (uint32_t)lo | ((uint32_t)hi << 16);
      }
      *reinterpret_cast<uint4*>(vt + (size_t)(kvh * HD + d) * tp + p0 + tb * 64 + tl) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// The keys and values of sequences that live in the paged cache, made contiguous for the kernel below:
// K rows -> kbuf [tp, n_kv * HD] (row = padded key index), V -> vt [n_kv * HD, tp] transposed as above,
// pstart[s] = padded start of sequence s (every sequence starts at a multiple of 8 keys, padding
// zeroed). Token t of sequence s is read from block tables[s * max_blocks + t / 16], slot t % 16 of
// k_pool / v_pool [n_pool_blocks, 16, n_kv * HD] (the row layout of FlatKvCache,
// crates/cache/src/flat.rs:36-69; the read is KvCache::get, :254-304). A block id outside the pool
// yields zero rows and raises the status word. Grid (key blocks of 64, kv heads, sequences).
template <int HD>
__global__ void __launch_bounds__(256)
gather_paged_kv_kernel(const __nv_bfloat16* __restrict__ kpool, const __nv_bfloat16* __restrict__ vpool,
                       const int* __restrict__ tables, int max_blocks, int n_pool_blocks, const int* __restrict__ kv_lens,
                       __nv_bfloat16* __restrict__ kbuf, __nv_bfloat16* __restrict__ vt, int* __restrict__ pstart, int n_seqs,
                       int tp, int tx, int n_kv, int* __restrict__ status) {
  lg::pdl_prologue();
  __shared__ __align__(16) __nv_bfloat16 tile[64][HD + 8];
  constexpr int kParts = 256 / HD, kChunks = HD / 8;
  __shared__ int p0_s;
  const int tid = threadIdx.x;
  const int tb = (int)blockIdx.x % tx, kvh = ((int)blockIdx.x / tx) % n_kv, s = (int)blockIdx.x / (tx * n_kv);
  if (tid < 32) {
    int part = 0;
    for (int i = tid; i < s; i += 32) part += round8(max(kv_lens[i], 0));
    part += __shfl_xor_sync(0xffffffffu, part, 16);
    part += __shfl_xor_sync(0xffffffffu, part, 8);
    part += __shfl_xor_sync(0xffffffffu, part, 4);
    part += __shfl_xor_sync(0xffffffffu, part, 2);
    part += __shfl_xor_sync(0xffffffffu, part, 1);
    if (tid == 0) p0_s = part;
  }
  __syncthreads();
  const int p0 = p0_s;
  const int len = max(kv_lens[s], 0), plen = round8(len);
  const int row_w = n_kv * HD;
  if (p0 + plen > tp) {  // the caller's total does not cover these lengths: nothing is written
    if (tid == 0 && status) atomicExch(status, 1);
    return;
  }
  if (tb == 0 && kvh == 0 && tid == 0) pstart[s] = p0;
  if (tb == 0 && s == n_seqs - 1) {  // rows / columns after the last sequence are read as padding by the last key block
    const int d = tid / kParts;
    for (int col = p0 + plen + (tid % kParts) * 8; col + 8 <= tp; col += 8 * kParts)
      *reinterpret_cast<uint4*>(vt + (size_t)(kvh * HD + d) * tp + col) = make_uint4(0u, 0u, 0u, 0u);
    for (int u = tid; u < (tp - p0 - plen) * kChunks; u += 256)
      *reinterpret_cast<uint4*>(kbuf + (size_t)(p0 + plen + u / kChunks) * row_w + kvh * HD + (u % kChunks) * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
  if (tb * 64 >= plen) return;
  for (int u = tid; u < 64 * kChunks; u += 256) {
    const int r = u / kChunks, ch = u % kChunks, t = tb * 64 + r;
    uint4 kq = make_uint4(0u, 0u, 0u, 0u), vq = kq;
    if (t < len) {
      const int bi = t >> 4;
      const int blk = bi < max_blocks ? __ldg(tables + (size_t)s * max_blocks + bi) : -1;
      if (blk < 0 || blk >= n_pool_blocks) {
        if (ch == 0 && status) atomicExch(status, 1);
      } else {
        const size_t src = ((size_t)blk * 16 + (t & 15)) * row_w + kvh * HD + ch * 8;
        kq = __ldg(reinterpret_cast<const uint4*>(kpool + src));
        vq = __ldg(reinterpret_cast<const uint4*>(vpool + src));
      }
    }
    if (t < plen) *reinterpret_cast<uint4*>(kbuf + (size_t)(p0 + t) * row_w + kvh * HD + ch * 8) = kq;
    *reinterpret_cast<uint4*>(&tile[r][ch * 8]) = vq;
  }
  __syncthreads();
  const int d = tid / kParts, half = tid % kParts;
#pragma unroll
  for (int g8 = 0; g8 < 8 / kParts; ++g8) {
    const int tl = half * (64 / kParts) + g8 * 8;
    if (tb * 64 + tl < plen) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint16_t lo = *reinterpret_cast<const uint16_t*>(&tile[tl + 2 * i][d]);
        const uint16_t hi = *reinterpret_cast<const uint16_t*>(&tile[tl + 2 * i + 1][d]);
        w[i] = (uint32_t)lo | ((uint32_t)hi << 16);
      }
      *reinterpret_cast<uint4*>(vt + (size_t)(kvh * HD + d) * tp + p0 + tb * 64 + tl) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// The same gather from TurboQuant 3-bit pools (u8 [n_pool_blocks, 16, n_kv * HD / 128 * 56], kvquant.cu):
// every 128-value head chunk of a key is decoded by one warp (decode_turbo3_0_head, crates/quant/src/
// lib.rs:378-413), K chunks go straight to kbuf as bf16, V chunks through the shared tile for the
// transposed write. Same grid, same padding rules.
template <int HD>
__global__ void __launch_bounds__(256)
gather_paged_kv_turbo3_kernel(const uint8_t* __restrict__ kpool, const uint8_t* __restrict__ vpool, const int* __restrict__ tables,
                              int max_blocks, int n_pool_blocks, const int* __restrict__ kv_lens, __nv_bfloat16* __restrict__ kbuf,
                              __nv_bfloat16* __restrict__ vt, int* __restrict__ pstart, int n_seqs, int tp, int tx, int n_kv,
                              int* __restrict__ status) {
  lg::pdl_prologue();
  __shared__ __align__(16) __nv_bfloat16 tile[64][HD + 8];
  __shared__ uint32_t words[8][16];
  constexpr int kParts = 256 / HD, kCh = HD / 128;  // threads per d row; head chunks per key
  __shared__ int p0_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tb = (int)blockIdx.x % tx, kvh = ((int)blockIdx.x / tx) % n_kv, s = (int)blockIdx.x / (tx * n_kv);
  if (tid < 32) {
    int part = 0;
    for (int i = tid; i < s; i += 32) part += round8(max(kv_lens[i], 0));
    part += __shfl_xor_sync(0xffffffffu, part, 16);
    part += __shfl_xor_sync(0xffffffffu, part, 8);
    part += __shfl_xor_sync(0xffffffffu, part, 4);
    part += __shfl_xor_sync(0xffffffffu, part, 2);
    part += __shfl_xor_sync(0xffffffffu, part, 1);
    if (tid == 0) p0_s = part;
  }
  __syncthreads();
  const int p0 = p0_s;
  const int len = max(kv_lens[s], 0), plen = round8(len);
  const int row_w = n_kv * HD, chunks_row = n_kv * kCh;
  if (p0 + plen > tp) {
    if (tid == 0 && status) atomicExch(status, 1);
    return;
  }
  if (tb == 0 && kvh == 0 && tid == 0) pstart[s] = p0;
  if (tb == 0 && s == n_seqs - 1) {
    const int d = tid / kParts;
    for (int col = p0 + plen + (tid % kParts) * 8; col + 8 <= tp; col += 8 * kParts)
      *reinterpret_cast<uint4*>(vt + (size_t)(kvh * HD + d) * tp + col) = make_uint4(0u, 0u, 0u, 0u);
    for (int u = tid; u < (tp - p0 - plen) * (HD / 8); u += 256)
      *reinterpret_cast<uint4*>(kbuf + (size_t)(p0 + plen + u / (HD / 8)) * row_w + kvh * HD + (u % (HD / 8)) * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
  if (tb * 64 >= plen) return;
  // warp tasks: (key r of the tile, head chunk c, K or V)
  for (int task = warp; task < 64 * kCh * 2; task += 8) {
    const int kv = task & 1, c = (task >> 1) % kCh, r = (task >> 1) / kCh, t = tb * 64 + r;
    float o[4] = {0.f, 0.f, 0.f, 0.f};
    if (t < len) {
      const int bi = t >> 4;
      const int blk = bi < max_blocks ? __ldg(tables + (size_t)s * max_blocks + bi) : -1;
      if (blk < 0 || blk >= n_pool_blocks) {
        if (lane == 0 && status) atomicExch(status, 1);
      } else {
        const uint8_t* src = (kv ? vpool : kpool) + (((size_t)blk * 16 + (t & 15)) * chunks_row + kvh * kCh + c) * lg::t3::kChunkBytes;
        lg::t3::decode_chunk(src, o, words[warp], lane);
      }
    }
    const uint2 pk = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
    if (kv == 0) {
      if (t < plen) *reinterpret_cast<uint2*>(kbuf + (size_t)(p0 + t) * row_w + kvh * HD + c * 128 + lane * 4) = pk;
    } else {
      *reinterpret_cast<uint2*>(&tile[r][c * 128 + lane * 4]) = pk;
    }
  }
  __syncthreads();
  const int d = tid / kParts, half = tid % kParts;
#pragma unroll
  for (int g8 = 0; g8 < 8 / kParts; ++g8) {
    const int tl = half * (64 / kParts) + g8 * 8;
    if (tb * 64 + tl < plen) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint16_t lo = *reinterpret_cast<const uint16_t*>(&tile[tl + 2 * i][d]);
        const uint16_t hi = *reinterpret_cast<const uint16_t*>(&tile[tl + 2 * i + 1][d]);
        w[i] = (uint32_t)lo | ((uint32_t)hi << 16);
      }
      *reinterpret_cast<uint4*>(vt + (size_t)(kvh * HD + d) * tp + p0 + tb * 64 + tl) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

template <bool CAUSAL, int HD>
__global__ void __launch_bounds__(192, HD == 128 ? 2 : 1)
attn_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_vt, const int* __restrict__ cu, const int* __restrict__ pstart,
                    const int* __restrict__ kv_lens, __nv_bfloat16* __restrict__ out, int n_heads, int n_kv, int k_off,
                    float sl2, int* __restrict__ status) {
  lg::pdl_prologue();
  using C = Attn<HD>;
  constexpr int kQBytes = C::kQBytes, kKBytes = C::kKBytes, kVBytes = C::kVBytes, kVTile = C::kVTile;
  constexpr uint32_t kTmemCols = C::kTmemCols;
  // causal: the query tiles with the most keys start first
  const int s = blockIdx.z, h = blockIdx.y, q0 = (CAUSAL ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x) * 128;
  const int t0 = cu[s], len = cu[s + 1] - t0;
  if (q0 >= len) return;  // before any barrier or TMEM allocation
  // kv_lens == nullptr: the keys are the sequence's own token rows (map_k is map_q). Otherwise the
  // sequence has kv_lens[s] >= len keys in a gathered buffer whose rows start at pstart[s] (the cached
  // prefix followed by the new tokens), and query i stands at position kv_lens[s] - len + i.
  const int kv_total = kv_lens ? kv_lens[s] : len;
  const int q_off = kv_total - len;
  if (q_off < 0) {  // fewer keys than queries: not a causal continuation
    if (threadIdx.x == 0 && status) atomicExch(status, 1);
    return;
  }
  const int k_row0 = kv_lens ? pstart[s] : t0;
  const int kvh = h / (n_heads / n_kv);
  const int kv_len = CAUSAL ? min(kv_total, q_off + q0 + 128) : kv_total;
  const int nb = (kv_len + 127) >> 7;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_smem = smem_base, k_smem = smem_base + kQBytes, v_smem = k_smem + kKBytes;
  const uint32_t bars = v_smem + kVBytes;
  uint8_t* bars_gen = smem_gen + kQBytes + kKBytes + kVBytes;
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  const uint32_t q_full = bar(0), k_full = bar(1), k_empty = bar(2), v_full = bar(3), v_empty = bar(4);
  const uint32_t s_full = bar(5), p_full = bar(6), o_done = bar(7);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * kBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_gen + 8 * kBars + 8);

  if (threadIdx.x == 0) {
    for (int i = 0; i < kBars; ++i) mbar_init(bar(i), i == 6 ? 4u : 1u);  // p_full: one arrival per softmax warp
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32((const void*)tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer: K(j) as soon as S(j-1) has read its slot, V(j) once PV(j-1) has ----------------
    if (lane == 0) {
      mbar_expect_tx(q_full, (uint32_t)kQBytes);
#pragma unroll
      for (int i = 0; i < HD / 64; ++i) tma_load_2d(q_smem + i * kTileBytes, &map_q, q_full, h * HD + i * 64, t0 + q0);
      const int pv = pstart[s];
      for (int j = 0; j < nb; ++j) {
        const uint32_t phase = (uint32_t)j & 1u;
        if (!mbar_wait(k_empty, phase ^ 1u, abort_flag)) break;
        mbar_expect_tx(k_full, (uint32_t)kKBytes);
#pragma unroll
        for (int i = 0; i < HD / 64; ++i) tma_load_2d(k_smem + i * kTileBytes, &map_k, k_full, k_off + kvh * HD + i * 64, k_row0 + j * 128);
        if (!mbar_wait(v_empty, phase ^ 1u, abort_flag)) break;
        mbar_expect_tx(v_full, (uint32_t)kVBytes);
        tma_load_2d(v_smem, &map_vt, v_full, pv + j * 128, kvh * HD);
        tma_load_2d(v_smem + kVTile, &map_vt, v_full, pv + j * 128 + 64, kvh * HD);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // The tensor pipe runs the MMAs of one CTA in issue order, so S(j) (issued after PV(j-1)) never
    // overwrites the P columns PV(j-1) still reads, and "S(j) complete" implies "PV(j-1) complete".
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc<128>(), idesc_o = make_idesc<HD>();
      bool ok = mbar_wait(q_full, 0u, abort_flag);
      for (int j = 0; j < nb && ok; ++j) {
        const uint32_t phase = (uint32_t)j & 1u;
        if (!mbar_wait(k_full, phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t da = make_smem_desc(q_smem + (kk >> 2) * kTileBytes) + (uint64_t)(2 * (kk & 3));
          const uint64_t db = make_smem_desc(k_smem + (kk >> 2) * kTileBytes) + (uint64_t)(2 * (kk & 3));
          tc_mma_bf16(tmem_base + kColS, da, db, idesc_s, kk ? 1u : 0u);
        }
        tc_commit(s_full);
        tc_commit(k_empty);
        if (!mbar_wait(p_full, phase, abort_flag)) { ok = false; break; }
        if (!mbar_wait(v_full, phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t db = make_smem_desc(v_smem + (kk >> 2) * kVTile) + (uint64_t)(2 * (kk & 3));
          tc_mma_bf16_ts(tmem_base + kColO, tmem_base + kColS + 8u * kk, db, idesc_o, (j | kk) ? 1u : 0u);
        }
        tc_commit(v_empty);
        if (j == nb - 1) tc_commit(o_done);
      }
    }
  } else {
    // ---------------- softmax and epilogue: thread = query row ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const int row = q * 32 + lane;
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const uint32_t t_s = tmem_base + lane_off + kColS, t_o = tmem_base + lane_off + kColO;
    float m = -1e30f, l = 0.0f;
    bool ok = true;
    for (int j = 0; j < nb; ++j) {
      if (!mbar_wait_warp(s_full, (uint32_t)j & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      // keys this row may see in this block: [0, lim)
      int lim = kv_len - j * 128;
      if (CAUSAL) lim = min(lim, q_off + q0 + row + 1 - j * 128);
      const bool full = lim >= 128;
      float mx = -1e30f;
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        uint32_t ra[32], rb[32];
        tc_ld32(t_s + c2 * 64, ra);
        tc_ld32(t_s + c2 * 64 + 32, rb);
        tc_wait_ld();
        if (full) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(__uint_as_float(ra[i]), __uint_as_float(rb[i])));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (c2 * 64 + i < lim) mx = fmaxf(mx, __uint_as_float(ra[i]));
            if (c2 * 64 + 32 + i < lim) mx = fmaxf(mx, __uint_as_float(rb[i]));
          }
        }
      }
      // The maximum only moves when it would grow by more than 2^8: P then stays below 256 (exact
      // enough in bf16, summed in fp32) and O is rescaled far less often.
      const float cand = mx * sl2;
      float alpha = 1.0f;
      if (cand > m + 8.0f) { alpha = fast_exp2(m - cand); m = cand; }
      float sum = 0.0f;
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        uint32_t ra[32], rb[32], v[32];
        tc_ld32(t_s + c2 * 64, ra);
        tc_ld32(t_s + c2 * 64 + 32, rb);
        tc_wait_ld();
        if (full) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float a0 = fast_exp2(fmaf(__uint_as_float(ra[i]), sl2, -m)), a1 = fast_exp2(fmaf(__uint_as_float(ra[i + 1]), sl2, -m));
            const float b0 = fast_exp2(fmaf(__uint_as_float(rb[i]), sl2, -m)), b1 = fast_exp2(fmaf(__uint_as_float(rb[i + 1]), sl2, -m));
            sum += (a0 + a1) + (b0 + b1);
            v[i >> 1] = pack_bf16x2(a0, a1);
            v[16 + (i >> 1)] = pack_bf16x2(b0, b1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int ka = c2 * 64 + i, kb = ka + 32;
            const float a0 = ka < lim ? fast_exp2(fmaf(__uint_as_float(ra[i]), sl2, -m)) : 0.0f;
            const float a1 = ka + 1 < lim ? fast_exp2(fmaf(__uint_as_float(ra[i + 1]), sl2, -m)) : 0.0f;
            const float b0 = kb < lim ? fast_exp2(fmaf(__uint_as_float(rb[i]), sl2, -m)) : 0.0f;
            const float b1 = kb + 1 < lim ? fast_exp2(fmaf(__uint_as_float(rb[i + 1]), sl2, -m)) : 0.0f;
            sum += (a0 + a1) + (b0 + b1);
            v[i >> 1] = pack_bf16x2(a0, a1);
            v[16 + (i >> 1)] = pack_bf16x2(b0, b1);
          }
        }
        // P takes the place of S: columns [32 c2, 32 c2 + 32) hold keys [64 c2, 64 c2 + 64); the S values
        // they replace (keys [32 c2, 32 c2 + 32)) were read in this or the previous half
        tc_st32(t_s + c2 * 32, v);
      }
      l = l * alpha + sum;
      // S(j) complete means PV(j-1) is complete: O may be rescaled in place
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t r[32];
          tc_ld32(t_o + c * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tc_st32(t_o + c * 32, r);
        }
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && mbar_wait_warp(o_done, 0u, abort_flag)) {
      tc_fence_after();
      const float inv = 1.0f / l;
      const bool store = q0 + row < len;
      __nv_bfloat16* dst = out + (size_t)(t0 + q0 + row) * (size_t)(n_heads * HD) + h * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        tc_ld32(t_o + c * 32, r);
        tc_wait_ld();
        if (store) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + i) = w;
          }
        }
      }
    }
  }

  // ---------------- teardown ----------------
  __syncwarp();
  if (*abort_flag) {
    // a wait expired somewhere: give copies that may still be in flight time to land before the
    // shared memory and TMEM are released, and report
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && status) atomicExch(status, 2 | (3 << 8));  // low byte 2: a bounded wait expired; next byte: which kernel family
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

}  // namespace

namespace {
inline size_t pstart_bytes(int n_seqs) { return ((size_t)n_seqs * 4 + 255) & ~(size_t)255; }
inline int padded_tokens(int n_tokens, int n_seqs) { return (n_tokens + 8 * n_seqs + 7) & ~7; }
}  // namespace

extern "C" {

size_t logismos_varlen_attention_tc_scratch_bytes(int32_t n_tokens, int32_t n_seqs, int32_t n_kv_heads, int32_t head_dim) {
  if (n_tokens < 0 || n_seqs < 0 || n_kv_heads <= 0 || (head_dim != 128 && head_dim != 256)) return 0;
  return pstart_bytes(n_seqs) + (size_t)n_kv_heads * head_dim * (size_t)padded_tokens(n_tokens, n_seqs) * 2;
}

static uint32_t launch_attn_tc(const void* qkv, const void* cu_seqlens, void* out, void* scratch, int32_t n_tokens,
                               int32_t n_seqs, int32_t max_seqlen, int32_t n_heads, int32_t n_kv_heads, int32_t head_dim,
                               int32_t row_stride, int32_t k_off, int32_t v_off, int32_t causal, RopeArgs rope, void* status,
                               void* stream) {
  const int D = head_dim;
  if (n_tokens < 0 || n_seqs < 0 || max_seqlen < 0 || n_heads <= 0 || n_kv_heads <= 0 || (D != 128 && D != 256) ||
      (n_heads % n_kv_heads) || (row_stride % 8) || (k_off % 8) || (v_off % 8) || k_off + n_kv_heads * D > row_stride ||
      v_off + n_kv_heads * D > row_stride || n_heads * D > row_stride || ((uintptr_t)qkv & 15) || ((uintptr_t)out & 15) ||
      !scratch || ((uintptr_t)scratch & 255))
    return lg::kInvalidValue;
  if (rope.qk && (rope.n_rot_heads <= 0 || rope.n_rot_heads * D > row_stride || rope.max_pos <= 0 || !rope.cosT || !rope.sinT ||
                  !rope.positions || (((uintptr_t)rope.cosT | (uintptr_t)rope.sinT) & 15)))
    return lg::kInvalidValue;
  if (n_seqs == 0 || max_seqlen == 0 || n_tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  int* pstart = (int*)scratch;
  __nv_bfloat16* vt = (__nv_bfloat16*)((uint8_t*)scratch + pstart_bytes(n_seqs));
  const int tp = padded_tokens(n_tokens, n_seqs);
  CUtensorMap map_qk, map_vt;
  if (!make_map(&map_qk, qkv, (uint64_t)n_tokens, (uint64_t)row_stride, (uint64_t)row_stride, 128) ||
      !make_map(&map_vt, vt, (uint64_t)n_kv_heads * D, (uint64_t)tp, (uint64_t)tp, (uint32_t)D))
    return lg::kInvalidValue;
  const int max8 = (max_seqlen + 7) & ~7;
  const int tx = (max8 + 63) / 64;
  const int64_t rope_threads = rope.qk ? (int64_t)rope.n_tokens * rope.n_rot_heads * (D / 16) : 0;
  const int64_t blocks = (int64_t)tx * n_kv_heads * n_seqs + (rope_threads + 255) / 256;
  if (blocks > 0x7fffffff) return lg::kInvalidValue;
  if (D == 128)
    lg::launch(transpose_v_kernel<128>, dim3((unsigned)blocks), dim3(256), 0, s, (const __nv_bfloat16*)qkv, (const int*)cu_seqlens, vt, pstart, n_seqs,
                                                             row_stride, v_off, tp, tx, n_kv_heads, rope);
  else
    lg::launch(transpose_v_kernel<256>, dim3((unsigned)blocks), dim3(256), 0, s, (const __nv_bfloat16*)qkv, (const int*)cu_seqlens, vt, pstart, n_seqs,
                                                             row_stride, v_off, tp, tx, n_kv_heads, rope);
  uint32_t rc = lg::launch_status();
  if (rc) return rc;
  const float sl2 = 1.4426950408889634f / sqrtf((float)D);
  dim3 grid((max_seqlen + 127) / 128, n_heads, n_seqs);
  auto launch = [&](auto kern, size_t smem) -> uint32_t {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (uint32_t)e;
    lg::launch(kern, grid, dim3(192), smem, s, map_qk, map_qk, map_vt, (const int*)cu_seqlens, pstart, (const int*)nullptr, (__nv_bfloat16*)out,
                                 n_heads, n_kv_heads, k_off, sl2, (int*)status);
    return lg::launch_status();
  };
  if (D == 128) return causal ? launch(attn_tcgen05_kernel<true, 128>, Attn<128>::kSmem) : launch(attn_tcgen05_kernel<false, 128>, Attn<128>::kSmem);
  return causal ? launch(attn_tcgen05_kernel<true, 256>, Attn<256>::kSmem) : launch(attn_tcgen05_kernel<false, 256>, Attn<256>::kSmem);
}

uint32_t logismos_launch_varlen_attention_tc_bf16(const void* qkv, const void* cu_seqlens, void* out, void* scratch,
                                                  int32_t n_tokens, int32_t n_seqs, int32_t max_seqlen, int32_t n_heads,
                                                  int32_t n_kv_heads, int32_t head_dim, int32_t row_stride, int32_t k_off,
                                                  int32_t v_off, int32_t causal, void* status, void* stream) {
  lg::LaunchScope launch_scope_;
  RopeArgs none{};
  return launch_attn_tc(qkv, cu_seqlens, out, scratch, n_tokens, n_seqs, max_seqlen, n_heads, n_kv_heads, head_dim, row_stride,
                        k_off, v_off, causal, none, status, stream);
}

uint32_t logismos_launch_rope_varlen_attention_tc_bf16(void* qkv, const void* cos_f32, const void* sin_f32, const void* positions,
                                                       int32_t n_rot_heads, int32_t max_pos, const void* cu_seqlens, void* out,
                                                       void* scratch, int32_t n_tokens, int32_t n_seqs, int32_t max_seqlen,
                                                       int32_t n_heads, int32_t n_kv_heads, int32_t head_dim, int32_t row_stride,
                                                       int32_t k_off, int32_t v_off, int32_t causal, void* status, void* stream) {
  lg::LaunchScope launch_scope_;
  if (!qkv) return lg::kInvalidValue;
  RopeArgs r{(__nv_bfloat16*)qkv, (const float*)cos_f32, (const float*)sin_f32, (const int*)positions, n_tokens, n_rot_heads, max_pos,
             (int*)status};
  return launch_attn_tc(qkv, cu_seqlens, out, scratch, n_tokens, n_seqs, max_seqlen, n_heads, n_kv_heads, head_dim, row_stride,
                        k_off, v_off, causal, r, status, stream);
}

size_t logismos_paged_prefix_attention_scratch_bytes(int32_t total_kv_tokens, int32_t n_seqs, int32_t n_kv_heads, int32_t head_dim) {
  if (total_kv_tokens < 0 || n_seqs < 0 || n_kv_heads <= 0 || (head_dim != 128 && head_dim != 256)) return 0;
  return pstart_bytes(n_seqs) + 2 * (size_t)n_kv_heads * head_dim * (size_t)padded_tokens(total_kv_tokens, n_seqs) * 2;
}

static uint32_t launch_prefix_attn(const void* q, int32_t q_row_stride, const void* cu_seqlens_q, const void* kv_lens, const void* k_pool,
                                   const void* v_pool, const void* block_tables, int32_t max_blocks, int32_t n_pool_blocks, void* out,
                                   void* scratch, int32_t n_q_tokens, int32_t total_kv_tokens, int32_t n_seqs, int32_t max_q_len,
                                   int32_t max_kv_len, int32_t n_heads, int32_t n_kv_heads, int32_t head_dim, bool turbo3, void* status,
                                   void* stream) {
  const int D = head_dim;
  if (n_q_tokens < 0 || total_kv_tokens < 0 || n_seqs < 0 || max_q_len < 0 || max_kv_len < 0 || max_blocks <= 0 ||
      n_pool_blocks <= 0 || n_heads <= 0 || n_kv_heads <= 0 || (D != 128 && D != 256) || (n_heads % n_kv_heads) ||
      (q_row_stride % 8) || n_heads * D > q_row_stride || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) ||
      ((uintptr_t)k_pool & (turbo3 ? 7 : 15)) || ((uintptr_t)v_pool & (turbo3 ? 7 : 15)) || !scratch || ((uintptr_t)scratch & 255) || !kv_lens ||
      !block_tables || max_kv_len > total_kv_tokens)
    return lg::kInvalidValue;
  if (n_seqs == 0 || max_q_len == 0 || n_q_tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int tp = padded_tokens(total_kv_tokens, n_seqs);
  const int row_w = n_kv_heads * D;
  int* pstart = (int*)scratch;
  __nv_bfloat16* vt = (__nv_bfloat16*)((uint8_t*)scratch + pstart_bytes(n_seqs));
  __nv_bfloat16* kbuf = vt + (size_t)row_w * tp;
  CUtensorMap map_q, map_k, map_vt;
  if (!make_map(&map_q, q, (uint64_t)n_q_tokens, (uint64_t)q_row_stride, (uint64_t)q_row_stride, 128) ||
      !make_map(&map_k, kbuf, (uint64_t)tp, (uint64_t)row_w, (uint64_t)row_w, 128) ||
      !make_map(&map_vt, vt, (uint64_t)row_w, (uint64_t)tp, (uint64_t)tp, (uint32_t)D))
    return lg::kInvalidValue;
  const int tx = (((max_kv_len + 7) & ~7) + 63) / 64;
  const int64_t blocks = (int64_t)tx * n_kv_heads * n_seqs;
  if (blocks > 0x7fffffff) return lg::kInvalidValue;
  if (blocks > 0) {
    auto go = [&](auto kern, auto* kp, auto* vp) {
      lg::launch(kern, dim3((unsigned)blocks), dim3(256), 0, s, kp, vp, (const int*)block_tables, max_blocks, n_pool_blocks, (const int*)kv_lens, kbuf, vt, pstart,
                                            n_seqs, tp, tx, n_kv_heads, (int*)status);
    };
    if (turbo3) {
      if (D == 128) go(gather_paged_kv_turbo3_kernel<128>, (const uint8_t*)k_pool, (const uint8_t*)v_pool);
      else go(gather_paged_kv_turbo3_kernel<256>, (const uint8_t*)k_pool, (const uint8_t*)v_pool);
    } else {
      if (D == 128) go(gather_paged_kv_kernel<128>, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool);
      else go(gather_paged_kv_kernel<256>, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool);
    }
    uint32_t rc = lg::launch_status();
    if (rc) return rc;
  }
  const float sl2 = 1.4426950408889634f / sqrtf((float)D);
  dim3 grid((max_q_len + 127) / 128, n_heads, n_seqs);
  auto launch = [&](auto kern, size_t smem) -> uint32_t {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (uint32_t)e;
    lg::launch(kern, grid, dim3(192), smem, s, map_q, map_k, map_vt, (const int*)cu_seqlens_q, pstart, (const int*)kv_lens, (__nv_bfloat16*)out,
                                 n_heads, n_kv_heads, 0, sl2, (int*)status);
    return lg::launch_status();
  };
  if (D == 128) return launch(attn_tcgen05_kernel<true, 128>, Attn<128>::kSmem);
  return launch(attn_tcgen05_kernel<true, 256>, Attn<256>::kSmem);
}

uint32_t logismos_launch_paged_prefix_attention_tc_bf16(const void* q, int32_t q_row_stride, const void* cu_seqlens_q,
                                                        const void* kv_lens, const void* k_pool, const void* v_pool,
                                                        const void* block_tables, int32_t max_blocks, int32_t n_pool_blocks,
                                                        void* out, void* scratch, int32_t n_q_tokens, int32_t total_kv_tokens,
                                                        int32_t n_seqs, int32_t max_q_len, int32_t max_kv_len, int32_t n_heads,
                                                        int32_t n_kv_heads, int32_t head_dim, void* status, void* stream) {
  lg::LaunchScope launch_scope_;
  return launch_prefix_attn(q, q_row_stride, cu_seqlens_q, kv_lens, k_pool, v_pool, block_tables, max_blocks, n_pool_blocks, out, scratch,
                            n_q_tokens, total_kv_tokens, n_seqs, max_q_len, max_kv_len, n_heads, n_kv_heads, head_dim, false, status, stream);
}

uint32_t logismos_launch_paged_prefix_attention_turbo3_bf16(const void* q, int32_t q_row_stride, const void* cu_seqlens_q,
                                                            const void* kv_lens, const void* k_pool_t3, const void* v_pool_t3,
                                                            const void* block_tables, int32_t max_blocks, int32_t n_pool_blocks,
                                                            void* out, void* scratch, int32_t n_q_tokens, int32_t total_kv_tokens,
                                                            int32_t n_seqs, int32_t max_q_len, int32_t max_kv_len, int32_t n_heads,
                                                            int32_t n_kv_heads, int32_t head_dim, void* status, void* stream) {
  lg::LaunchScope launch_scope_;
  return launch_prefix_attn(q, q_row_stride, cu_seqlens_q, kv_lens, k_pool_t3, v_pool_t3, block_tables, max_blocks, n_pool_blocks, out,
                            scratch, n_q_tokens, total_kv_tokens, n_seqs, max_q_len, max_kv_len, n_heads, n_kv_heads, head_dim, true, status,
                            stream);
}

}  // extern "C"
