// Gated delta rule, one decode step per (sequence, head): the T = 1 case of
// gated_delta_rule_recurrent_fwd (crates/kernels/src/gated_delta_rule/cpu.rs:92-182) over a
// batch, with the fp32 state [K=128, V=128] (row-major, k rows) updated in place.
//
//   h <- h * exp(g);  hk[v] = sum_k h[k,v] k[k];  vd = beta * (v - hk);
//   h[k,v] += k[k] * vd[v];  o[v] = sum_k h[k,v] * q[k] * scale
//
// The reference walks the 64 KB state three times per token; here each CTA (4 warps) reads it
// once into registers (warp w holds k rows 32w..32w+31 as float4 per lane, i.e. every load and
// store is a full 512-byte row), and the two column sums are reduced across the four warps
// through shared memory. The kernel is bound by the state read + write (128 KB per head).
#include "common.cuh"
#include "logismos_kernels.h"

namespace {

using namespace lg;
constexpr int KD = 128, VD = 128;

__global__ void __launch_bounds__(128)
gdn_decode_step_kernel(float* __restrict__ state, const __nv_bfloat16* __restrict__ q,
                       const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                       const float* __restrict__ g, const float* __restrict__ beta,
                       __nv_bfloat16* __restrict__ o, float scale) {
  lg::pdl_prologue();
  __shared__ float ks[KD], qs[KD];
  __shared__ float4 red[4][32];
  const int64_t sh = blockIdx.x;  // seq * heads + head
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  ks[tid] = __bfloat162float(k[sh * KD + tid]);
  qs[tid] = __bfloat162float(q[sh * KD + tid]);
  const float decay = expf(g[sh]);
  const float bt = beta[sh];
  float* hp = state + sh * (int64_t)(KD * VD) + (int64_t)(warp * 32) * VD + lane * 4;
  float4 h[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) h[i] = *reinterpret_cast<const float4*>(hp + i * VD);
  __syncthreads();
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    h[i].x *= decay; h[i].y *= decay; h[i].z *= decay; h[i].w *= decay;
    const float kk = ks[warp * 32 + i];
    acc.x += h[i].x * kk; acc.y += h[i].y * kk; acc.z += h[i].z * kk; acc.w += h[i].w * kk;
  }
  red[warp][lane] = acc;
  __syncthreads();
  float4 hk = red[0][lane];
#pragma unroll
  for (int w = 1; w < 4; ++w) { const float4 t = red[w][lane]; hk.x += t.x; hk.y += t.y; hk.z += t.z; hk.w += t.w; }
  const uint2 vraw = *reinterpret_cast<const uint2*>(v + sh * VD + lane * 4);
  const float2 v01 = unpack_bf16x2(vraw.x), v23 = unpack_bf16x2(vraw.y);
  const float4 vd = make_float4(bt * (v01.x - hk.x), bt * (v01.y - hk.y), bt * (v23.x - hk.z), bt * (v23.y - hk.w));
  __syncthreads();  // red is reused below
  acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float kk = ks[warp * 32 + i], qq = qs[warp * 32 + i];
    h[i].x += kk * vd.x; h[i].y += kk * vd.y; h[i].z += kk * vd.z; h[i].w += kk * vd.w;
    *reinterpret_cast<float4*>(hp + i * VD) = h[i];
    acc.x += h[i].x * qq * scale; acc.y += h[i].y * qq * scale;
    acc.z += h[i].z * qq * scale; acc.w += h[i].w * qq * scale;
  }
  red[warp][lane] = acc;
  __syncthreads();
  if (warp == 0) {
    float4 ov = red[0][lane];
#pragma unroll
    for (int w = 1; w < 4; ++w) { const float4 t = red[w][lane]; ov.x += t.x; ov.y += t.y; ov.z += t.z; ov.w += t.w; }
    uint2 p;
    p.x = pack_bf16x2(ov.x, ov.y);
    p.y = pack_bf16x2(ov.z, ov.w);
    *reinterpret_cast<uint2*>(o + sh * VD + lane * 4) = p;
  }
}


// The same recurrence over the tokens of each sequence of a ragged batch (prefill, and decode as
// sequences of one token): tokens are taken in order, which is what gated_delta_rule_chunk_fwd
// specifies (the recurrence applied chunk by chunk with the state carried, cpu.rs:201-249).
//
// CTA = (sequence, head, a block of value columns), 128 threads. A thread owns CPT value columns and
// 1/KS of the key rows (CPT x 128/KS floats of state in registers); the KS owners of a column are
// neighbouring lanes and the column sums are log2(KS) shuffles. There is no cross-warp reduction.
// Two shapes are built:
//   <CPT=2, KS=4>  64 columns per CTA: the throughput shape (decode and many sequences). Every read of
//                  k and q from shared memory serves two columns; at decode the kernel moves the
//                  state at 87 % of the measured HBM rate.
//   <CPT=1, KS=4>  32 columns per CTA: the shape for a few long sequences, where the token-serial
//                  dependency chain bounds the prompt (about 0.5 us per token whatever the split: 16
//                  columns with key rows in eighths measured the same) and more CTAs per head fill
//                  the SMs.
// k is read once per token and kept in registers for both passes over the state; the decay is folded
// into the second pass (hk = decay * h^T k). Inputs arrive eight tokens at a time: the k, q, v, z rows
// and gates of the next eight tokens are fetched with cp.async while the current eight are computed,
// so the memory latency is paid once per eight tokens and there are two barriers per eight tokens.
constexpr int kPfChunk = 8;            // tokens per staged chunk

template <int COLS>
struct PfRaw {  // one staged chunk as it arrives from global memory
  __nv_bfloat16 k[kPfChunk][KD], q[kPfChunk][KD];
  __nv_bfloat16 v[kPfChunk][COLS], z[kPfChunk][COLS];
  float g[kPfChunk], beta[kPfChunk];
};

template <int CPT, int KS>
struct PfCfg {
  static constexpr int kRows = KD / KS;                 // key rows per thread: 32 or 16
  static constexpr int kCols = 4 * (32 / KS) * CPT;     // value columns per CTA: 64 or 16
  static constexpr int kPitch = kRows + 4;              // floats between the row blocks of k / q in shared memory
  static constexpr int kParts = VD / kCols;
};

template <int CPT, int KS>
__global__ void __launch_bounds__(128, 4)  // 128 registers at most: four CTAs per SM (130 registers gave three)
gdn_prefill_kernel(float* __restrict__ state, const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                   const __nv_bfloat16* __restrict__ v, const float* __restrict__ g, const float* __restrict__ beta,
                   __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ z, const int* __restrict__ cu,
                   const int* __restrict__ slots, const uint8_t* __restrict__ fresh, int heads, int64_t qkv_stride, float scale,
                   int state_static) {
  // state_static: no kernel still in flight writes the states or the index arrays (they were left by an
  // earlier model step), so the 64 KB of state are read ahead of the dependency wait, while the
  // kernels that produce this step's q, k, v and gates are still running
  lg::pdl_trigger();
  if (!state_static) lg::pdl_wait();
  using C = PfCfg<CPT, KS>;
  constexpr int R = C::kRows, R4 = R / 4;
  __shared__ __align__(16) PfRaw<C::kCols> raw[2];
  __shared__ __align__(16) float kf[kPfChunk][KS * C::kPitch], qf[kPfChunk][KS * C::kPitch];
  const int part = blockIdx.x % C::kParts, sh = blockIdx.x / C::kParts;
  const int seq = sh / heads, head = sh % heads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kq = lane % KS;                                        // block of key rows: R kq .. R kq + R - 1
  const int lcol = CPT * (warp * (32 / KS) + lane / KS);           // first of this thread's columns inside the CTA's block
  const int col = part * C::kCols + lcol;
  const int t0 = cu[seq], t1 = cu[seq + 1];
  if (t1 <= t0) {
    if (state_static) lg::pdl_wait();  // every block passes the wait before it retires
    return;
  }
  const int64_t slot = slots ? slots[seq] : seq;
  float* hp = state + (slot * heads + head) * (int64_t)(KD * VD) + (int64_t)(kq * R) * VD + col;
  const bool zero_start = fresh && fresh[seq];  // a sequence that starts here begins from the zero state
  float h[R][CPT];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    if (CPT == 2) {  // the two columns are adjacent and even-aligned: one 8-byte access
      const float2 x = zero_start ? make_float2(0.f, 0.f) : *reinterpret_cast<const float2*>(hp + i * VD);
      h[i][0] = x.x;
      h[i][CPT - 1] = x.y;
    } else {
#pragma unroll
      for (int c = 0; c < CPT; ++c) h[i][c] = zero_start ? 0.f : hp[i * VD + c];
    }
  }
  if (state_static) lg::pdl_wait();

  // thread tid fetches 16-byte piece (tid % 16) of token (tid / 16) of k and of q; the first threads the
  // 16-byte pieces of the v (and z) slices; threads 0..7 the two gates of token tid
  constexpr int kVPieces = C::kCols / 8;  // 16-byte pieces of one token's v slice: 8 or 2
  auto fetch = [&](int chunk, int buf) {
    const int tb = t0 + chunk * kPfChunk;
    const int tt = tb + (tid >> 4);
    if (tt < t1) {
      const int64_t row = (int64_t)tt * qkv_stride + head * KD + (tid & 15) * 8;
      cp_async16(smem_u32(&raw[buf].k[tid >> 4][(tid & 15) * 8]), k + row);
      cp_async16(smem_u32(&raw[buf].q[tid >> 4][(tid & 15) * 8]), q + row);
    }
    if (tid < kPfChunk * kVPieces) {
      const int tv = tb + tid / kVPieces;
      if (tv < t1) {
        const int64_t row = (int64_t)tv * qkv_stride + head * KD + part * C::kCols + (tid % kVPieces) * 8;
        cp_async16(smem_u32(&raw[buf].v[tid / kVPieces][(tid % kVPieces) * 8]), v + row);
        if (z) cp_async16(smem_u32(&raw[buf].z[tid / kVPieces][(tid % kVPieces) * 8]), z + row);
      }
    }
    if (tid < kPfChunk && tb + tid < t1) {
      raw[buf].g[tid] = g[(int64_t)(tb + tid) * heads + head];
      raw[buf].beta[tid] = beta[(int64_t)(tb + tid) * heads + head];
    }
    cp_async_commit();
  };

  const int n_chunks = (t1 - t0 + kPfChunk - 1) / kPfChunk;
  fetch(0, 0);
  for (int c = 0; c < n_chunks; ++c) {
    const int buf = c & 1;
    cp_async_wait<0>();
    __syncthreads();  // chunk c has landed; everyone is done with chunk c - 1 (kf / qf and its raw buffer)
    if (c + 1 < n_chunks) fetch(c + 1, buf ^ 1);  // lands while chunk c is computed
    // bf16 -> fp32 once per chunk, into the pitched layout the float4 reads want
    const int n_tok = min(kPfChunk, t1 - t0 - c * kPfChunk);
    for (int i = 0; i < n_tok; ++i) {
      kf[i][(tid / R) * C::kPitch + (tid % R)] = __bfloat162float(raw[buf].k[i][tid]);
      qf[i][(tid / R) * C::kPitch + (tid % R)] = __bfloat162float(raw[buf].q[i][tid]);
    }
    __syncthreads();
    for (int i = 0; i < n_tok; ++i) {
      const int t = t0 + c * kPfChunk + i;
      const float decay = expf(raw[buf].g[i]);
      const float b_cur = raw[buf].beta[i];
      float v_cur[CPT];
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) v_cur[cc] = __bfloat162float(raw[buf].v[i][lcol + cc]);
      const float4* k4 = reinterpret_cast<const float4*>(&kf[i][kq * C::kPitch]);
      const float4* q4 = reinterpret_cast<const float4*>(&qf[i][kq * C::kPitch]);
      float4 kk[R4];
#pragma unroll
      for (int j = 0; j < R4; ++j) kk[j] = k4[j];
      // hk = (decay h)^T k = decay (h^T k): the decay joins the state in the second pass
      float acc[4][CPT];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) acc[a][cc] = 0.f;
#pragma unroll
      for (int j = 0; j < R4; ++j)
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          acc[0][cc] += h[4 * j][cc] * kk[j].x;
          acc[1][cc] += h[4 * j + 1][cc] * kk[j].y;
          acc[2][cc] += h[4 * j + 2][cc] * kk[j].z;
          acc[3][cc] += h[4 * j + 3][cc] * kk[j].w;
        }
      float vd[CPT];
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) {
        float hk = (acc[0][cc] + acc[1][cc]) + (acc[2][cc] + acc[3][cc]);
#pragma unroll
        for (int m = 1; m < KS; m <<= 1) hk += __shfl_xor_sync(0xffffffffu, hk, m);
        vd[cc] = b_cur * (v_cur[cc] - decay * hk);
      }
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) acc[a][cc] = 0.f;
#pragma unroll
      for (int j = 0; j < R4; ++j) {
        const float4 qq = q4[j];
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          h[4 * j][cc] = fmaf(h[4 * j][cc], decay, kk[j].x * vd[cc]);
          h[4 * j + 1][cc] = fmaf(h[4 * j + 1][cc], decay, kk[j].y * vd[cc]);
          h[4 * j + 2][cc] = fmaf(h[4 * j + 2][cc], decay, kk[j].z * vd[cc]);
          h[4 * j + 3][cc] = fmaf(h[4 * j + 3][cc], decay, kk[j].w * vd[cc]);
          acc[0][cc] += h[4 * j][cc] * qq.x;
          acc[1][cc] += h[4 * j + 1][cc] * qq.y;
          acc[2][cc] += h[4 * j + 2][cc] * qq.z;
          acc[3][cc] += h[4 * j + 3][cc] * qq.w;
        }
      }
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) {
        float ov = (acc[0][cc] + acc[1][cc]) + (acc[2][cc] + acc[3][cc]);
#pragma unroll
        for (int m = 1; m < KS; m <<= 1) ov += __shfl_xor_sync(0xffffffffu, ov, m);
        ov *= scale;
        if (z) {  // output gate silu(z), fused
          const float zc = __bfloat162float(raw[buf].z[i][lcol + cc]);
          ov *= zc / (1.0f + __expf(-zc));
        }
        if (kq == 0) o[((int64_t)t * heads + head) * VD + col + cc] = __float2bfloat16(ov);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    if (CPT == 2) {
      *reinterpret_cast<float2*>(hp + i * VD) = make_float2(h[i][0], h[i][CPT - 1]);
    } else {
#pragma unroll
      for (int c = 0; c < CPT; ++c) hp[i * VD + c] = h[i][c];
    }
  }
}

// Per (token, head): g = -exp(A_log[h]) * softplus(a + dt_bias[h]) with softplus(x) = x for
// x > 20, beta = sigmoid(b), all fp32; and q, k rows of 128 scaled to unit L2 norm in place
// (l2_norm_in_place, cpu.rs:19-34, norm clamped at 1e-12). One warp per (token, head).
__global__ void gdn_prepare_kernel(__nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                                   const float* __restrict__ a, const float* __restrict__ b,
                                   const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                   float* __restrict__ g, float* __restrict__ beta, int64_t rows, int heads,
                                   int64_t qk_stride, int ab_stride) {
  lg::pdl_prologue();
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    __nv_bfloat16* p = (which ? k : q) + (r / heads) * qk_stride + (r % heads) * KD + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 x01 = unpack_bf16x2(raw.x), x23 = unpack_bf16x2(raw.y);
    float sq = x01.x * x01.x + x01.y * x01.y + x23.x * x23.x + x23.y * x23.y;
    sq = warp_sum(sq);
    const float inv = 1.0f / fmaxf(sqrtf(sq), 1e-12f);
    uint2 w;
    w.x = pack_bf16x2(x01.x * inv, x01.y * inv);
    w.y = pack_bf16x2(x23.x * inv, x23.y * inv);
    *reinterpret_cast<uint2*>(p) = w;
  }
  if (lane == 0) {
    const int h = (int)(r % heads);
    const int64_t ab = (r / heads) * ab_stride + h;
    const float x = a[ab] + dt_bias[h];
    const float sp = x > 20.0f ? x : log1pf(expf(x));
    g[r] = -expf(A_log[h]) * sp;
    beta[r] = 1.0f / (1.0f + expf(-b[ab]));
  }
}

// The same preparation straight from the fp32 accumulation workspace of the input projection
// (columns q | k | v | z | a | b of every token row): one warp per (token, head) normalises q and k in
// fp32, rounds q, k, v, z to bf16 once, computes the gates, and leaves the workspace zeroed.
__global__ void gdn_finish_kernel(float* __restrict__ acc, int64_t ld_acc, const float* __restrict__ A_log,
                                  const float* __restrict__ dt_bias, __nv_bfloat16* __restrict__ proj, int64_t ld_proj,
                                  float* __restrict__ g, float* __restrict__ beta, int64_t rows, int heads) {
  lg::pdl_prologue();
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const int64_t t = r / heads;
  const int h = (int)(r % heads);
  const int w = heads * KD;
  float* arow = acc + t * ld_acc + h * KD + lane * 4;
  __nv_bfloat16* prow = proj + t * ld_proj + h * KD + lane * 4;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int which = 0; which < 4; ++which) {  // q, k, v, z
    float4* src = reinterpret_cast<float4*>(arow + which * w);
    float4 x = *src;
    *src = zero;
    if (which < 2) {
      const float sq = warp_sum(x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w);
      const float inv = 1.0f / fmaxf(sqrtf(sq), 1e-12f);
      x.x *= inv; x.y *= inv; x.z *= inv; x.w *= inv;
    }
    uint2 o;
    o.x = pack_bf16x2(x.x, x.y);
    o.y = pack_bf16x2(x.z, x.w);
    *reinterpret_cast<uint2*>(prow + which * w) = o;
  }
  if (lane == 0) {
    float* ab = acc + t * ld_acc + 4 * w;
    const float x = ab[h] + dt_bias[h];
    const float sp = x > 20.0f ? x : log1pf(expf(x));
    g[r] = -expf(A_log[h]) * sp;
    beta[r] = 1.0f / (1.0f + expf(-ab[heads + h]));
    ab[h] = 0.0f;
    ab[heads + h] = 0.0f;
  }
}


// One decode token per sequence straight from the fp32 accumulation workspace of the input projection:
// gdn_finish_kernel and the <2, 4> shape of gdn_prefill_kernel in one launch, with the same arithmetic
// in the same order (fp32 L2 norms over float4 pieces and a warp butterfly, one bf16 rounding of q, k,
// v, z, the gates, then the recurrence), so a pure decode step gives the bits of the two-launch route.
// CTA = (sequence, head, half of the value columns), 128 threads. The 64 KB of state are read ahead of
// the dependency wait (they date from an earlier step). The two CTAs of a (sequence, head) both read
// its q, k, a, b; each zeroes its own v and z columns, and the one that arrives second at the pair's
// counter zeroes the shared columns and resets the counter.
__global__ void __launch_bounds__(128, 4)  // 128 registers at most: four CTAs per SM (130 registers gave three)
gdn_decode_fused_kernel(float* __restrict__ state, float* __restrict__ acc, int64_t ld_acc, const float* __restrict__ A_log,
                        const float* __restrict__ dt_bias, __nv_bfloat16* __restrict__ o, const int* __restrict__ slots,
                        const uint8_t* __restrict__ fresh, int* __restrict__ pair_count, int heads, float scale) {
  lg::pdl_trigger();
  using C = PfCfg<2, 4>;
  constexpr int R = C::kRows, R4 = R / 4, KS = 4, CPT = 2;
  __shared__ __align__(16) float kf[KS * C::kPitch], qf[KS * C::kPitch];
  __shared__ float vs[C::kCols], zs[C::kCols];
  __shared__ float gate_s[2];
  __shared__ int last_s;
  const int part = blockIdx.x % C::kParts, sh = blockIdx.x / C::kParts;
  const int seq = sh / heads, head = sh % heads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kq = lane % KS;
  const int lcol = CPT * (warp * (32 / KS) + lane / KS);
  const int col = part * C::kCols + lcol;
  const int64_t slot = slots ? slots[seq] : seq;
  float* hp = state + (slot * heads + head) * (int64_t)(KD * VD) + (int64_t)(kq * R) * VD + col;
  const bool zero_start = fresh && fresh[seq];
  float h[R][CPT];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const float2 x = zero_start ? make_float2(0.f, 0.f) : *reinterpret_cast<const float2*>(hp + i * VD);
    h[i][0] = x.x;
    h[i][1] = x.y;
  }
  lg::pdl_wait();
  const int w = heads * KD;
  float* arow = acc + (int64_t)seq * ld_acc;
  if (warp < 2) {  // q (warp 0) and k (warp 1): unit L2 norm in fp32, one bf16 rounding, into the pitched layout
    const float4 x0 = *reinterpret_cast<const float4*>(arow + warp * w + head * KD + lane * 4);
    float4 x = x0;
    const float sq = warp_sum(x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w);
    const float inv = 1.0f / fmaxf(sqrtf(sq), 1e-12f);
    x.x *= inv; x.y *= inv; x.z *= inv; x.w *= inv;
    const float2 lo = unpack_bf16x2(pack_bf16x2(x.x, x.y)), hi = unpack_bf16x2(pack_bf16x2(x.z, x.w));
    float* dst = (warp == 0 ? qf : kf) + ((lane * 4) / R) * C::kPitch + (lane * 4) % R;
    *reinterpret_cast<float4*>(dst) = make_float4(lo.x, lo.y, hi.x, hi.y);
  } else {  // v (warp 2) and z (warp 3): this CTA's 64 columns, rounded once; the workspace columns are this CTA's to clear
    float* src = arow + (warp == 2 ? 2 : 3) * w + head * KD + part * C::kCols + lane * 2;
    const float2 x = *reinterpret_cast<const float2*>(src);
    *reinterpret_cast<float2*>(src) = make_float2(0.f, 0.f);
    const float2 r = unpack_bf16x2(pack_bf16x2(x.x, x.y));
    float* dst = (warp == 2 ? vs : zs) + lane * 2;
    dst[0] = r.x;
    dst[1] = r.y;
    if (warp == 2 && lane == 0) {
      const float* ab = arow + 4 * w;
      const float x = ab[head] + dt_bias[head];
      const float sp = x > 20.0f ? x : log1pf(expf(x));
      gate_s[0] = -expf(A_log[head]) * sp;
      gate_s[1] = 1.0f / (1.0f + expf(-ab[heads + head]));
    }
  }
  __syncthreads();  // every read of the shared workspace columns by this CTA is done
  if (tid == 0) {
    // the pair's counter: its round trip stays off the critical path (the result is only needed at the end)
    __threadfence();
    const int old = atomicAdd(pair_count + (int64_t)seq * heads + head, 1);
    last_s = old == C::kParts - 1;
    if (old == C::kParts - 1) pair_count[(int64_t)seq * heads + head] = 0;
  }
  // the recurrence for the one token (gdn_prefill_kernel's loop body)
  const float decay = expf(gate_s[0]);
  const float b_cur = gate_s[1];
  float v_cur[CPT];
#pragma unroll
  for (int cc = 0; cc < CPT; ++cc) v_cur[cc] = vs[lcol + cc];
  const float4* k4 = reinterpret_cast<const float4*>(&kf[kq * C::kPitch]);
  const float4* q4 = reinterpret_cast<const float4*>(&qf[kq * C::kPitch]);
  float4 kk[R4];
#pragma unroll
  for (int j = 0; j < R4; ++j) kk[j] = k4[j];
  float a4[4][CPT];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int cc = 0; cc < CPT; ++cc) a4[a][cc] = 0.f;
#pragma unroll
  for (int j = 0; j < R4; ++j)
#pragma unroll
    for (int cc = 0; cc < CPT; ++cc) {
      a4[0][cc] += h[4 * j][cc] * kk[j].x;
      a4[1][cc] += h[4 * j + 1][cc] * kk[j].y;
      a4[2][cc] += h[4 * j + 2][cc] * kk[j].z;
      a4[3][cc] += h[4 * j + 3][cc] * kk[j].w;
    }
  float vd[CPT];
#pragma unroll
  for (int cc = 0; cc < CPT; ++cc) {
    float hk = (a4[0][cc] + a4[1][cc]) + (a4[2][cc] + a4[3][cc]);
#pragma unroll
    for (int m = 1; m < KS; m <<= 1) hk += __shfl_xor_sync(0xffffffffu, hk, m);
    vd[cc] = b_cur * (v_cur[cc] - decay * hk);
  }
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int cc = 0; cc < CPT; ++cc) a4[a][cc] = 0.f;
#pragma unroll
  for (int j = 0; j < R4; ++j) {
    const float4 qq = q4[j];
#pragma unroll
    for (int cc = 0; cc < CPT; ++cc) {
      h[4 * j][cc] = fmaf(h[4 * j][cc], decay, kk[j].x * vd[cc]);
      h[4 * j + 1][cc] = fmaf(h[4 * j + 1][cc], decay, kk[j].y * vd[cc]);
      h[4 * j + 2][cc] = fmaf(h[4 * j + 2][cc], decay, kk[j].z * vd[cc]);
      h[4 * j + 3][cc] = fmaf(h[4 * j + 3][cc], decay, kk[j].w * vd[cc]);
      a4[0][cc] += h[4 * j][cc] * qq.x;
      a4[1][cc] += h[4 * j + 1][cc] * qq.y;
      a4[2][cc] += h[4 * j + 2][cc] * qq.z;
      a4[3][cc] += h[4 * j + 3][cc] * qq.w;
    }
  }
#pragma unroll
  for (int cc = 0; cc < CPT; ++cc) {
    float ov = (a4[0][cc] + a4[1][cc]) + (a4[2][cc] + a4[3][cc]);
#pragma unroll
    for (int m = 1; m < KS; m <<= 1) ov += __shfl_xor_sync(0xffffffffu, ov, m);
    ov *= scale;
    const float zc = zs[lcol + cc];
    ov *= zc / (1.0f + __expf(-zc));
    if (kq == 0) o[((int64_t)seq * heads + head) * VD + col + cc] = __float2bfloat16(ov);
  }
#pragma unroll
  for (int i = 0; i < R; ++i) *reinterpret_cast<float2*>(hp + i * VD) = make_float2(h[i][0], h[i][1]);
  __syncthreads();
  if (last_s) {  // the other CTA of the pair has read q, k, a, b: clear them for the next accumulation
    arow[head * KD + tid] = 0.f;
    arow[w + head * KD + tid] = 0.f;
    if (tid == 0) {
      arow[4 * w + head] = 0.f;
      arow[4 * w + heads + head] = 0.f;
    }
  }
}

}  // namespace

extern "C" uint32_t logismos_launch_gdn_finish(void* acc, int32_t ld_acc, const void* A_log, const void* dt_bias, void* proj,
                                               int32_t ld_proj, void* g, void* beta, int32_t n_tokens, int32_t heads,
                                               void* stream) {
  lg::LaunchScope launch_scope_;
  const int w = heads * KD;
  if (n_tokens < 0 || heads <= 0 || ld_acc < 4 * w + 2 * heads || (ld_acc % 4) || ld_proj < 4 * w || (ld_proj % 4)) return lg::kInvalidValue;
  if (n_tokens == 0) return 0;
  if (((uintptr_t)acc & 15) || ((uintptr_t)proj & 7)) return lg::kInvalidValue;
  const int64_t rows = (int64_t)n_tokens * heads;
  const int wpb = 8;
  lg::launch(gdn_finish_kernel, dim3((unsigned)((rows + wpb - 1) / wpb)), dim3(wpb * 32), 0, (cudaStream_t)stream, 
      (float*)acc, (int64_t)ld_acc, (const float*)A_log, (const float*)dt_bias, (__nv_bfloat16*)proj, (int64_t)ld_proj, (float*)g,
      (float*)beta, rows, heads);
  return lg::launch_status();
}

extern "C" uint32_t logismos_launch_gdn_decode_from_acc(void* state, void* acc, int32_t ld_acc, const void* A_log, const void* dt_bias,
                                                        void* o, const void* state_slots, const void* fresh, void* pair_count,
                                                        int32_t n_seqs, int32_t heads, float scale, void* stream) {
  lg::LaunchScope launch_scope_;
  const int w = heads * KD;
  if (n_seqs < 0 || heads <= 0 || ld_acc < 4 * w + 2 * heads || (ld_acc % 4) || !pair_count) return lg::kInvalidValue;
  if (n_seqs == 0) return 0;
  if (((uintptr_t)state & 15) || ((uintptr_t)acc & 15) || ((uintptr_t)o & 1) || ((uintptr_t)pair_count & 3)) return lg::kInvalidValue;
  const int64_t ctas = (int64_t)n_seqs * heads * PfCfg<2, 4>::kParts;
  if (ctas > 2147483647ll) return lg::kInvalidValue;
  lg::launch(gdn_decode_fused_kernel, dim3((unsigned)ctas), dim3(128), 0, (cudaStream_t)stream, (float*)state, (float*)acc,
             (int64_t)ld_acc, (const float*)A_log, (const float*)dt_bias, (__nv_bfloat16*)o, (const int*)state_slots,
             (const uint8_t*)fresh, (int*)pair_count, heads, scale);
  return lg::launch_status();
}

extern "C" uint32_t logismos_launch_gdn_decode_step(void* state, const void* q, const void* k, const void* v,
                                                    const void* g, const void* beta, void* o, int32_t n_seqs,
                                                    int32_t heads, float scale, void* stream) {
  lg::LaunchScope launch_scope_;
  if (n_seqs < 0 || heads <= 0) return lg::kInvalidValue;
  if (n_seqs == 0) return 0;
  if (((uintptr_t)state & 15) || ((uintptr_t)v & 7) || ((uintptr_t)o & 7)) return lg::kInvalidValue;
  const int64_t ctas = (int64_t)n_seqs * heads;
  if (ctas > 2147483647ll) return lg::kInvalidValue;
  lg::launch(gdn_decode_step_kernel, dim3((unsigned)ctas), dim3(128), 0, (cudaStream_t)stream, 
      (float*)state, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const float*)g,
      (const float*)beta, (__nv_bfloat16*)o, scale);
  return lg::launch_status();
}

extern "C" uint32_t logismos_launch_gdn_prefill(void* state, const void* q, const void* k, const void* v, const void* g,
                                                const void* beta, void* o, const void* gate_z, const void* cu_seqlens,
                                                const void* state_slots, const void* fresh, int32_t n_seqs,
                                                int32_t heads, int32_t qkv_stride, float scale, int32_t mode, void* stream) {
  lg::LaunchScope launch_scope_;
  const int state_static = (mode & LG_GDN_STATIC_STATE) ? 1 : 0;
  mode &= ~LG_GDN_STATIC_STATE;
  if (n_seqs < 0 || heads <= 0 || qkv_stride < heads * KD || (qkv_stride % 8) || mode < 0 || mode > 2) return lg::kInvalidValue;
  if (n_seqs == 0) return 0;
  // rows are fetched in 16-byte pieces
  if (((uintptr_t)state & 15) || ((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15) || ((uintptr_t)gate_z & 15) || ((uintptr_t)o & 1))
    return lg::kInvalidValue;
  // few (sequence, head) pairs: the latency shape (more, shorter dependency chains per head); otherwise
  // the throughput shape
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const bool latency = mode == 2 || (mode == 0 && (int64_t)n_seqs * heads < 2ll * sms);
  const int64_t ctas = (int64_t)n_seqs * heads * (latency ? PfCfg<1, 4>::kParts : PfCfg<2, 4>::kParts);
  if (ctas > 2147483647ll) return lg::kInvalidValue;
  auto kern = latency ? gdn_prefill_kernel<1, 4> : gdn_prefill_kernel<2, 4>;
  lg::launch(kern, dim3((unsigned)ctas), dim3(128), 0, (cudaStream_t)stream, 
      (float*)state, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const float*)g,
      (const float*)beta, (__nv_bfloat16*)o, (const __nv_bfloat16*)gate_z, (const int*)cu_seqlens, (const int*)state_slots, (const uint8_t*)fresh, heads,
      (int64_t)qkv_stride, scale, state_static);
  return lg::launch_status();
}

extern "C" uint32_t logismos_launch_gdn_prepare(void* q, void* k, const void* a, const void* b, const void* A_log,
                                                const void* dt_bias, void* g, void* beta, int32_t n_tokens,
                                                int32_t heads, int32_t qk_stride, int32_t ab_stride, void* stream) {
  lg::LaunchScope launch_scope_;
  if (n_tokens < 0 || heads <= 0 || qk_stride < heads * KD || (qk_stride % 4) || ab_stride < heads) return lg::kInvalidValue;
  if (n_tokens == 0) return 0;
  if (((uintptr_t)q & 7) || ((uintptr_t)k & 7)) return lg::kInvalidValue;
  const int64_t rows = (int64_t)n_tokens * heads;
  const int wpb = 8;
  lg::launch(gdn_prepare_kernel, dim3((unsigned)((rows + wpb - 1) / wpb)), dim3(wpb * 32), 0, (cudaStream_t)stream, 
      (__nv_bfloat16*)q, (__nv_bfloat16*)k, (const float*)a, (const float*)b, (const float*)A_log, (const float*)dt_bias,
      (float*)g, (float*)beta, rows, heads, (int64_t)qk_stride, ab_stride);
  return lg::launch_status();
}
