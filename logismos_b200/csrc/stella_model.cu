// Host-side executor of the Stella embedding model on one GPU: the composition of
// StellaEncoder::forward (crates/encoders/src/stella.rs:278-313, layer body :190-206) and
// StellaModel::encode_raw / encode_batch (crates/embed/src/stella.rs:221-294) over the kernel
// launchers, for a ragged batch (no padding; the reference's mask is all ones).
//
// Data layout in HBM: weights bf16 (QKV rows fused into one [q|k|v, hidden] matrix, gate/up
// fused into one matrix, optionally interleaved in 32-row blocks for the fused SwiGLU epilogue),
// biases and norm gains fp32, the residual stream fp32 [tokens, hidden], every GEMM operand
// bf16. The RoPE table is the reference's f64-evaluated table (cpu_f32/mod.rs:599-619).
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "logismos_kernels.h"
#include "logismos_model.h"

namespace {

thread_local std::string g_last_error;

void set_error(const std::string& s) { g_last_error = s; }
}  // namespace

// shared with the other executors of the library
namespace lgm {
void set_error(const std::string& s) { g_last_error = s; }
}  // namespace lgm

namespace {

inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

struct DevBuf {
  void* p = nullptr;
  size_t bytes = 0;
  bool alloc(size_t n) {
    bytes = n;
    return cudaMalloc(&p, n ? n : 1) == cudaSuccess;
  }
  void release() {
    if (p) cudaFree(p);
    p = nullptr;
  }
};

struct Layer {
  DevBuf norm1, norm2, wqkv, bqkv, wo, wgu, wdown;
};

struct Stella {
  lg_stella_config_t cfg{};
  int device = 0;
  int head_dim = 0, qkv_dim = 0;
  DevBuf tok_embed, final_norm, cos, sin;
  std::vector<Layer> layers;
  DevBuf head_w[8], head_b[8];
  // workspace
  DevBuf x, h, qkv, attn, attn_ws, gu, act, hidden_out, pooled, ids, pos, cu, out, status;
  // pinned staging
  uint32_t* h_ids = nullptr;
  int32_t* h_pos = nullptr;
  int32_t* h_cu = nullptr;
  float* h_out = nullptr;
  cudaStream_t stream = nullptr;
  std::mutex mu;
  std::vector<DevBuf*> all;
};

bool upload_bf16(DevBuf& dst, const float* src, size_t n, std::vector<uint16_t>& tmp) {
  tmp.resize(n);
  for (size_t i = 0; i < n; ++i) tmp[i] = f32_to_bf16(src[i]);
  if (!dst.alloc(n * 2)) return false;
  return cudaMemcpy(dst.p, tmp.data(), n * 2, cudaMemcpyHostToDevice) == cudaSuccess;
}
bool upload_f32(DevBuf& dst, const float* src, size_t n) {
  if (!dst.alloc(n * 4)) return false;
  return cudaMemcpy(dst.p, src, n * 4, cudaMemcpyHostToDevice) == cudaSuccess;
}

#define LG_TRY(expr, what)                                                        \
  do {                                                                            \
    uint32_t rc_ = (expr);                                                        \
    if (rc_ != 0) {                                                               \
      char buf_[160];                                                             \
      std::snprintf(buf_, sizeof(buf_), "%s failed: %s (code %u)", what,          \
                    cudaGetErrorString((cudaError_t)rc_), rc_);                   \
      set_error(buf_);                                                            \
      return LG_EMB_COMPUTE;                                                      \
    }                                                                             \
  } while (0)

int find_dim(const Stella* m, int dim) {
  for (int i = 0; i < m->cfg.n_dims; ++i)
    if (m->cfg.dims[i] == dim) return i;
  return -1;
}

uint32_t forward_device(Stella* m, const void* ids, const void* cu, const void* pos, int T, int n_seqs,
                        int max_seqlen, int dim_idx, int causal, void* out, cudaStream_t s) {
  const lg_stella_config_t& c = m->cfg;
  const int H = c.hidden, I = c.intermediate, D = m->head_dim, QKV = m->qkv_dim;
  void* st = m->status.p;
  LG_TRY(logismos_launch_embed_lookup_bf16(m->tok_embed.p, ids, m->x.p, T, H, c.vocab, s), "embed_lookup");
  for (int l = 0; l < c.n_layers; ++l) {
    Layer& L = m->layers[l];
    LG_TRY(logismos_launch_rms_norm_f32(m->x.p, L.norm1.p, m->h.p, T, H, c.rms_eps, 0, s), "rms_norm");
    LG_TRY(logismos_launch_linear_t_bf16(m->h.p, L.wqkv.p, L.bqkv.p, m->qkv.p, T, QKV, H, H, QKV, LG_EPI_BF16 | LG_EPI_STATIC_W, st, s), "qkv_proj");
    if (D == 128) {  // tcgen05 kernel; its first launch rotates q and k and transposes V into attn_ws
      LG_TRY(logismos_launch_rope_varlen_attention_tc_bf16(m->qkv.p, m->cos.p, m->sin.p, pos, c.n_heads + c.n_kv_heads, c.max_pos, cu,
                                                           m->attn.p, m->attn_ws.p, T, n_seqs, max_seqlen, c.n_heads, c.n_kv_heads, D,
                                                           QKV, H, H + c.n_kv_heads * D, causal, st, s), "rope + attention");
    } else {
      LG_TRY(logismos_launch_rope_halves_bf16(m->qkv.p, m->cos.p, m->sin.p, pos, T, c.n_heads + c.n_kv_heads, D, QKV,
                                              c.max_pos, st, s), "rope");
      LG_TRY(logismos_launch_varlen_attention_bf16(m->qkv.p, cu, m->attn.p, n_seqs, max_seqlen, c.n_heads, c.n_kv_heads,
                                                   D, QKV, H, H + c.n_kv_heads * D, causal, s), "attention");
    }
    LG_TRY(logismos_launch_linear_t_bf16(m->attn.p, L.wo.p, nullptr, m->x.p, T, H, H, H, H, LG_EPI_RESID_F32 | LG_EPI_STATIC_W, st, s), "o_proj");
    LG_TRY(logismos_launch_rms_norm_f32(m->x.p, L.norm2.p, m->h.p, T, H, c.rms_eps, 0, s), "rms_norm");
    if (c.fuse_swiglu) {
      LG_TRY(logismos_launch_linear_t_bf16(m->h.p, L.wgu.p, nullptr, m->act.p, T, 2 * I, H, H, I, LG_EPI_SWIGLU | LG_EPI_STATIC_W, st, s), "gate_up_swiglu");
    } else {
      LG_TRY(logismos_launch_linear_t_bf16(m->h.p, L.wgu.p, nullptr, m->gu.p, T, 2 * I, H, H, 2 * I, LG_EPI_BF16 | LG_EPI_STATIC_W, st, s), "gate_up");
      LG_TRY(logismos_launch_swiglu_bf16(m->gu.p, m->act.p, T, I, s), "swiglu");
    }
    LG_TRY(logismos_launch_linear_t_bf16(m->act.p, L.wdown.p, nullptr, m->x.p, T, H, I, I, H, LG_EPI_RESID_F32 | LG_EPI_STATIC_W, st, s), "down_proj");
  }
  LG_TRY(logismos_launch_rms_norm_f32(m->x.p, m->final_norm.p, m->hidden_out.p, T, H, c.rms_eps, 1, s), "final_norm");
  LG_TRY(logismos_launch_pool_head_f32(m->hidden_out.p, cu, m->head_w[dim_idx].p, m->head_b[dim_idx].p, out, m->pooled.p,
                                       n_seqs, H, c.dims[dim_idx], s), "pool_head");
  return LG_EMB_OK;
}

}  // namespace

extern "C" {

const char* lg_last_error(void) { return g_last_error.c_str(); }

uint32_t lg_stella_create(int32_t device, const lg_stella_config_t* cfg, const lg_stella_weights_t* w, void** model) {
  if (!cfg || !w || !model) { set_error("null argument"); return LG_EMB_COMPUTE; }
  *model = nullptr;
  const lg_stella_config_t& c = *cfg;
  if (c.hidden <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.hidden % c.n_heads || c.n_heads % c.n_kv_heads ||
      c.hidden / c.n_heads != 128 || c.hidden % 64 || c.intermediate % 64 || c.n_dims < 1 || c.n_dims > 8 ||
      c.max_batch_tokens <= 0 || c.max_batch_seqs <= 0 || c.max_pos <= 0 || c.n_layers < 0) {
    set_error("unsupported StellaConfig (head_dim must be 128; hidden and intermediate multiples of 64)");
    return LG_EMB_COMPUTE;
  }
  if (cudaSetDevice(device) != cudaSuccess) { set_error("cudaSetDevice failed"); return LG_EMB_COMPUTE; }
  Stella* m = new Stella();
  m->cfg = c;
  if (m->cfg.max_tokens <= 0) m->cfg.max_tokens = 512;
  m->device = device;
  m->head_dim = c.hidden / c.n_heads;
  m->qkv_dim = c.hidden + 2 * c.n_kv_heads * m->head_dim;
  const size_t H = c.hidden, I = c.intermediate, KV = (size_t)c.n_kv_heads * m->head_dim, QKV = m->qkv_dim;
  std::vector<uint16_t> tmp;
  std::vector<float> ftmp;
  bool ok = true;
  ok = ok && upload_bf16(m->tok_embed, w->tok_embed, (size_t)c.vocab * H, tmp);
  ok = ok && upload_f32(m->final_norm, w->final_norm, H);
  m->layers.resize(c.n_layers);
  for (int l = 0; l < c.n_layers && ok; ++l) {
    const lg_stella_layer_weights_t& lw = w->layers[l];
    Layer& L = m->layers[l];
    ok = ok && upload_f32(L.norm1, lw.norm1, H) && upload_f32(L.norm2, lw.norm2, H);
    // fused QKV: rows [wq; wk; wv], bias [bq; bk; bv]
    ftmp.resize(QKV * H);
    std::memcpy(ftmp.data(), lw.wq, H * H * 4);
    std::memcpy(ftmp.data() + H * H, lw.wk, KV * H * 4);
    std::memcpy(ftmp.data() + (H + KV) * H, lw.wv, KV * H * 4);
    ok = ok && upload_bf16(L.wqkv, ftmp.data(), QKV * H, tmp);
    ftmp.resize(QKV);
    std::memcpy(ftmp.data(), lw.bq, H * 4);
    std::memcpy(ftmp.data() + H, lw.bk, KV * 4);
    std::memcpy(ftmp.data() + H + KV, lw.bv, KV * 4);
    ok = ok && upload_f32(L.bqkv, ftmp.data(), QKV);
    ok = ok && upload_bf16(L.wo, lw.wo, H * H, tmp);
    // fused gate/up: plain [gate; up], or 32-row blocks gate/up interleaved for the fused epilogue
    ftmp.resize(2 * I * H);
    if (c.fuse_swiglu) {
      for (size_t b = 0; b < I / 32; ++b) {
        std::memcpy(ftmp.data() + (2 * b) * 32 * H, lw.w_gate + b * 32 * H, 32 * H * 4);
        std::memcpy(ftmp.data() + (2 * b + 1) * 32 * H, lw.w_up + b * 32 * H, 32 * H * 4);
      }
    } else {
      std::memcpy(ftmp.data(), lw.w_gate, I * H * 4);
      std::memcpy(ftmp.data() + I * H, lw.w_up, I * H * 4);
    }
    ok = ok && upload_bf16(L.wgu, ftmp.data(), 2 * I * H, tmp);
    ok = ok && upload_bf16(L.wdown, lw.w_down, H * I, tmp);
  }
  for (int i = 0; i < c.n_dims && ok; ++i) {
    ok = ok && upload_bf16(m->head_w[i], w->head_w[i], (size_t)c.dims[i] * H, tmp);
    ok = ok && upload_f32(m->head_b[i], w->head_b[i], (size_t)c.dims[i]);
  }
  // RoPE table: inv_freq and angle in f64, cast to f32 (cpu_f32/mod.rs:599-619)
  if (ok) {
    const size_t half = m->head_dim / 2;
    std::vector<float> cs((size_t)c.max_pos * half), sn((size_t)c.max_pos * half);
    for (int p = 0; p < c.max_pos; ++p)
      for (size_t i = 0; i < half; ++i) {
        const double inv_freq = std::pow(c.rope_theta, -(2.0 * (double)i) / (double)m->head_dim);
        const double ang = (double)p * inv_freq;
        cs[p * half + i] = (float)std::cos(ang);
        sn[p * half + i] = (float)std::sin(ang);
      }
    ok = ok && upload_f32(m->cos, cs.data(), cs.size()) && upload_f32(m->sin, sn.data(), sn.size());
  }
  const size_t T = c.max_batch_tokens, S = c.max_batch_seqs;
  int max_dim = 0;
  for (int i = 0; i < c.n_dims; ++i) max_dim = c.dims[i] > max_dim ? c.dims[i] : max_dim;
  ok = ok && m->x.alloc(T * H * 4) && m->h.alloc(T * H * 2) && m->qkv.alloc(T * QKV * 2) && m->attn.alloc(T * H * 2) &&
       m->attn_ws.alloc(logismos_varlen_attention_tc_scratch_bytes((int)T, (int)S, c.n_kv_heads, 128)) &&
       m->gu.alloc(c.fuse_swiglu ? 16 : T * 2 * I * 2) && m->act.alloc(T * I * 2) && m->hidden_out.alloc(T * H * 4) && m->pooled.alloc(S * H * 4) &&
       m->ids.alloc(T * 4) && m->pos.alloc(T * 4) && m->cu.alloc((S + 1) * 4) && m->out.alloc(S * max_dim * 4) &&
       m->status.alloc(4);
  ok = ok && cudaMemset(m->status.p, 0, 4) == cudaSuccess;
  ok = ok && cudaMallocHost((void**)&m->h_ids, T * 4) == cudaSuccess && cudaMallocHost((void**)&m->h_pos, T * 4) == cudaSuccess &&
       cudaMallocHost((void**)&m->h_cu, (S + 1) * 4) == cudaSuccess &&
       cudaMallocHost((void**)&m->h_out, S * max_dim * 4) == cudaSuccess;
  ok = ok && cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking) == cudaSuccess;
  if (!ok) {
    set_error(std::string("lg_stella_create: allocation or upload failed: ") + cudaGetErrorString(cudaGetLastError()));
    lg_stella_destroy(m);
    return LG_EMB_COMPUTE;
  }
  *model = m;
  return LG_EMB_OK;
}

void lg_stella_destroy(void* model) {
  if (!model) return;
  Stella* m = static_cast<Stella*>(model);
  cudaSetDevice(m->device);
  DevBuf* bufs[] = {&m->tok_embed, &m->final_norm, &m->cos, &m->sin, &m->x, &m->h, &m->qkv, &m->attn, &m->attn_ws, &m->gu,
                    &m->act, &m->hidden_out, &m->pooled, &m->ids, &m->pos, &m->cu, &m->out, &m->status};
  for (DevBuf* b : bufs) b->release();
  for (auto& L : m->layers) {
    L.norm1.release(); L.norm2.release(); L.wqkv.release(); L.bqkv.release(); L.wo.release(); L.wgu.release(); L.wdown.release();
  }
  for (int i = 0; i < 8; ++i) { m->head_w[i].release(); m->head_b[i].release(); }
  if (m->h_ids) cudaFreeHost(m->h_ids);
  if (m->h_pos) cudaFreeHost(m->h_pos);
  if (m->h_cu) cudaFreeHost(m->h_cu);
  if (m->h_out) cudaFreeHost(m->h_out);
  if (m->stream) cudaStreamDestroy(m->stream);
  delete m;
}

int32_t lg_stella_default_dim(const void* model) { return static_cast<const Stella*>(model)->cfg.dims[0]; }
int32_t lg_stella_supported_dims(const void* model, int32_t* out, int32_t cap) {
  const Stella* m = static_cast<const Stella*>(model);
  for (int i = 0; i < m->cfg.n_dims && i < cap; ++i) out[i] = m->cfg.dims[i];
  return m->cfg.n_dims;
}
int32_t lg_stella_max_tokens(const void* model) { return static_cast<const Stella*>(model)->cfg.max_tokens; }
int32_t lg_stella_launches_per_forward(const void* model) {
  const Stella* m = static_cast<const Stella*>(model);
  return 1 + m->cfg.n_layers * (m->cfg.fuse_swiglu ? 8 : 9) + 4;
}

uint32_t lg_stella_forward_device(void* model, const void* dev_ids, const void* dev_cu, const void* dev_pos,
                                  int32_t n_tokens, int32_t n_seqs, int32_t max_seqlen, int32_t dim, int32_t causal,
                                  void* dev_out, void* stream) {
  Stella* m = static_cast<Stella*>(model);
  const int di = find_dim(m, dim == 0 ? m->cfg.dims[0] : dim);
  if (di < 0) { set_error("unsupported dim"); return LG_EMB_UNSUPPORTED_DIM; }
  // pooled sums, the padded V^T scratch and the output are sized from max_batch_seqs
  if (n_tokens < 0 || n_tokens > m->cfg.max_batch_tokens || n_seqs < 0 || n_seqs > m->cfg.max_batch_seqs) {
    set_error("forward: batch exceeds workspace capacity (max_batch_tokens / max_batch_seqs)");
    return LG_EMB_COMPUTE;
  }
  if (max_seqlen < 0) { set_error("forward: max_seqlen < 0"); return LG_EMB_COMPUTE; }
  if (max_seqlen > m->cfg.max_pos) { set_error("forward: seq > max_pos"); return LG_EMB_COMPUTE; }
  if (n_tokens == 0 || n_seqs == 0) return LG_EMB_OK;
  if (cudaSetDevice(m->device) != cudaSuccess) { set_error("cudaSetDevice failed"); return LG_EMB_COMPUTE; }
  return forward_device(m, dev_ids, dev_cu, dev_pos, n_tokens, n_seqs, max_seqlen, di, causal, dev_out, (cudaStream_t)stream);
}

uint32_t lg_stella_encode_ids_batch(void* model, const uint32_t* host_ids, const int32_t* host_cu, int32_t n_seqs,
                                    int32_t dim, int32_t max_tokens, float* host_out) {
  Stella* m = static_cast<Stella*>(model);
  const int want = dim == 0 ? m->cfg.dims[0] : dim;
  const int di = find_dim(m, want);
  if (di < 0) {  // StellaModel::encode checks the dim before anything else (stella.rs:301-304)
    char b[64]; std::snprintf(b, sizeof(b), "unsupported dim %d", want); set_error(b);
    return LG_EMB_UNSUPPORTED_DIM;
  }
  if (n_seqs < 0 || (n_seqs > 0 && (!host_ids || !host_cu || !host_out))) { set_error("null argument"); return LG_EMB_COMPUTE; }
  const int limit = max_tokens > 0 ? max_tokens : m->cfg.max_tokens;
  for (int i = 0; i < n_seqs; ++i) {
    const int len = host_cu[i + 1] - host_cu[i];
    if (len < 0) { set_error("cu_seqlens not monotone"); return LG_EMB_COMPUTE; }
    if (len > limit) {  // check_token_limit: an error, never truncation (stella.rs:365-378)
      char b[96]; std::snprintf(b, sizeof(b), "input exceeds max_tokens: got %d, limit %d", len, limit); set_error(b);
      return LG_EMB_INPUT_TOO_LONG;
    }
    if (len > m->cfg.max_pos || len > m->cfg.max_batch_tokens) { set_error("forward: seq > max_pos"); return LG_EMB_COMPUTE; }
  }
  std::lock_guard<std::mutex> lock(m->mu);
  if (cudaSetDevice(m->device) != cudaSuccess) { set_error("cudaSetDevice failed"); return LG_EMB_COMPUTE; }
  const int d = m->cfg.dims[di];
  int i0 = 0;
  while (i0 < n_seqs) {
    // greedy sub-batch within the workspace capacity
    int i1 = i0, toks = 0, max_len = 0;
    while (i1 < n_seqs && i1 - i0 < m->cfg.max_batch_seqs) {
      const int len = host_cu[i1 + 1] - host_cu[i1];
      if (toks + len > m->cfg.max_batch_tokens) break;
      toks += len;
      max_len = len > max_len ? len : max_len;
      ++i1;
    }
    const int ns = i1 - i0;
    const int base = host_cu[i0];
    std::memcpy(m->h_ids, host_ids + base, (size_t)toks * 4);
    for (int i = 0; i <= ns; ++i) m->h_cu[i] = host_cu[i0 + i] - base;
    for (int i = 0; i < ns; ++i)
      for (int t = m->h_cu[i]; t < m->h_cu[i + 1]; ++t) m->h_pos[t] = t - m->h_cu[i];
    cudaStream_t s = m->stream;
    LG_TRY((uint32_t)cudaMemcpyAsync(m->ids.p, m->h_ids, (size_t)toks * 4, cudaMemcpyHostToDevice, s), "H2D ids");
    LG_TRY((uint32_t)cudaMemcpyAsync(m->pos.p, m->h_pos, (size_t)toks * 4, cudaMemcpyHostToDevice, s), "H2D positions");
    LG_TRY((uint32_t)cudaMemcpyAsync(m->cu.p, m->h_cu, (size_t)(ns + 1) * 4, cudaMemcpyHostToDevice, s), "H2D cu_seqlens");
    if (toks > 0) {
      uint32_t rc = forward_device(m, m->ids.p, m->cu.p, m->pos.p, toks, ns, max_len, di, 0, m->out.p, s);
      if (rc) return rc;
    } else {
      LG_TRY((uint32_t)cudaMemsetAsync(m->out.p, 0, (size_t)ns * d * 4, s), "memset");
    }
    LG_TRY((uint32_t)cudaMemcpyAsync(m->h_out, m->out.p, (size_t)ns * d * 4, cudaMemcpyDeviceToHost, s), "D2H embeddings");
    LG_TRY((uint32_t)cudaStreamSynchronize(s), "stream synchronize");
    std::memcpy(host_out + (size_t)i0 * d, m->h_out, (size_t)ns * d * 4);
    i0 = i1;
  }
  if (lg_stella_device_status(m) != 0) { set_error("a device-side range check or bounded wait failed"); return LG_EMB_COMPUTE; }
  return LG_EMB_OK;
}

uint32_t lg_stella_last_hidden(void* model, int32_t n_tokens, float* host_out) {
  Stella* m = static_cast<Stella*>(model);
  if (n_tokens < 0 || n_tokens > m->cfg.max_batch_tokens) return LG_EMB_COMPUTE;
  cudaSetDevice(m->device);
  LG_TRY((uint32_t)cudaDeviceSynchronize(), "device synchronize");
  LG_TRY((uint32_t)cudaMemcpy(host_out, m->hidden_out.p, (size_t)n_tokens * m->cfg.hidden * 4, cudaMemcpyDeviceToHost), "D2H hidden");
  return LG_EMB_OK;
}

int32_t lg_stella_device_status(void* model) {
  Stella* m = static_cast<Stella*>(model);
  int32_t v = -1;
  cudaSetDevice(m->device);
  if (cudaMemcpy(&v, m->status.p, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return v;
}

}  // extern "C"
