// CPU oracle, part 2: attention, SwiGLU MLP, the Stella encoder stack and the
// embedding head. Test infrastructure only; see oracle.h.
//
// Follows, operation by operation:
//   crates/transformers/src/attention.rs:122-304 (+ helpers :323-382)
//   crates/transformers/src/mlp.rs:82-125
//   crates/transformers/src/rope.rs:35-92
//   crates/transformers/src/norm.rs:14-34
//   crates/encoders/src/stella.rs:190-206, :278-313
//   crates/embed/src/stella.rs:221-248, :264-294, :447-500
#include "oracle.h"

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <set>
#include <string>
#include <thread>
#include <utility>
#include <vector>

extern "C" {

// attention.rs:323-339: [seq, heads, d] -> [heads, seq, d]
void orc_transpose_seq_heads(const float* x, size_t seq, size_t heads, size_t d, float* out) {
  for (size_t s = 0; s < seq; ++s)
    for (size_t h = 0; h < heads; ++h)
      std::memcpy(out + (h * seq + s) * d, x + (s * heads + h) * d, d * sizeof(float));
}

// attention.rs:344-360: [heads, seq, d] -> [seq, heads, d]
void orc_merge_heads(const float* x, size_t heads, size_t seq, size_t d, float* out) {
  for (size_t h = 0; h < heads; ++h)
    for (size_t s = 0; s < seq; ++s)
      std::memcpy(out + (s * heads + h) * d, x + (h * seq + s) * d, d * sizeof(float));
}

// attention.rs:366-382: kv head h is copied to q-head slots h*groups .. h*groups+groups-1
void orc_repeat_kv(const float* kv, size_t n_kv, size_t groups, size_t seq, size_t d, float* out) {
  for (size_t h = 0; h < n_kv; ++h)
    for (size_t g = 0; g < groups; ++g)
      std::memcpy(out + (h * groups + g) * seq * d, kv + h * seq * d, seq * d * sizeof(float));
}

// rope.rs:50-92: per-position rows of the table; a position >= max_seq is an error (returns 1)
int orc_rope_gather(const float* cos_tab, const float* sin_tab, size_t max_seq, size_t head_dim,
                    const size_t* positions, size_t n_pos, float* cos_rows, float* sin_rows) {
  size_t half = head_dim / 2;
  for (size_t i = 0; i < n_pos; ++i) {
    if (positions[i] >= max_seq) return 1;
    std::memcpy(cos_rows + i * half, cos_tab + positions[i] * half, half * sizeof(float));
    std::memcpy(sin_rows + i * half, sin_tab + positions[i] * half, half * sizeof(float));
  }
  return 0;
}

// attention.rs:217-299: the score / mask / softmax / PV stage on already projected and rotated
// q [seq, n_h, d], k and v [seq, n_kv, d]; writes the merged heads [seq, n_h * d].
int orc_sdpa(const float* q, const float* k, const float* v, const uint8_t* mask, size_t seq,
             size_t n_h, size_t n_kv, size_t d, int causal, float* merged_out) {
  if (n_kv == 0 || n_h % n_kv != 0) return 2;
  const size_t hidden = n_h * d, kvw = n_kv * d, groups = n_h / n_kv;
  std::vector<float> q_hsd(seq * hidden), k_hsd(seq * kvw), v_hsd(seq * kvw);
  orc_transpose_seq_heads(q, seq, n_h, d, q_hsd.data());
  orc_transpose_seq_heads(k, seq, n_kv, d, k_hsd.data());
  orc_transpose_seq_heads(v, seq, n_kv, d, v_hsd.data());
  std::vector<float> k_exp(n_h * seq * d), v_exp(n_h * seq * d);
  orc_repeat_kv(k_hsd.data(), n_kv, groups, seq, d, k_exp.data());
  orc_repeat_kv(v_hsd.data(), n_kv, groups, seq, d, v_exp.data());

  // scores = (q @ k^T) * scale, the scale applied after the GEMM (attention.rs:226-242)
  const float scale = 1.0f / std::sqrt((float)d);
  std::vector<float> scores(n_h * seq * seq), sc(seq * seq);
  for (size_t h = 0; h < n_h; ++h) {
    orc_linear_t(q_hsd.data() + h * seq * d, seq * d, k_exp.data() + h * seq * d, seq * d, nullptr,
                 0, seq, seq, d, sc.data());
    float* dst = scores.data() + h * seq * seq;
    for (size_t i = 0; i < seq * seq; ++i) dst[i] = sc[i] * scale;
  }

  // column mask broadcast over rows (attention.rs:247-271)
  std::vector<uint8_t> col_mask(seq * seq);
  for (size_t i = 0; i < seq; ++i)
    for (size_t j = 0; j < seq; ++j) col_mask[i * seq + j] = (causal && j > i) ? 0 : mask[j];
  for (size_t h = 0; h < n_h; ++h)
    orc_mask_additive_in_place(scores.data() + h * seq * seq, seq * seq, col_mask.data(),
                               seq * seq, seq, seq);

  std::vector<float> sm(seq * seq);
  for (size_t h = 0; h < n_h; ++h) {
    float* head = scores.data() + h * seq * seq;
    orc_softmax_last_dim(head, seq, seq, sm.data());
    std::memcpy(head, sm.data(), seq * seq * sizeof(float));
  }

  std::vector<float> attn(n_h * seq * d);
  for (size_t h = 0; h < n_h; ++h)
    orc_linear(scores.data() + h * seq * seq, seq * seq, v_exp.data() + h * seq * d, seq * d,
               nullptr, 0, seq, d, seq, attn.data() + h * seq * d);

  orc_merge_heads(attn.data(), n_h, seq, d, merged_out);
  return 0;
}

// attention.rs:122-304. Returns 1 for seq > rope max_seq, 2 for a GQA/shape violation.
// causal=1 additionally masks key j > query i (this build's decoder variant; the reference
// forward is bidirectional with a per-key-column padding mask).
int orc_attention_forward(const orc_attn_t* a, const float* x, const uint8_t* mask, size_t seq,
                          const float* cos_tab, const float* sin_tab, size_t rope_max_seq,
                          int causal, float* out) {
  const size_t hidden = a->hidden, n_h = a->n_heads, n_kv = a->n_kv_heads, d = a->head_dim;
  const size_t kvw = n_kv * d;
  if (n_kv == 0 || n_h % n_kv != 0 || d * n_h != hidden) return 2;
  if (seq > rope_max_seq) return 1;

  std::vector<float> q(seq * hidden), k(seq * kvw), v(seq * kvw);
  orc_linear_t(x, seq * hidden, a->wq, hidden * hidden, a->bq, hidden, seq, hidden, hidden, q.data());
  orc_linear_t(x, seq * hidden, a->wk, kvw * hidden, a->bk, kvw, seq, kvw, hidden, k.data());
  orc_linear_t(x, seq * hidden, a->wv, kvw * hidden, a->bv, kvw, seq, kvw, hidden, v.data());

  // positions: row r of q is (s = r / n_h); row r of k is (s = r / n_kv)   (attention.rs:203-213)
  {
    std::vector<size_t> pos_q(seq * n_h), pos_k(seq * n_kv);
    for (size_t s = 0; s < seq; ++s) {
      for (size_t h = 0; h < n_h; ++h) pos_q[s * n_h + h] = s;
      for (size_t h = 0; h < n_kv; ++h) pos_k[s * n_kv + h] = s;
    }
    size_t half = d / 2;
    std::vector<float> cq(seq * n_h * half), sq(seq * n_h * half);
    std::vector<float> ck(seq * n_kv * half), sk(seq * n_kv * half);
    if (orc_rope_gather(cos_tab, sin_tab, rope_max_seq, d, pos_q.data(), pos_q.size(), cq.data(), sq.data())) return 1;
    if (orc_rope_gather(cos_tab, sin_tab, rope_max_seq, d, pos_k.data(), pos_k.size(), ck.data(), sk.data())) return 1;
    orc_rope_halves_in_place(q.data(), cq.data(), sq.data(), seq * n_h, d);
    orc_rope_halves_in_place(k.data(), ck.data(), sk.data(), seq * n_kv, d);
  }

  std::vector<float> merged(seq * hidden);
  orc_sdpa(q.data(), k.data(), v.data(), mask, seq, n_h, n_kv, d, causal, merged.data());
  orc_linear_t(merged.data(), seq * hidden, a->wo, hidden * hidden, nullptr, 0, seq, hidden, hidden, out);
  return 0;
}

// mlp.rs:82-125: down( silu(gate(x)) * up(x) ), no biases
int orc_swiglu_forward(const float* w_gate, const float* w_up, const float* w_down, size_t hidden,
                       size_t inter, const float* x, size_t seq, float* out) {
  std::vector<float> gate(seq * inter), up(seq * inter), sg(seq * inter), prod(seq * inter);
  orc_linear_t(x, seq * hidden, w_gate, inter * hidden, nullptr, 0, seq, inter, hidden, gate.data());
  orc_linear_t(x, seq * hidden, w_up, inter * hidden, nullptr, 0, seq, inter, hidden, up.data());
  orc_silu(gate.data(), seq * inter, sg.data());
  orc_hadamard(sg.data(), seq * inter, up.data(), seq * inter, prod.data());
  orc_linear_t(prod.data(), seq * inter, w_down, hidden * inter, nullptr, 0, seq, hidden, inter, out);
  return 0;
}

}  // extern "C"

namespace {

struct Stella {
  orc_stella_t d;
  std::vector<orc_layer_weights_t> layers;
  std::vector<float> cos, sin;
  size_t head_dim;
};

}  // namespace

extern "C" {

// encoders/src/stella.rs:230-256: the RoPE table covers max_pos positions
void* orc_stella_create(const orc_stella_t* desc) {
  Stella* m = new Stella();
  m->d = *desc;
  m->layers.assign(desc->layers, desc->layers + desc->n_layers);
  m->d.layers = m->layers.data();
  m->head_dim = desc->hidden / desc->n_heads;
  size_t half = m->head_dim / 2;
  m->cos.resize(desc->max_pos * half);
  m->sin.resize(desc->max_pos * half);
  orc_build_rope_table_f32(desc->max_pos, m->head_dim, desc->rope_theta, m->cos.data(), m->sin.data());
  return m;
}

void orc_stella_destroy(void* model) { delete static_cast<Stella*>(model); }

// encoders/src/stella.rs:278-313 with the layer body of :190-206
int orc_stella_forward(void* model, const uint32_t* ids, const uint8_t* mask, size_t seq,
                       int causal, float* hidden_out) {
  Stella* m = static_cast<Stella*>(model);
  const size_t hidden = m->d.hidden;
  if (seq > m->d.max_pos) return -2;
  std::vector<float> x(seq * hidden), norm(seq * hidden), tmp(seq * hidden);
  orc_embed_lookup(m->d.tok_embed, hidden, m->d.vocab, ids, seq, x.data());
  for (size_t l = 0; l < m->d.n_layers; ++l) {
    const orc_layer_weights_t& w = m->layers[l];
    orc_attn_t a{hidden, m->d.n_heads, m->d.n_kv_heads, m->head_dim,
                 w.wq, w.bq, w.wk, w.bk, w.wv, w.bv, w.wo};
    orc_rms_norm(x.data(), w.norm1, seq, hidden, m->d.rms_eps, norm.data());
    int rc = orc_attention_forward(&a, norm.data(), mask, seq, m->cos.data(), m->sin.data(),
                                   m->d.max_pos, causal, tmp.data());
    if (rc) return rc;
    for (size_t i = 0; i < seq * hidden; ++i) x[i] += tmp[i];
    orc_rms_norm(x.data(), w.norm2, seq, hidden, m->d.rms_eps, norm.data());
    orc_swiglu_forward(w.w_gate, w.w_up, w.w_down, hidden, m->d.intermediate, norm.data(), seq, tmp.data());
    for (size_t i = 0; i < seq * hidden; ++i) x[i] += tmp[i];
  }
  orc_rms_norm(x.data(), m->d.final_norm, seq, hidden, m->d.rms_eps, hidden_out);
  return 0;
}

// embed/src/stella.rs:221-248: mean pool -> L2 -> dense head (+bias) -> L2
int orc_stella_encode_raw(void* model, const uint32_t* ids, const uint8_t* mask, size_t seq,
                          float* emb_out) {
  Stella* m = static_cast<Stella*>(model);
  const size_t hidden = m->d.hidden, dim = m->d.head_out_dim;
  std::vector<float> hs(seq * hidden), pooled(hidden);
  int rc = orc_stella_forward(model, ids, mask, seq, 0, hs.data());
  if (rc) return rc;
  orc_mean_pool_masked(hs.data(), mask, seq, hidden, pooled.data());
  orc_l2_normalize_in_place(pooled.data(), hidden);
  orc_linear_t(pooled.data(), hidden, m->d.head_w, dim * hidden, m->d.head_b, dim, 1, dim, hidden, emb_out);
  orc_l2_normalize_in_place(emb_out, dim);
  return 0;
}

// embed/src/stella.rs:264-294: one worker per sentence on a pool of n_threads, each worker
// running the single-threaded forward; the first failure is returned.
int orc_stella_encode_batch(void* model, const uint32_t* ids, const int32_t* cu_seqlens,
                            size_t n_seq, size_t n_threads, float* emb_out) {
  Stella* m = static_cast<Stella*>(model);
  const size_t dim = m->d.head_out_dim;
  if (n_threads == 0) n_threads = 1;
  std::atomic<size_t> next{0};
  std::atomic<int> err{0};
  auto worker = [&]() {
    for (;;) {
      size_t i = next.fetch_add(1);
      if (i >= n_seq) return;
      size_t s0 = (size_t)cu_seqlens[i], len = (size_t)(cu_seqlens[i + 1] - cu_seqlens[i]);
      std::vector<uint8_t> mask(len, 1);  // embed/src/stella.rs:318: no padding ever exists
      int rc = orc_stella_encode_raw(model, ids + s0, mask.data(), len, emb_out + i * dim);
      if (rc) err.store(rc);
    }
  };
  std::vector<std::thread> pool;
  size_t nt = std::min(n_threads, n_seq);
  for (size_t t = 0; t < nt; ++t) pool.emplace_back(worker);
  for (auto& t : pool) t.join();
  return err.load();
}

// embed/src/stella.rs:447-500: distinct (physical id, core id) pairs in /proc/cpuinfo. A block
// without a "physical id" line counts under socket 0; a block without "core id" is not
// counted; a zero count falls back to the logical thread count.
size_t orc_count_physical_cores_text(const char* text) {
  std::set<std::pair<long, long>> cores;
  long phys = -1, core = -1;
  auto flush = [&]() {
    if (core >= 0) cores.insert({phys < 0 ? 0 : phys, core});
    phys = core = -1;
  };
  std::string s(text), line;
  size_t pos = 0;
  while (pos <= s.size()) {
    size_t nl = s.find('\n', pos);
    line = s.substr(pos, nl == std::string::npos ? std::string::npos : nl - pos);
    pos = nl == std::string::npos ? s.size() + 1 : nl + 1;
    if (line.rfind("physical id\t: ", 0) == 0) phys = std::atol(line.c_str() + 14);
    else if (line.rfind("core id\t: ", 0) == 0) core = std::atol(line.c_str() + 10);
    else if (line.find_first_not_of(" \t\r") == std::string::npos) flush();
  }
  flush();
  return cores.size();
}

size_t orc_physical_cores(void) {
  std::ifstream f("/proc/cpuinfo");
  std::string text((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
  size_t n = orc_count_physical_cores_text(text.c_str());
  if (n > 0) return n;
  unsigned hc = std::thread::hardware_concurrency();
  return hc ? hc : 4;
}

}  // extern "C"
