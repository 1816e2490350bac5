// CPU oracle, part 4: the hybrid decoder stack (gated-delta-rule linear-attention layers and
// gated full-attention layers), one sequence at a time, full recomputation (no cache).
// Test infrastructure only; see oracle.h.
//
// PARITY UNPINNED: the reference has no decoder model (crates/decoders/src/lib.rs:1-15). The layer
// definitions below are this build's; they are composed only of functions that ARE pinned:
// rms_norm, linear_t, rope_halves, the causal score/softmax/PV stage (orc_sdpa), silu
// (crates/kernels/src/cpu_f32/mod.rs), gated_delta_rule_recurrent_fwd and l2_norm_in_place
// (crates/kernels/src/gated_delta_rule/cpu.rs:19-34, :92-182), and the gate formulas of
// research/14-gdn-aiter-preflight.md:190-198, :209-219 (orc_gdn_gates).
//
//   block:  x += mixer(rms_norm(x, norm1));  x += swiglu(rms_norm(x, norm2))
//   full-attention mixer (n_heads q heads, n_kv_heads kv heads of attn_head_dim, no biases):
//     [q | gate | k | v] = h W^T; RoPE(halves) on q, k; causal attention; out *= sigmoid(gate); o_proj
//   linear-attention mixer (gdn_heads heads, key = value dim 128):
//     [q | k | v | z] = h W_in^T; [a | b] = h W_ab^T; q, k L2-normalised per head;
//     g = -exp(A_log) softplus(a + dt_bias), beta = sigmoid(b); o = gated delta rule(q,k,v,g,beta),
//     scale 1/sqrt(128); o *= silu(z); out_proj
#include <cmath>
#include <cstring>
#include <vector>

#include "oracle.h"

namespace {
struct Hybrid {
  orc_hybrid_t d;
  std::vector<orc_hybrid_layer_t> layers;
  std::vector<float> cos, sin;
};
}  // namespace

extern "C" {

void* orc_hybrid_create(const orc_hybrid_t* desc) {
  Hybrid* m = new Hybrid();
  m->d = *desc;
  m->layers.assign(desc->layers, desc->layers + desc->n_layers);
  const size_t half = desc->attn_head_dim / 2;
  m->cos.resize(desc->max_pos * half);
  m->sin.resize(desc->max_pos * half);
  orc_build_rope_table_f32(desc->max_pos, desc->attn_head_dim, desc->rope_theta, m->cos.data(), m->sin.data());
  return m;
}

void orc_hybrid_destroy(void* model) { delete static_cast<Hybrid*>(model); }

// hidden_out: final-norm output [seq, hidden]; logits_last (may be NULL): [vocab] for the last token
int orc_hybrid_forward(void* model, const uint32_t* ids, size_t seq, float* hidden_out, float* logits_last) {
  Hybrid* m = static_cast<Hybrid*>(model);
  const orc_hybrid_t& c = m->d;
  const size_t H = c.hidden, I = c.intermediate, nq = c.n_heads, nkv = c.n_kv_heads, ad = c.attn_head_dim;
  const size_t gh = c.gdn_heads, gd = 128;
  if (seq > c.max_pos) return -2;
  std::vector<float> x(seq * H), h(seq * H), tmp(seq * H);
  orc_embed_lookup(c.tok_embed, H, c.vocab, ids, seq, x.data());
  std::vector<uint8_t> ones(seq, 1);
  for (size_t l = 0; l < c.n_layers; ++l) {
    const orc_hybrid_layer_t& L = m->layers[l];
    orc_rms_norm(x.data(), L.norm1, seq, H, c.rms_eps, h.data());
    if (L.kind == 0) {
      const size_t QW = nq * ad, KW = nkv * ad, N = 2 * QW + 2 * KW;
      std::vector<float> p(seq * N), q(seq * QW), gate(seq * QW), k(seq * KW), v(seq * KW), att(seq * QW);
      orc_linear_t(h.data(), seq * H, L.w_mix_in, N * H, nullptr, 0, seq, N, H, p.data());
      for (size_t t = 0; t < seq; ++t) {
        std::memcpy(&q[t * QW], &p[t * N], QW * 4);
        std::memcpy(&gate[t * QW], &p[t * N + QW], QW * 4);
        std::memcpy(&k[t * KW], &p[t * N + 2 * QW], KW * 4);
        std::memcpy(&v[t * KW], &p[t * N + 2 * QW + KW], KW * 4);
      }
      std::vector<size_t> pq(seq * nq), pk(seq * nkv);
      for (size_t t = 0; t < seq; ++t) {
        for (size_t j = 0; j < nq; ++j) pq[t * nq + j] = t;
        for (size_t j = 0; j < nkv; ++j) pk[t * nkv + j] = t;
      }
      const size_t half = ad / 2;
      std::vector<float> cq(seq * nq * half), sq(seq * nq * half), ck(seq * nkv * half), sk(seq * nkv * half);
      orc_rope_gather(m->cos.data(), m->sin.data(), c.max_pos, ad, pq.data(), pq.size(), cq.data(), sq.data());
      orc_rope_gather(m->cos.data(), m->sin.data(), c.max_pos, ad, pk.data(), pk.size(), ck.data(), sk.data());
      orc_rope_halves_in_place(q.data(), cq.data(), sq.data(), seq * nq, ad);
      orc_rope_halves_in_place(k.data(), ck.data(), sk.data(), seq * nkv, ad);
      orc_sdpa(q.data(), k.data(), v.data(), ones.data(), seq, nq, nkv, ad, 1, att.data());
      for (size_t i = 0; i < seq * QW; ++i) att[i] *= 1.0f / (1.0f + std::exp(-gate[i]));
      orc_linear_t(att.data(), seq * QW, L.w_mix_out, H * QW, nullptr, 0, seq, H, QW, tmp.data());
    } else {
      const size_t W = gh * gd, N = 4 * W;
      std::vector<float> p(seq * N), ab(seq * 2 * gh), g(seq * gh), beta(seq * gh), o(seq * W);
      orc_linear_t(h.data(), seq * H, L.w_mix_in, N * H, nullptr, 0, seq, N, H, p.data());
      orc_linear_t(h.data(), seq * H, L.w_ab, 2 * gh * H, nullptr, 0, seq, 2 * gh, H, ab.data());
      std::vector<float> a(seq * gh), b(seq * gh);
      for (size_t t = 0; t < seq; ++t)
        for (size_t j = 0; j < gh; ++j) { a[t * gh + j] = ab[t * 2 * gh + j]; b[t * gh + j] = ab[t * 2 * gh + gh + j]; }
      orc_gdn_gates(a.data(), b.data(), L.A_log, L.dt_bias, seq, gh, g.data(), beta.data());
      std::vector<float> qh(seq * gd), kh(seq * gd), vh(seq * gd), gg(seq), bb(seq), oh(seq * gd), st(gd * gd), st_out(gd * gd);
      const float scale = 1.0f / std::sqrt((float)gd);
      for (size_t j = 0; j < gh; ++j) {
        for (size_t t = 0; t < seq; ++t) {
          std::memcpy(&qh[t * gd], &p[t * N + j * gd], gd * 4);
          std::memcpy(&kh[t * gd], &p[t * N + W + j * gd], gd * 4);
          std::memcpy(&vh[t * gd], &p[t * N + 2 * W + j * gd], gd * 4);
          gg[t] = g[t * gh + j];
          bb[t] = beta[t * gh + j];
        }
        orc_l2_norm_rows(qh.data(), seq * gd, gd);
        orc_l2_norm_rows(kh.data(), seq * gd, gd);
        std::fill(st.begin(), st.end(), 0.0f);
        orc_gdn_recurrent_fwd(qh.data(), kh.data(), vh.data(), bb.data(), gg.data(), seq, scale, st.data(), gd, gd, oh.data(), st_out.data());
        for (size_t t = 0; t < seq; ++t)
          for (size_t i = 0; i < gd; ++i) {
            const float z = p[t * N + 3 * W + j * gd + i];
            o[t * W + j * gd + i] = oh[t * gd + i] * (z / (1.0f + std::exp(-z)));
          }
      }
      orc_linear_t(o.data(), seq * W, L.w_mix_out, H * W, nullptr, 0, seq, H, W, tmp.data());
    }
    for (size_t i = 0; i < seq * H; ++i) x[i] += tmp[i];
    orc_rms_norm(x.data(), L.norm2, seq, H, c.rms_eps, h.data());
    orc_swiglu_forward(L.w_gate, L.w_up, L.w_down, H, I, h.data(), seq, tmp.data());
    for (size_t i = 0; i < seq * H; ++i) x[i] += tmp[i];
  }
  orc_rms_norm(x.data(), c.final_norm, seq, H, c.rms_eps, hidden_out);
  if (logits_last) orc_linear_t(hidden_out + (seq - 1) * H, H, c.lm_head, c.vocab * H, nullptr, 0, 1, c.vocab, H, logits_last);
  return 0;
}

}  // extern "C"
