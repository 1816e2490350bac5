// CPU oracle (test infrastructure): the logit processors and samplers of the reference's decode
// crate, restated in the reference's operation order.
//   TemperatureScale / TopK / TopP / MinP / RepetitionPenalty   crates/decode/src/processors.rs:15-199
//   softmax helper                                               crates/decode/src/processors.rs:190-199
//   MultinomialSampler::sample                                   crates/decode/src/sampler.rs:31-58
// Pinned against the crate's own unit-test vectors (processors.rs:213-360, sampler.rs:66-100).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <numeric>
#include <vector>

#include "oracle.h"

namespace {

// processors.rs:190-199: max-subtracted exp, divided by the sum only when the sum is positive
std::vector<float> softmax(const float* logits, size_t n) {
  float mx = -INFINITY;
  for (size_t i = 0; i < n; ++i) mx = std::fmax(mx, logits[i]);  // f32::max ignores NaN like fmaxf
  std::vector<float> e(n);
  for (size_t i = 0; i < n; ++i) e[i] = std::exp(logits[i] - mx);
  float sum = 0.0f;
  for (size_t i = 0; i < n; ++i) sum += e[i];
  if (sum > 0.0f)
    for (size_t i = 0; i < n; ++i) e[i] /= sum;
  return e;
}

}  // namespace

extern "C" {

// processors.rs:18-28: t = max(T, 1e-6); |t - 1| < 1e-9 is the identity; otherwise l /= t
void orc_temperature(float* logits, size_t n, float temperature) {
  const float t = std::fmax(temperature, 1e-6f);
  if (std::fabs(t - 1.0f) < 1e-9f) return;
  for (size_t i = 0; i < n; ++i) logits[i] /= t;
}

// processors.rs:50-82: k == 0 or k >= n is the identity; NaN sorts as -inf; threshold = k-th largest;
// every NaN and every logit below the threshold becomes -inf (ties with the threshold survive)
void orc_top_k(float* logits, size_t n, size_t k) {
  if (k == 0 || k >= n) return;
  std::vector<float> s(n);
  for (size_t i = 0; i < n; ++i) s[i] = std::isnan(logits[i]) ? -INFINITY : logits[i];
  std::stable_sort(s.begin(), s.end(), [](float a, float b) { return a > b; });
  const float threshold = s[k - 1];
  for (size_t i = 0; i < n; ++i)
    if (std::isnan(logits[i]) || logits[i] < threshold) logits[i] = -INFINITY;
}

// processors.rs:89-122: p clamped to [0, 1]; p >= 1 or empty is the identity; indices stably sorted by
// descending probability; kept until the running fp32 sum reaches p (the element that crosses it is
// kept); the rest becomes -inf
void orc_top_p(float* logits, size_t n, float p_in) {
  const float p = std::fmin(std::fmax(p_in, 0.0f), 1.0f);
  if (p >= 1.0f || n == 0) return;
  const std::vector<float> probs = softmax(logits, n);
  std::vector<size_t> idx(n);
  std::iota(idx.begin(), idx.end(), (size_t)0);
  std::stable_sort(idx.begin(), idx.end(), [&](size_t a, size_t b) { return probs[a] > probs[b]; });
  std::vector<uint8_t> keep(n, 0);
  float cum = 0.0f;
  for (size_t i : idx) {
    keep[i] = 1;
    cum += probs[i];
    if (cum >= p) break;
  }
  for (size_t i = 0; i < n; ++i)
    if (!keep[i]) logits[i] = -INFINITY;
}

// processors.rs:130-146: p clamped; p <= 0 or empty is the identity; tokens whose probability is below
// p * max probability become -inf
void orc_min_p(float* logits, size_t n, float p_in) {
  const float p = std::fmin(std::fmax(p_in, 0.0f), 1.0f);
  if (p <= 0.0f || n == 0) return;
  const std::vector<float> probs = softmax(logits, n);
  float max_p = 0.0f;
  for (size_t i = 0; i < n; ++i) max_p = std::fmax(max_p, probs[i]);
  const float threshold = p * max_p;
  for (size_t i = 0; i < n; ++i)
    if (probs[i] < threshold) logits[i] = -INFINITY;
}

// processors.rs:160-181: |penalty - 1| < 1e-9 is the identity; for every listed token in order
// (a token listed twice is penalised twice; ids outside the vocabulary are skipped): a positive logit
// is divided by the penalty, any other multiplied
void orc_repetition_penalty(float* logits, size_t n, const uint32_t* tokens, size_t n_tokens, float penalty) {
  if (std::fabs(penalty - 1.0f) < 1e-9f) return;
  for (size_t j = 0; j < n_tokens; ++j) {
    const size_t i = tokens[j];
    if (i >= n) continue;
    if (logits[i] > 0.0f) logits[i] /= penalty;
    else logits[i] *= penalty;
  }
}

// sampler.rs:31-58 with the uniform draw u in [0, 1) supplied by the caller (the reference draws it
// from its RNG at that point): probabilities = exp(l - max) of the finite logits over their fp32 sum;
// a non-positive sum falls back to greedy; walk: u < p_i returns i, else u -= p_i; the last index
// when the walk runs out. An empty slice returns 0.
uint32_t orc_multinomial(const float* logits, size_t n, float u) {
  if (n == 0) return 0;
  float mx = -INFINITY;
  for (size_t i = 0; i < n; ++i) mx = std::fmax(mx, logits[i]);
  std::vector<float> e(n);
  for (size_t i = 0; i < n; ++i) e[i] = std::isfinite(logits[i]) ? std::exp(logits[i] - mx) : 0.0f;
  float sum = 0.0f;
  for (size_t i = 0; i < n; ++i) sum += e[i];
  if (sum <= 0.0f) return orc_greedy(logits, n);
  for (size_t i = 0; i < n; ++i) e[i] /= sum;
  for (size_t i = 0; i < n; ++i) {
    if (u < e[i]) return (uint32_t)i;
    u -= e[i];
  }
  return (uint32_t)(n - 1);
}

}  // extern "C"
