// C++ mirror of the reference's token sampler interface (tools/sampler.h:15-26 `SamplingParams`,
// :28-144 `Sampler::sample` / `Sampler::sample_allowed`) over the C ABI of include/arcsample.h:
// same class and member names, same argument meaning, same results for the same seed. A server
// that includes tools/sampler.h today includes this header instead and links libarcsample.so.
//
// The draw is the reference's: std::uniform_real_distribution<double>(0, tot)(mt19937_64), which
// libstdc++ evaluates as tot * (rng() * 2^-64); one draw per non-greedy call (tools/sampler.h:71-72),
// none when a constrained call is left with a single candidate (:122). The generator lives here, on
// the host; the device receives the uniform number.
#pragma once
#include <cmath>
#include <cstdint>
#include <functional>
#include <random>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/arcsample.h"

namespace arcinfer_b200 {

struct SamplingParams {  // tools/sampler.h:15-26, field for field
  float temperature = 1.0f, top_p = 0.95f, min_p = 0.0f, presence_penalty = 0.0f;
  float frequency_penalty = 0.0f, repeat_penalty = 1.0f;
  int repeat_last_n = 64;
  int top_k = 20;
  uint64_t seed = 0;
  std::vector<std::pair<int, float>> logit_bias;
};

class Sampler {
 public:
  static constexpr float kBanned = ARCS_BANNED;  // tools/sampler.h:32

  // max_vocab: the largest vocabulary this sampler will see (device buffers are sized once)
  explicit Sampler(const SamplingParams& p, int max_vocab = 1 << 18, int device = 0)
      : p_(p), rng_(p.seed ? p.seed : std::random_device{}()) {
    for (const auto& tb : p_.logit_bias) {
      bias_id_.push_back(tb.first);
      bias_val_.push_back(tb.second);
    }
    const int rc = arcs_host_create(&ctx_, device, 1, max_vocab, ARCS_F32, kMaxRecent, (int64_t)bias_id_.size() + 1,
                                    (int64_t)(max_vocab + 31) / 32);
    if (rc != ARCS_OK) throw std::runtime_error(std::string("arcs_host_create: ") + arcs_last_error());
  }
  ~Sampler() { arcs_host_destroy(ctx_); }
  Sampler(const Sampler&) = delete;
  Sampler& operator=(const Sampler&) = delete;

  // tools/sampler.h:36-78
  int sample(const std::vector<float>& raw, const std::vector<int>& recent) { return run(raw, recent, nullptr); }

  // tools/sampler.h:82-144. The predicate is evaluated here for every token (the device takes a
  // bitmask); a caller that can describe its constraint as a byte automaton builds the mask on the
  // device with arcs_dfa_mask instead and calls sample_masked.
  int sample_allowed(const std::vector<float>& raw, const std::vector<int>& recent, const std::function<bool(int)>& ok) {
    const int V = (int)raw.size();
    mask_.assign((size_t)(V + 31) / 32, 0u);
    for (int t = 0; t < V; ++t)
      if (ok(t)) mask_[(size_t)t >> 5] |= 1u << (t & 31);
    return run(raw, recent, mask_.data());
  }
  int sample_masked(const std::vector<float>& raw, const std::vector<int>& recent, const uint32_t* allowed_bits) {
    return run(raw, recent, allowed_bits);
  }
  int last_flags() const { return flags_; }  // ARCS_FLAG_* of the last call (FIRST_REFUSED: tools/server_chat.h:542)

 private:
  static constexpr int64_t kMaxRecent = 1 << 16;
  int run(const std::vector<float>& raw, const std::vector<int>& recent, const uint32_t* mask) {
    const int V = (int)raw.size();
    if (V == 0) return -1;
    if ((int64_t)recent.size() > kMaxRecent) throw std::runtime_error("Sampler: history longer than the context was created for");
    const arcs_row_params rp{p_.temperature, p_.top_p,         p_.min_p,         p_.presence_penalty,
                             p_.frequency_penalty, p_.repeat_penalty, p_.repeat_last_n, p_.top_k};
    const int32_t hoff[2] = {0, (int32_t)recent.size()}, boff[2] = {0, (int32_t)bias_id_.size()};
    const std::mt19937_64 saved = rng_;
    double u = (double)rng_() * 5.42101086242752217e-20;  // 2^-64
    if (u >= 1.0) u = std::nextafter(1.0, 0.0);
    int32_t token = -1, n_cand = 0;
    arcs_sample_args a{};
    a.logits = raw.data();
    a.dtype = ARCS_F32;
    a.B = 1;
    a.V = V;
    a.row_stride = V;
    a.params = &rp;
    a.hist_off = hoff;
    a.hist_ids = recent.data();
    a.max_hist = hoff[1];
    a.bias_off = boff;
    a.bias_ids = bias_id_.data();
    a.bias_vals = bias_val_.data();
    a.max_bias = boff[1];
    a.u = &u;
    a.mask = mask;
    a.mask_stride = (V + 31) / 32;
    a.token = &token;
    a.n_cand = &n_cand;
    a.flags = &flags_;
    if (arcs_sample_batch_host(ctx_, &a) != ARCS_OK) throw std::runtime_error(std::string("arcs_sample_batch_host: ") + arcs_last_error());
    // tools/sampler.h:38 and :122: a greedy call, and a constrained call with at most one candidate, draw nothing
    if (p_.temperature <= 0.0f || (mask && n_cand <= 1)) rng_ = saved;
    return token;
  }
  SamplingParams p_;
  std::mt19937_64 rng_;
  std::vector<int32_t> bias_id_;
  std::vector<float> bias_val_;
  std::vector<uint32_t> mask_;
  arcs_host_ctx* ctx_ = nullptr;
  int32_t flags_ = 0;
};

}  // namespace arcinfer_b200
