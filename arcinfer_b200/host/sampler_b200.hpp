// C++ mirror of the reference's token sampler interface (tools/sampler.h:15-26 `SamplingParams`,
// :28-176 `Sampler::sample` / `sample_allowed` / `adjusted`) over the C ABI of include/arcsample.h:
// same class and member names, same argument meaning, same results for the same seed, and - for
// sample_allowed - the same sequence of predicate calls. A server that includes tools/sampler.h
// today includes this header instead and links libarcsample.so.
//
// The draw is the reference's: std::uniform_real_distribution<double>(0, tot)(mt19937_64), which
// libstdc++ evaluates as tot * (rng() * 2^-64); one draw per non-greedy call (tools/sampler.h:71-72),
// none when a constrained call is left with a single candidate (:122). The generator lives here, on
// the host; the device receives the uniform number.
#pragma once
#include <algorithm>
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
      : p_(p), rng_(p.seed ? p.seed : std::random_device{}()), max_vocab_(max_vocab) {
    for (const auto& tb : p_.logit_bias) {
      bias_id_.push_back(tb.first);
      bias_val_.push_back(tb.second);
      bans_ = bans_ || tb.second <= -100.0f;  // tools/sampler.h:34
    }
    const int rc = arcs_host_create(&ctx_, device, 1, max_vocab, ARCS_F32, kMaxRecent, (int64_t)bias_id_.size() + 1,
                                    (int64_t)(max_vocab + 31) / 32);
    if (rc != ARCS_OK) throw std::runtime_error(std::string("arcs_host_create: ") + arcs_last_error());
  }
  ~Sampler() { arcs_host_destroy(ctx_); }
  Sampler(const Sampler&) = delete;
  Sampler& operator=(const Sampler&) = delete;

  // tools/sampler.h:36-78
  int sample(const std::vector<float>& raw, const std::vector<int>& recent) {
    int32_t n_cand = 0;
    return run(raw, recent, nullptr, /*draw=*/true, &n_cand, false);
  }

  // tools/sampler.h:82-144. The predicate is called lazily, from the most likely token down, until
  // `need` allowed tokens are found - the reference's call sequence: the device ranks the 512 most
  // likely tokens (banned ones are skipped here before the predicate, :118), the e^-20 rule of :111
  // ends the scan at rank 512, and only where the reference itself goes on into the sorted rest of
  // the vocabulary does this call fetch the adjusted row and sort the rest on the host as it does.
  // The softmax, the cuts and the draw over the tokens found run on the device.
  int sample_allowed(const std::vector<float>& raw, const std::vector<int>& recent, const std::function<bool(int)>& ok) {
    const int V = (int)raw.size();
    flags_ = 0;
    if (V == 0) return -1;
    const int need = p_.temperature <= 0.0f ? 1 : (p_.top_k > 0 ? std::min(p_.top_k, V) : 40);  // :86
    mask_.assign((size_t)(V + 31) / 32, 0u);  // nothing allowed: the device call only ranks the head
    head_id_.resize(ARCS_HEAD);
    head_val_.resize(ARCS_HEAD);
    int32_t n_cand = 0;
    run(raw, recent, mask_.data(), /*draw=*/false, &n_cand, /*want_head=*/true);
    std::vector<int32_t> c;
    std::vector<float> cv;
    bool first = true;
    auto test = [&](int t, float v) {
      if (bans_ && v <= kBanned) return;  // :118
      const bool allowed = ok(t);
      if (first && !allowed) flags_ |= ARCS_FLAG_FIRST_REFUSED;  // tools/server_chat.h:542
      first = false;
      if (allowed) {
        c.push_back(t);
        cv.push_back(v);
      }
    };
    for (int r = 0; r < n_head_ && (int)c.size() < need; ++r) test(head_id_[r], head_val_[r]);
    if ((int)c.size() < need && V > ARCS_HEAD && n_head_ == ARCS_HEAD) {
      if (!c.empty() && (cv[0] - head_val_[ARCS_HEAD - 1]) / p_.temperature > 20.0f) {  // :111
        flags_ |= ARCS_FLAG_TAIL_SKIPPED;
      } else {  // :112-115: the rest of the vocabulary, sorted
        flags_ |= ARCS_FLAG_TAIL_USED;
        const std::vector<float>& adj = adjusted(raw, recent);
        std::vector<char> in_head((size_t)V, 0);
        for (int r = 0; r < n_head_; ++r) in_head[(size_t)head_id_[r]] = 1;
        std::vector<int> rest;
        rest.reserve((size_t)V - ARCS_HEAD);
        for (int t = 0; t < V; ++t)
          if (!in_head[(size_t)t]) rest.push_back(t);
        std::sort(rest.begin(), rest.end(), [&](int x, int y) { return adj[x] > adj[y] || (adj[x] == adj[y] && x < y); });
        for (size_t r = 0; r < rest.size() && (int)c.size() < need; ++r) test(rest[r], adj[rest[r]]);
      }
    }
    if (c.empty()) return -1;                                       // :121
    if (p_.temperature <= 0.0f || c.size() == 1) return c[0];       // :122, no draw
    double u = (double)rng_() * 5.42101086242752217e-20;  // 2^-64
    if (u >= 1.0) u = std::nextafter(1.0, 0.0);
    const arcs_row_params rp = row_params();
    int32_t token = -1;
    if (arcs_draw_candidates_host(ctx_, c.data(), cv.data(), (int32_t)c.size(), &rp, u, V, &token, nullptr) != ARCS_OK)
      throw std::runtime_error(std::string("arcs_draw_candidates_host: ") + arcs_last_error());
    return token;
  }
  // the mask form: bit t of allowed_bits is ok(t) (built on the device by arcs_dfa_mask for a byte automaton)
  int sample_masked(const std::vector<float>& raw, const std::vector<int>& recent, const uint32_t* allowed_bits) {
    int32_t n_cand = 0;
    return run(raw, recent, allowed_bits, /*draw=*/true, &n_cand, false);
  }
  // tools/sampler.h:147-176: the input itself when nothing is set
  const std::vector<float>& adjusted(const std::vector<float>& logits, const std::vector<int>& recent) {
    const bool fp = p_.frequency_penalty != 0.0f, rp = p_.repeat_penalty != 1.0f && p_.repeat_penalty > 0.0f && p_.repeat_last_n != 0;
    const bool pp = p_.presence_penalty != 0.0f;
    if (!fp && !rp && !pp && p_.logit_bias.empty()) return logits;
    const int V = (int)logits.size();
    adj_.resize((size_t)V);
    if (V == 0) return adj_;
    check_vocab(V);
    const arcs_row_params rpm = row_params();
    size_t h0 = 0;
    const int32_t nh = needed_history(recent, &h0);
    const int32_t hoff[2] = {0, nh}, boff[2] = {0, (int32_t)bias_id_.size()};
    arcs_adjusted_args a{};
    a.logits = logits.data();
    a.dtype = ARCS_F32;
    a.B = 1;
    a.V = V;
    a.row_stride = V;
    a.params = &rpm;
    a.hist_off = hoff;
    a.hist_ids = recent.data() + h0;
    a.bias_off = boff;
    a.bias_ids = bias_id_.data();
    a.bias_vals = bias_val_.data();
    a.out = adj_.data();
    a.out_stride = V;
    if (arcs_adjusted_batch_host(ctx_, &a) != ARCS_OK) throw std::runtime_error(std::string("arcs_adjusted_batch_host: ") + arcs_last_error());
    return adj_;
  }
  int last_flags() const { return flags_; }  // ARCS_FLAG_* of the last call (FIRST_REFUSED: tools/server_chat.h:542)

 private:
  static constexpr int64_t kMaxRecent = 1 << 16;  // most history ids one device call takes
  arcs_row_params row_params() const {
    return arcs_row_params{p_.temperature, p_.top_p,         p_.min_p,         p_.presence_penalty,
                           p_.frequency_penalty, p_.repeat_penalty, p_.repeat_last_n, p_.top_k};
  }
  void check_vocab(int V) const {
    if (V > max_vocab_) throw std::runtime_error("Sampler: vocabulary larger than the sampler was created for");
  }
  // The part of `recent` the penalties read (tools/sampler.h:156-172): nothing when no penalty is
  // set, the last repeat_last_n ids when only the repeat penalty is, else all of it.
  int32_t needed_history(const std::vector<int>& recent, size_t* first) const {
    const bool fp = p_.frequency_penalty != 0.0f, pp = p_.presence_penalty != 0.0f;
    const bool rp = p_.repeat_penalty != 1.0f && p_.repeat_penalty > 0.0f && p_.repeat_last_n != 0;
    size_t n = 0;
    if (fp || pp) n = recent.size();
    else if (rp) n = p_.repeat_last_n < 0 ? recent.size() : std::min(recent.size(), (size_t)p_.repeat_last_n);
    if ((int64_t)n > kMaxRecent) throw std::runtime_error("Sampler: history longer than the sampler's device buffers");
    *first = recent.size() - n;
    return (int32_t)n;
  }
  // one device call: Sampler::sample (mask == nullptr) or the constrained form with a mask;
  // draw: a uniform number is taken from the generator (and given back when the call used none)
  int run(const std::vector<float>& raw, const std::vector<int>& recent, const uint32_t* mask, bool draw, int32_t* n_cand, bool want_head) {
    const int V = (int)raw.size();
    if (V == 0) return -1;
    check_vocab(V);
    const arcs_row_params rp = row_params();
    size_t h0 = 0;
    const int32_t nh = needed_history(recent, &h0);
    const int32_t hoff[2] = {0, nh}, boff[2] = {0, (int32_t)bias_id_.size()};
    const std::mt19937_64 saved = rng_;
    double u = 0.0;
    if (draw) {
      u = (double)rng_() * 5.42101086242752217e-20;  // 2^-64
      if (u >= 1.0) u = std::nextafter(1.0, 0.0);
    }
    int32_t token = -1, flags = 0;
    arcs_sample_args a{};
    a.logits = raw.data();
    a.dtype = ARCS_F32;
    a.B = 1;
    a.V = V;
    a.row_stride = V;
    a.params = &rp;
    a.hist_off = hoff;
    a.hist_ids = recent.data() + h0;
    a.max_hist = nh;
    a.bias_off = boff;
    a.bias_ids = bias_id_.data();
    a.bias_vals = bias_val_.data();
    a.max_bias = boff[1];
    a.u = &u;
    a.mask = mask;
    a.mask_stride = (V + 31) / 32;
    a.token = &token;
    a.n_cand = n_cand;
    a.flags = &flags;
    if (want_head) {
      a.head_id = head_id_.data();
      a.head_val = head_val_.data();
      a.n_head = &n_head_;
    }
    if (arcs_sample_batch_host(ctx_, &a) != ARCS_OK) throw std::runtime_error(std::string("arcs_sample_batch_host: ") + arcs_last_error());
    if (!want_head) flags_ = flags;
    // tools/sampler.h:38 and :122: a greedy call, and a constrained call with at most one candidate, draw nothing
    if (draw && (p_.temperature <= 0.0f || (mask && *n_cand <= 1))) rng_ = saved;
    return token;
  }
  SamplingParams p_;
  std::mt19937_64 rng_;
  int max_vocab_;
  bool bans_ = false;
  std::vector<int32_t> bias_id_;
  std::vector<float> bias_val_;
  std::vector<uint32_t> mask_;
  std::vector<float> adj_, head_val_;
  std::vector<int32_t> head_id_;
  int32_t n_head_ = 0;
  arcs_host_ctx* ctx_ = nullptr;
  int32_t flags_ = 0;
};

}  // namespace arcinfer_b200
