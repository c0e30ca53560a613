// Binds the names the reference's own sampler test uses (`SamplingParams`, `Sampler`, global
// namespace) to the CUDA-backed mirror, so that the test's comparisons against its verbatim copy
// of the earlier implementation (`OldSampler`) run against this library. The reference's
// tools/sampler.h is included from where it lies (include path given on the command line) with
// its class renamed, for `SamplingParams` alone. Test infrastructure only.
#pragma once
#define Sampler ReferenceCpuSampler
#include "tools/sampler.h"
#undef Sampler
#include "../../arcinfer_b200/host/sampler_b200.hpp"

class Sampler {
 public:
  static constexpr float kBanned = arcinfer_b200::Sampler::kBanned;
  explicit Sampler(const SamplingParams& p) : s_(convert(p)) {}
  int sample(const std::vector<float>& raw, const std::vector<int>& recent) { return s_.sample(raw, recent); }
  int sample_allowed(const std::vector<float>& raw, const std::vector<int>& recent, const std::function<bool(int)>& ok) {
    return s_.sample_allowed(raw, recent, ok);
  }
  const std::vector<float>& adjusted(const std::vector<float>& logits, const std::vector<int>& recent) { return s_.adjusted(logits, recent); }

 private:
  static arcinfer_b200::SamplingParams convert(const SamplingParams& p) {
    arcinfer_b200::SamplingParams q;
    q.temperature = p.temperature;
    q.top_p = p.top_p;
    q.min_p = p.min_p;
    q.presence_penalty = p.presence_penalty;
    q.frequency_penalty = p.frequency_penalty;
    q.repeat_penalty = p.repeat_penalty;
    q.repeat_last_n = p.repeat_last_n;
    q.top_k = p.top_k;
    q.seed = p.seed;
    q.logit_bias = p.logit_bias;
    return q;
  }
  arcinfer_b200::Sampler s_;
};
