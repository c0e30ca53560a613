// C-ABI shim around the reference's OWN sources, compiled from where they lie in the
// reference tree (include path given on the command line; nothing is copied). TEST AND
// BASELINE INFRASTRUCTURE ONLY: it validates the plain-C restatement in arcs_oracle.c,
// generates the fixtures under tests/golden/, and is the "reference" CPU baseline that
// bench.py times. The output (oracle/_ref/libarcs_ref.so) is not tracked.
//
// Wrapped: Sampler / SamplingParams (tools/sampler.h), jcon::Checker
// (tools/json_constraint.h), tcon::GemmaCall / QwenCall (tools/tool_constraint.h).
#include "tools/sampler.h"
#include "tools/json_constraint.h"
#include "tools/tool_constraint.h"

#include <atomic>
#include <chrono>
#include <cstring>
#include <memory>
#include <thread>

extern "C" {

struct ref_params {  // layout of orc_params / arcs_row_params
  float temperature, top_p, min_p, presence_penalty, frequency_penalty, repeat_penalty;
  int32_t repeat_last_n, top_k;
};

static SamplingParams make(const ref_params* p, uint64_t seed, const int32_t* bias_id, const float* bias_val, int nb) {
  SamplingParams s;
  s.temperature = p->temperature;
  s.top_p = p->top_p;
  s.min_p = p->min_p;
  s.presence_penalty = p->presence_penalty;
  s.frequency_penalty = p->frequency_penalty;
  s.repeat_penalty = p->repeat_penalty;
  s.repeat_last_n = p->repeat_last_n;
  s.top_k = p->top_k;
  s.seed = seed;
  for (int i = 0; i < nb; ++i) s.logit_bias.push_back({bias_id[i], bias_val[i]});
  return s;
}

// ndraws calls of Sampler::sample on one Sampler(seed); with append != 0 each drawn token is
// appended to the history before the next call (as tests/test_sampler.cpp:315-319 does).
int ref_sample_seq(const ref_params* p, uint64_t seed, const int32_t* bias_id, const float* bias_val, int nb,
                   const float* logits, int V, const int32_t* hist, int H, int ndraws, int append,
                   int32_t* out_tokens) {
  Sampler s(make(p, seed, bias_id, bias_val, nb));
  const std::vector<float> l(logits, logits + V);
  std::vector<int> rec(hist, hist + H);
  for (int d = 0; d < ndraws; ++d) {
    out_tokens[d] = s.sample(l, rec);
    if (append) rec.push_back(out_tokens[d]);
  }
  return 0;
}

// the same for Sampler::sample_allowed with a bitmask predicate; out_ncalls[d] = predicate calls,
// out_first[d] = 1 when the first call was refused (tools/server_chat.h:538-545)
int ref_sample_allowed_seq(const ref_params* p, uint64_t seed, const int32_t* bias_id, const float* bias_val,
                           int nb, const float* logits, int V, const int32_t* hist, int H,
                           const uint32_t* allowed, int ndraws, int append, int32_t* out_tokens,
                           int32_t* out_ncalls, int32_t* out_first) {
  Sampler s(make(p, seed, bias_id, bias_val, nb));
  const std::vector<float> l(logits, logits + V);
  std::vector<int> rec(hist, hist + H);
  for (int d = 0; d < ndraws; ++d) {
    int calls = 0, first_refused = 0;
    out_tokens[d] = s.sample_allowed(l, rec, [&](int t) {
      const bool ok = (allowed[t >> 5] >> (t & 31)) & 1u;
      if (calls == 0 && !ok) first_refused = 1;
      ++calls;
      return ok;
    });
    if (out_ncalls) out_ncalls[d] = calls;
    if (out_first) out_first[d] = first_refused;
    if (append && out_tokens[d] >= 0) rec.push_back(out_tokens[d]);
  }
  return 0;
}

int ref_adjusted(const ref_params* p, const int32_t* bias_id, const float* bias_val, int nb, const float* logits,
                 int V, const int32_t* hist, int H, float* out) {
  Sampler s(make(p, 1, bias_id, bias_val, nb));
  const std::vector<float> l(logits, logits + V);
  const std::vector<int> rec(hist, hist + H);
  const std::vector<float>& a = s.adjusted(l, rec);
  std::memcpy(out, a.data(), sizeof(float) * (size_t)V);
  return &a != &l;
}

// n successive draws of std::uniform_real_distribution<double>(0, tot) on mt19937_64(seed)
void ref_uniform(uint64_t seed, double tot, int n, double* out) {
  std::mt19937_64 g(seed);
  for (int i = 0; i < n; ++i) {
    std::uniform_real_distribution<double> u(0.0, tot);
    out[i] = u(g);
  }
}

// Timed batch for the CPU baseline: rows [B][V] fp32, per-row params / history CSR / seed; one
// Sampler per row (the server builds one per request, tools/server_chat.h:381); rows are handed
// to `threads` workers. With allowed != nullptr (one mask of mask_words words per row) it calls
// sample_allowed. Returns the wall time of the sampling loop in seconds.
double ref_sample_batch(const ref_params* p, const uint64_t* seeds, const float* logits, int64_t B, int V,
                        const int32_t* hist_off, const int32_t* hist, const uint32_t* allowed,
                        int64_t mask_words, int threads, int32_t* out_tokens) {
  if (threads < 1) threads = 1;
  std::atomic<int64_t> next{0};
  auto work = [&]() {
    std::vector<float> l((size_t)V);
    for (;;) {
      const int64_t b = next.fetch_add(1);
      if (b >= B) break;
      // (the reference's caller owns a std::vector<float>; the copy stands for the read-back of
      //  the row from the device, zero/engine.h:255)
      std::memcpy(l.data(), logits + (size_t)b * V, sizeof(float) * (size_t)V);
      Sampler s(make(&p[b], seeds[b] ? seeds[b] : 1, nullptr, nullptr, 0));
      const std::vector<int> rec(hist + hist_off[b], hist + hist_off[b + 1]);
      if (allowed) {
        const uint32_t* m = allowed + (size_t)b * mask_words;
        out_tokens[b] = s.sample_allowed(l, rec, [&](int t) { return (bool)((m[t >> 5] >> (t & 31)) & 1u); });
      } else {
        out_tokens[b] = s.sample(l, rec);
      }
    }
  };
  const auto t0 = std::chrono::steady_clock::now();
  std::vector<std::thread> th;
  for (int i = 1; i < threads; ++i) th.emplace_back(work);
  work();
  for (auto& t : th) t.join();
  return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
}

int ref_hardware_threads() { return (int)std::thread::hardware_concurrency(); }

// jcon::Checker::check (tools/json_constraint.h:37-47) on a schema given as JSON text:
// 0 FAIL, 1 PARTIAL, 2 DONE, -1 schema does not parse
int ref_jcon_check(const char* schema_json, int object_only, const char* text, int text_len) {
  Json sc;
  if (!Json::try_parse(schema_json, sc)) return -1;
  jcon::Checker c(sc, object_only != 0);
  return (int)c.check(std::string(text, (size_t)text_len));
}

// tcon::GemmaCall (kind 0) / tcon::QwenCall (kind 1) check on the text after the open marker
int ref_tcon_check(int kind, const char* tools_json, const char* text, int text_len) {
  Json tools;
  if (!Json::try_parse(tools_json, tools)) return -1;
  std::unique_ptr<tcon::ToolCon> c;
  if (kind == 0) c.reset(new tcon::GemmaCall(tools));
  else c.reset(new tcon::QwenCall(tools));
  return (int)c->check(std::string(text, (size_t)text_len));
}

}  // extern "C"
