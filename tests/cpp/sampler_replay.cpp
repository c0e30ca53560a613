// Replays a recorded sequence of sampler calls through the C++ mirror of the reference's Sampler
// (arcinfer_b200/host/sampler_b200.hpp) and prints the tokens, one per line. Test program: the
// Python test writes the case file and compares the output with the CPU oracle.
//
// case file (little endian): int32 V, n_recent, n_bias, n_calls, masked, append; float temperature,
// top_p, min_p, presence_penalty, frequency_penalty, repeat_penalty; int32 repeat_last_n, top_k;
// uint64 seed; float logits[V]; int32 recent[n_recent]; int32 bias_id[n_bias]; float
// bias_val[n_bias]; uint32 mask[(V + 31) / 32] when masked.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../../arcinfer_b200/host/sampler_b200.hpp"

template <typename T>
static bool rd(FILE* f, T* p, size_t n) { return n == 0 || fread(p, sizeof(T), n, f) == n; }

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  FILE* f = fopen(argv[1], "rb");
  if (!f) return 2;
  int32_t h[6];
  arcinfer_b200::SamplingParams p;
  bool ok = rd(f, h, 6) && rd(f, &p.temperature, 1) && rd(f, &p.top_p, 1) && rd(f, &p.min_p, 1) && rd(f, &p.presence_penalty, 1) &&
            rd(f, &p.frequency_penalty, 1) && rd(f, &p.repeat_penalty, 1) && rd(f, &p.repeat_last_n, 1) && rd(f, &p.top_k, 1) &&
            rd(f, &p.seed, 1);
  const int V = h[0], n_recent = h[1], n_bias = h[2], n_calls = h[3], masked = h[4], append = h[5];
  std::vector<float> logits(V), bval(n_bias);
  std::vector<int> recent(n_recent), bid(n_bias);
  std::vector<uint32_t> mask(masked ? (V + 31) / 32 : 0);
  ok = ok && rd(f, logits.data(), V) && rd(f, recent.data(), n_recent) && rd(f, bid.data(), n_bias) && rd(f, bval.data(), n_bias) &&
       rd(f, mask.data(), mask.size());
  fclose(f);
  if (!ok) return 3;
  for (int i = 0; i < n_bias; ++i) p.logit_bias.push_back({bid[i], bval[i]});
  try {
    arcinfer_b200::Sampler s(p, V);
    for (int c = 0; c < n_calls; ++c) {
      const int t = masked ? s.sample_allowed(logits, recent, [&](int x) { return ((mask[x >> 5] >> (x & 31)) & 1u) != 0; })
                           : s.sample(logits, recent);
      printf("%d\n", t);
      if (append && t >= 0) recent.push_back(t);
    }
  } catch (const std::exception& e) {
    fprintf(stderr, "%s\n", e.what());
    return 4;
  }
  return 0;
}
