// C-ABI wrappers around FRAGMENTS of the reference's sources that cannot be compiled as whole
// files here (their headers pull Win32 / Level Zero): the Makefile cuts the few lines that hold
// the arithmetic out of the reference tree, where they lie, into oracle/_ref/*.inc at build time
// (untracked, nothing is copied into this repository), and this file gives them a function to
// live in. TEST INFRASTRUCTURE ONLY: it pins the plain-C restatements of arcs_oracle.c.
//
//   lp_lse.inc       tools/server_chat.h   the `mx`, `z`, `lse` lines of the lp_entry lambda
//   lp_top.inc       tools/server_chat.h   the index array + std::partial_sort lines of the same lambda
//   softmax_den.inc  zero/engine_drafters.h  static double softmax_den(const float*, size_t, float)
//   dflash_select.inc zero/engine_drafters.h  the candidate-selector loop of dflash_draft()
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

namespace {
struct Slices {
#include "_ref/softmax_den.inc"
};
inline float bf16_to_f32(uint16_t v) {  // exact widening (what the reference's helper of that name does)
  uint32_t u = (uint32_t)v << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
}  // namespace

extern "C" {

double ref_softmax_den(const float* l, int64_t n, float mx) { return Slices::softmax_den(l, (size_t)n, mx); }

// lp_entry: lse of the row, the token's log probability, the top_lp alternatives in the order
// std::partial_sort leaves them
double ref_lp_entry(const float* l, int V, int tok, int top_lp, double* logprob, int32_t* top_id, double* top_logprob) {
  const std::vector<float> lg(l, l + V);
#include "_ref/lp_lse.inc"
  if (tok >= 0 && logprob) *logprob = (double)lg[tok] - lse;
  if (top_lp > 0) {
#include "_ref/lp_top.inc"
    for (int i = 0; i < top_lp; ++i) {
      top_id[i] = idx[i];
      top_logprob[i] = (double)lg[idx[i]] - lse;
    }
  }
  return lse;
}

// The DFlash2 candidate selector (greedy path over nd positions): logits [nd][V] fp32, projected
// hidden states [nd][rank] fp32, codebooks pred / succ [V][rank] bf16 bit patterns. Returns the
// number of drafts kept, written to out_tokens. min_p_arg replaces the ARC_DFL_P environment
// default (0.3) of the reference.
int ref_dflash_select(const float* logits, const float* hproj, const uint16_t* pred, const uint16_t* succ, int V,
                      int rank, int topk, int nd, int max_drafts, int tok, double min_p_arg, int32_t* out_tokens) {
  const float* dfl_lg_base = logits;
  const float* dfl_hph_base = hproj;
  struct View {
    const float* p;
    const float& operator[](size_t i) const { return p[i]; }
  } dfl_lg_{dfl_lg_base}, dfl_hph_{dfl_hph_base};
  const uint16_t* dfl_pred_ = pred;
  const uint16_t* dfl_succ_ = succ;
  const int dfl_rank_ = rank, dfl_topk_ = topk;
  const double min_p = min_p_arg;
  auto softmax_den = [](const float* l, size_t n, float mx) { return Slices::softmax_den(l, n, mx); };
#include "_ref/dflash_select.inc"
  for (size_t i = 0; i < out.size(); ++i) out_tokens[i] = out[i];
  return (int)out.size();
}

}  // extern "C"
