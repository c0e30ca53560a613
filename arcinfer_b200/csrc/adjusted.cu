// adjusted_batch: the penalised logits of whole rows, Sampler::adjusted (tools/sampler.h:147-176),
// as fp32: logit_bias added (entries above -100, in list order, duplicates add again), frequency
// penalty times the count over the whole history, repeat penalty over the unique ids of the last
// repeat_last_n entries, presence penalty once per unique id, bans (-1e30) last. Every operation
// is a separate fp32 rounding in the reference's order. Two launches: an elementwise copy that
// widens the row, and one CTA per row that rewrites the touched tokens.
#include <algorithm>

#include "sample_common.cuh"

namespace arcs {

template <typename T>
__global__ void __launch_bounds__(256) widen_rows_kernel(const T* __restrict__ in, int64_t in_stride, float* __restrict__ out,
                                                         int64_t out_stride, int32_t V) {
  const T* row = in + (size_t)blockIdx.y * in_stride;
  float* o = out + (size_t)blockIdx.y * out_stride;
  for (int32_t i = blockIdx.x * 256 + threadIdx.x; i < V; i += gridDim.x * 256) o[i] = Elem<T>::load(row + i);
}

template <typename T>
__global__ void __launch_bounds__(256) touch_rows_kernel(const SampleDev a, float* __restrict__ out, int64_t out_stride) {
  const int b = blockIdx.x, gt = threadIdx.x;
  const RowCfg r = row_cfg<false>(a, b);
  const T* row = reinterpret_cast<const T*>(a.logits) + (size_t)b * a.row_stride;
  float* o = out + (size_t)b * out_stride;
  if (!r.pen_on && r.NB == 0) return;  // tools/sampler.h:151: nothing is set, the row is the input itself
  const int32_t w0 = window_start(r);
  // what the bias list does to token t, in list order (:154-155, :173-174)
  auto biased = [&](int32_t t, float v, bool& ban) {
    for (int j = 0; j < r.NB; ++j) {
      if (a.bias_ids[r.q0 + j] != t) continue;
      const float bv = a.bias_vals[r.q0 + j];
      if (bv > -100.0f) v = __fadd_rn(v, bv);
      else ban = true;
    }
    return v;
  };
  if (r.pen_on) {
    for (int i = gt; i < r.H; i += 256) {
      const int32_t t = __ldg(&a.hist_ids[r.h0 + i]);
      if (t < 0 || t >= a.V) continue;
      uint32_t cnt = 0;
      bool first = true, in_win = false;
      for (int j = 0; j < r.H; ++j)
        if (__ldg(&a.hist_ids[r.h0 + j]) == t) {
          first = first && j >= i;  // (rewritten once, by the thread of the id's first entry)
          ++cnt;
          in_win = in_win || j >= w0;
        }
      if (!first) continue;
      bool ban = false;
      float v = biased(t, Elem<T>::load(row + t), ban);
      v = penalise(r, v, cnt, in_win);
      o[t] = ban ? ARCS_BANNED : v;
    }
  }
  for (int i = gt; i < r.NB; i += 256) {
    const int32_t t = a.bias_ids[r.q0 + i];
    if (t < 0 || t >= a.V) continue;
    bool first = true;
    for (int j = 0; j < i && first; ++j) first = a.bias_ids[r.q0 + j] != t;
    if (r.pen_on)
      for (int j = 0; j < r.H && first; ++j) first = __ldg(&a.hist_ids[r.h0 + j]) != t;  // (done above with the history)
    if (!first) continue;
    bool ban = false;
    const float v = biased(t, Elem<T>::load(row + t), ban);
    o[t] = ban ? ARCS_BANNED : v;
  }
}

}  // namespace arcs

using namespace arcs;

extern "C" int arcs_adjusted_batch(const arcs_adjusted_args* g, void* stream) {
  if (int inj = fault_injected()) return inj;
  if (!g || !g->logits || !g->params || !g->out || g->B <= 0 || g->V <= 0 || g->row_stride < g->V || g->out_stride < g->V ||
      (g->dtype != ARCS_F32 && g->dtype != ARCS_BF16))
    return set_error(ARCS_ERR_ARG, "adjusted_batch: bad argument");
  if ((g->hist_off && !g->hist_ids) || (g->bias_off && (!g->bias_ids || !g->bias_vals)))
    return set_error(ARCS_ERR_ARG, "adjusted_batch: list offsets without the list");
  SampleDev a = {};
  a.logits = g->logits;
  a.row_stride = g->row_stride;
  a.B = g->B;
  a.V = g->V;
  a.nseg = 1;
  a.params = g->params;
  a.hist_off = g->hist_off;
  a.hist_ids = g->hist_ids;
  a.bias_off = g->bias_off;
  a.bias_ids = g->bias_ids;
  a.bias_vals = g->bias_vals;
  a.max_hist = 0x7FFFFFFF;  // (lists of any length: nothing is kept on chip here)
  a.max_bias = 0x7FFFFFFF;
  a.hash_slots = 0x40000000;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid((unsigned)std::min(64, (g->V + 255) / 256), (unsigned)g->B);
  if (g->dtype == ARCS_F32) {
    widen_rows_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(g->logits), g->row_stride, g->out, g->out_stride, g->V);
    touch_rows_kernel<float><<<(unsigned)g->B, 256, 0, st>>>(a, g->out, g->out_stride);
  } else {
    widen_rows_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(g->logits), g->row_stride, g->out, g->out_stride, g->V);
    touch_rows_kernel<__nv_bfloat16><<<(unsigned)g->B, 256, 0, st>>>(a, g->out, g->out_stride);
  }
  return check_launch("adjusted_batch");
}
