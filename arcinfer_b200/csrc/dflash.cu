// arcs_dflash_select: the DFlash2 drafter's candidate selector (zero/engine_drafters.h:461-506)
// for many slots at once.
//
// Two steps. What does not depend on the path - per draft position the K largest raw logits in
// (value descending, id ascending) order and the row's log-sum-exp - is one pass over all
// slots' rows: arcs_logprobs_batch. The path itself is sequential over the (at most 7)
// positions of a slot, because a position's scores depend on the token chosen before it: one
// warp per slot walks it, a candidate to a lane. A candidate's score is accumulated exactly as
// the reference does (:489-493): float products, added one by one in index order to a double
// that starts at the logit, so that the comparison of scores falls as it does there.
#include "common.cuh"
#include "plan.h"

namespace arcs {

constexpr int kDflMaxRank = 1024;  // the reference's own bound (its ph[1024], :486)
constexpr int kDflMaxK = 64;

struct DflDev {
  const void* logits;
  int64_t row_stride;
  int32_t slots, nd, V, rank, K, steps;
  const float* hproj;
  const uint16_t* pred;
  const uint16_t* succ;
  const int32_t* tok;
  double min_p;
  const int32_t* top_id;  // [slots * nd][K] from the first step
  const double* lse;      // [slots * nd]
  int32_t* n_out;
  int32_t* out_tokens;
  int32_t out_stride;
  double* path_p;         // [slots][nd] optional
  int32_t* status;
};

__device__ __forceinline__ float bf16_bits(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
template <typename T>
__device__ __forceinline__ float raw_logit(const void* row, int32_t i);
template <>
__device__ __forceinline__ float raw_logit<float>(const void* row, int32_t i) { return __ldg(static_cast<const float*>(row) + i); }
template <>
__device__ __forceinline__ float raw_logit<__nv_bfloat16>(const void* row, int32_t i) {
  return bf16_bits(__ldg(static_cast<const uint16_t*>(row) + i));
}

template <typename T>
__global__ void __launch_bounds__(32) dflash_path_kernel(const DflDev a) {
  __shared__ float ph[kDflMaxRank];
  const int s = blockIdx.x, lane = threadIdx.x;
  int32_t prev = __ldg(&a.tok[s]);
  double path_p = 1.0;
  int n_out = 0;
  for (int t = 0; t < a.steps; ++t) {
    if (prev < 0 || prev >= a.V) {  // (a token outside the codebooks: nothing can be scored from it)
      if (lane == 0) raise_status(a.status, ARCS_ERR_ARG);
      break;
    }
    const size_t row = (size_t)s * a.nd + t;
    const char* l = static_cast<const char*>(a.logits) + row * (size_t)a.row_stride * sizeof(T);
    const int32_t* ids = a.top_id + row * a.K;
    const float* h = a.hproj + row * a.rank;
    __syncwarp();
    for (int r = lane; r < a.rank; r += 32) ph[r] = __fmul_rn(bf16_bits(__ldg(&a.pred[(size_t)prev * a.rank + r])), __ldg(&h[r]));  // :487
    __syncwarp();
    // :488-495. A lane's candidates come in rising k, so "the first among equals" holds inside a
    // lane by the strict comparison and between lanes by the smaller k.
    double best = -1e300;
    int bk = 0x7FFFFFFF;
    for (int k = lane; k < a.K; k += 32) {
      const int32_t c = __ldg(&ids[k]);
      if (c < 0) continue;  // (fewer than K numbers in the row)
      double sc = (double)raw_logit<T>(l, c);
      const uint16_t* sv = a.succ + (size_t)c * a.rank;
      if ((a.rank & 7) == 0 && (reinterpret_cast<uintptr_t>(sv) & 15u) == 0) {
        for (int r0 = 0; r0 < a.rank; r0 += 8) {
          const uint4 q = __ldg(reinterpret_cast<const uint4*>(sv + r0));
          const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            sc = __dadd_rn(sc, (double)__fmul_rn(ph[r0 + 2 * j], __uint_as_float(w[j] << 16)));
            sc = __dadd_rn(sc, (double)__fmul_rn(ph[r0 + 2 * j + 1], __uint_as_float(w[j] & 0xFFFF0000u)));
          }
        }
      } else {
        for (int r = 0; r < a.rank; ++r) sc = __dadd_rn(sc, (double)__fmul_rn(ph[r], bf16_bits(__ldg(&sv[r]))));
      }
      if (sc > best) {
        best = sc;
        bk = k;
      }
    }
    double top = best;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmax(top, __shfl_xor_sync(0xFFFFFFFFu, top, o));
    int k_win = (bk != 0x7FFFFFFF && best == top) ? bk : 0x7FFFFFFF;
    k_win = (int)__reduce_min_sync(0xFFFFFFFFu, (unsigned)k_win);
    const int32_t first = __ldg(&ids[0]);
    const int32_t bt = k_win != 0x7FFFFFFF ? __ldg(&ids[k_win]) : first;  // (no score above -1e300: the best logit, :489)
    if (bt < 0) break;  // (a row without a single number)
    if (a.min_p > 0.0) {  // :496-503
      const float mx = raw_logit<T>(l, first);  // (the candidates are sorted: the first holds the largest logit)
      const double z = exp(__ldg(&a.lse[row]) - (double)mx);
      path_p *= exp((double)raw_logit<T>(l, bt) - (double)mx) / z;
      if (a.path_p && lane == 0) a.path_p[row] = path_p;
      if (t > 0 && path_p < a.min_p) break;  // (the first draft always goes)
    }
    if (lane == 0) a.out_tokens[(size_t)s * a.out_stride + n_out] = bt;
    ++n_out;
    prev = bt;
  }
  if (lane == 0) a.n_out[s] = n_out;
}

static size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }

}  // namespace arcs

extern "C" size_t arcs_dflash_workspace_bytes(int32_t slots, int32_t nd, int32_t V, int32_t topk) {
  using namespace arcs;
  if (slots <= 0 || nd <= 0 || V <= 0 || topk <= 0) return 0;
  const int K = topk < V ? topk : V;
  const size_t R = (size_t)slots * nd;
  return up256(arcs_logprobs_workspace_bytes((int32_t)R, V, K)) + up256(R * K * 4) + up256(R * K * 8) + up256(R * 8);
}

extern "C" int arcs_dflash_select(const arcs_dflash_args* g, void* stream) {
  using namespace arcs;
  if (int inj = fault_injected()) return inj;
  if (!g || !g->logits || !g->hproj || !g->pred || !g->succ || !g->tok || !g->n_out || !g->out_tokens || g->slots <= 0 || g->nd <= 0 ||
      g->V <= 0 || g->row_stride < g->V || (g->dtype != ARCS_F32 && g->dtype != ARCS_BF16) || g->max_drafts < 0 ||
      g->out_stride < (g->max_drafts < g->nd ? g->max_drafts : g->nd))
    return set_error(ARCS_ERR_ARG, "dflash_select: bad argument");
  if (g->rank <= 0 || g->rank > kDflMaxRank) return set_error(ARCS_ERR_ARG, "dflash_select: rank must be 1 .. 1024");
  if (g->topk <= 0 || g->topk > kDflMaxK) return set_error(ARCS_ERR_TOPK, "dflash_select: topk must be 1 .. 64");
  if ((int64_t)g->slots * g->nd > (1 << 20)) return set_error(ARCS_ERR_ARG, "dflash_select: too many rows");
  const int K = g->topk < g->V ? g->topk : g->V;
  const size_t R = (size_t)g->slots * g->nd;
  if (!g->workspace || g->workspace_bytes < arcs_dflash_workspace_bytes(g->slots, g->nd, g->V, g->topk))
    return set_error(ARCS_ERR_WORKSPACE, "dflash_select: workspace too small");
  if ((reinterpret_cast<uintptr_t>(g->workspace) & 255u) != 0) return set_error(ARCS_ERR_WORKSPACE, "dflash_select: workspace must be 256-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  char* p = static_cast<char*>(g->workspace);
  const size_t lp_bytes = up256(arcs_logprobs_workspace_bytes((int32_t)R, g->V, K));
  int32_t* top_id = reinterpret_cast<int32_t*>(p + lp_bytes);
  double* top_lp = reinterpret_cast<double*>(p + lp_bytes + up256(R * K * 4));
  double* lse = reinterpret_cast<double*>(p + lp_bytes + up256(R * K * 4) + up256(R * K * 8));
  // (entries the first step does not write - a row with fewer than K numbers - read as "no candidate")
  if (cudaMemsetAsync(top_id, 0xFF, R * K * 4, st) != cudaSuccess) return set_error(ARCS_ERR_CUDA, "dflash_select: memset failed");
  arcs_logprob_args lp = {};
  lp.logits = g->logits;
  lp.dtype = g->dtype;
  lp.B = (int32_t)R;
  lp.V = g->V;
  lp.row_stride = g->row_stride;
  lp.top_n = K;
  lp.top_stride = K;
  lp.lse = lse;
  lp.top_id = top_id;
  lp.top_logprob = top_lp;
  lp.workspace = p;
  lp.workspace_bytes = lp_bytes;
  lp.status = g->status;
  if (const int rc = arcs_logprobs_batch(&lp, stream)) return rc;
  DflDev a;
  a.logits = g->logits;
  a.row_stride = g->row_stride;
  a.slots = g->slots;
  a.nd = g->nd;
  a.V = g->V;
  a.rank = g->rank;
  a.K = K;
  a.steps = g->nd < g->max_drafts ? g->nd : g->max_drafts;
  a.hproj = g->hproj;
  a.pred = g->pred;
  a.succ = g->succ;
  a.tok = g->tok;
  a.min_p = g->min_p;
  a.top_id = top_id;
  a.lse = lse;
  a.n_out = g->n_out;
  a.out_tokens = g->out_tokens;
  a.out_stride = g->out_stride;
  a.path_p = g->path_p;
  a.status = g->status;
  if (g->dtype == ARCS_F32) dflash_path_kernel<float><<<(unsigned)g->slots, 32, 0, st>>>(a);
  else dflash_path_kernel<__nv_bfloat16><<<(unsigned)g->slots, 32, 0, st>>>(a);
  return check_launch("dflash_select");
}
