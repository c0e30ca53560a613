// logprobs_batch: per row the log-softmax of one token and the top_n largest raw logits as log
// probabilities (tools/server_chat.h:417-441; zero/runz.cpp:478-484 scores perplexity with the
// same sum). One CTA streams one row once through a ring of bulk-copied tiles and keeps
//  - per thread a running (reference value, sum of exponentials relative to it), the sum in fp64;
//  - for the whole CTA a candidate buffer with a rising threshold: the top_n best so far.
#include "plan.h"
#include "select.cuh"
#include "stream.cuh"

namespace arcs {

constexpr int kLpCap = 1024;                  // candidate buffer of a row
constexpr int kLpTrig = kLpCap - kThreads;    // prune when a further round of pushes might not fit

struct LogprobDev {
  const void* logits;
  int64_t row_stride;
  int32_t B, V;
  const int32_t* token;
  int32_t top_n, top_stride;
  double* logprob;
  double* lse;
  int32_t* top_id;
  double* top_logprob;
  int32_t* status;
};

// exp(v - m) for v <= m: a float exponential of the float difference, with the rounding error of
// that difference (recovered exactly by a two-sum) put back to first order
__device__ __forceinline__ float exp_diff(float v, float m) {
  const float s = __fsub_rn(v, m);
  const float bb = __fsub_rn(s, v);
  const float err = __fadd_rn(__fsub_rn(v, __fsub_rn(s, bb)), __fsub_rn(-m, bb));
  const float e = expf(s);
  return e > 0.0f ? fmaf(e, err, e) : 0.0f;  // (also keeps the NaN of inf - inf out when v is -inf)
}

constexpr size_t kLpSmem = (size_t)kStages * kTileBytes + (size_t)kLpCap * 8 + 512 * 4 + (size_t)kTmpCap * 8;

template <typename T>
__global__ void __launch_bounds__(kThreads) logprob_kernel(const LogprobDev a) {
  extern __shared__ __align__(128) char smem[];
  char* stage = smem;
  uint32_t* bkey = reinterpret_cast<uint32_t*>(smem + (size_t)kStages * kTileBytes);
  int32_t* bid = reinterpret_cast<int32_t*>(bkey + kLpCap);
  uint32_t* hist = reinterpret_cast<uint32_t*>(bid + kLpCap);
  uint32_t* tk = hist + 512;
  int32_t* ti = reinterpret_cast<int32_t*>(tk + kTmpCap);
  __shared__ __align__(8) uint64_t bars[kStages];
  __shared__ unsigned long long s_tau, s_m64;
  __shared__ int s_cnt, s_misc[8];
  __shared__ float red_m[kThreads / 32];
  __shared__ double red_s[kThreads / 32], s_lse;

  constexpr int E = Elem<T>::kPerChunk;
  constexpr int kChunks = kTileBytes / 16 / kThreads;
  static_assert(kChunks * E <= 32, "a thread's elements of one tile are tracked in a 32-bit mask");
  const int tid = threadIdx.x, b = blockIdx.x;
  const T* row = reinterpret_cast<const T*>(a.logits) + (size_t)b * a.row_stride;
  const SegPlan p = make_plan(row, 0, a.V);
  const int n = min(a.top_n, a.V);

  Sel sel{bkey, bid, &s_cnt, &s_tau, n, kLpTrig, kLpCap};
  PruneScratch ps{hist, tk, ti, s_misc, &s_m64};

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) mbar_init(&bars[i], 1);
    mbar_init_fence();
    s_cnt = 0;
    s_tau = 0ull;
  }
  __syncthreads();
  if (tid == 0)
    for (int t = 0; t < p.tiles && t < kStages; ++t) issue_tile(p, t, stage, bars);

  float lm = -INFINITY;  // what this thread's exponentials are relative to: at least every value it has seen
  double ls = 0.0;
  unsigned long long tau = 0ull;  // exclusive threshold of the candidate buffer (this thread's copy)

  // one more value for the sum (NaN skipped)
  auto lse_one = [&](float v) {
    if (v > lm) {
      ls *= exp((double)lm - (double)v);
      lm = v;
    }
    if (v == v && lm > -INFINITY) ls += (double)exp_diff(v, lm);
  };
  // Every thread calls: those with p set put (ky, id) into the buffer; when it has grown past the
  // trigger the CTA keeps the n best and the threshold rises.
  auto offer = [&](bool pr, uint32_t ky, int32_t id) {
    bool hot = false;
    sel_push(sel, pr, ky, id, hot, a.status);
    if (__syncthreads_or(hot)) sel_prune<1, kThreads>(sel, n, ps, tid);
    tau = s_tau;
  };

  bool failed = false;
  for (int t = 0; t < p.tiles; ++t) {
    const int slot = t % kStages;
    if (!mbar_wait(&bars[slot], (uint32_t)((t / kStages) & 1))) failed = true;
    const uint32_t nbytes = tile_bytes(p, t);
    uint4 q[kChunks];
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
      const uint32_t off = (uint32_t)(j * kThreads + tid) * 16u;
      q[j] = off < nbytes && !failed ? lds128(stage + (size_t)slot * kTileBytes + off) : make_uint4(0, 0, 0, 0);
    }
    // every thread has taken its chunks: the slot can be refilled
    if (__syncthreads_or(failed)) {
      if (tid == 0) {
        raise_status(a.status, ARCS_ERR_TIMEOUT);
        drain_tiles(p, t, bars);
      }
      __syncthreads();
      return;
    }
    if (tid == 0 && t + kStages < p.tiles) issue_tile(p, t + kStages, stage, bars);

    // ---- the sum of exponentials
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
      const uint32_t off = (uint32_t)(j * kThreads + tid) * 16u;
      if (off >= nbytes) continue;
      const float cm = Elem<T>::chunk_max(q[j]);
      if (cm > lm) {
        ls *= exp((double)lm - (double)cm);
        lm = cm;
      }
      if (lm > -INFINITY) {
        float ev[E];
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float v = Elem<T>::get(q[j], e);
          ev[e] = v == v ? exp_diff(v, lm) : 0.0f;
        }
#pragma unroll
        for (int w = E / 2; w > 0; w >>= 1)
#pragma unroll
          for (int e = 0; e < w; ++e) ev[e] += ev[e + w];
        ls += (double)ev[0];
      }
    }
    if (n <= 0) continue;

    // ---- the candidates
    // element idx (chunk idx / E, position idx % E) of this thread's part of the tile
    auto pick = [&](int idx, int32_t& id) -> float {
      const int j = idx / E;
      uint4 c = q[0];
#pragma unroll
      for (int x = 1; x < kChunks; ++x)
        if (j == x) c = q[x];
      id = p.body_first + (int32_t)(((uint32_t)t * kTileBytes + (uint32_t)(j * kThreads + tid) * 16u) / sizeof(T)) + idx % E;
      return Elem<T>::get(c, idx % E);
    };
    if (t == 0) {
      // first threshold: the n-th largest of the threads' own maxima over this tile is a lower
      // bound of the n-th largest element (the maxima belong to disjoint pieces)
      float bv = -INFINITY;
      int32_t bi = -1;
#pragma unroll
      for (int j = 0; j < kChunks; ++j) {
        const uint32_t off = (uint32_t)(j * kThreads + tid) * 16u;
        if (off >= nbytes) continue;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float v = Elem<T>::get(q[j], e);
          if (v > bv || (bi < 0 && v == v)) {
            bv = v;
            bi = p.body_first + (int32_t)(off / sizeof(T)) + e;
          }
        }
      }
      offer(bi >= 0, key_of(bv), bi);
      if (s_cnt > n) sel_prune<1, kThreads>(sel, n, ps, tid);  // (uniform: nothing is pushed between the barrier in offer and here)
      __syncthreads();
      if (tid == 0) s_cnt = 0;  // only the threshold is kept: the tile is gone through again below
      __syncthreads();
      tau = s_tau;
    }
    const uint32_t tkey = (uint32_t)(tau >> 32);
    const float tf = value_of(tkey < 0x007FFFFFu ? 0x007FFFFFu : tkey);  // inclusive value threshold
    uint32_t bits = 0;  // this thread's elements that may still belong to the n best
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
      const uint32_t off = (uint32_t)(j * kThreads + tid) * 16u;
      if (off >= nbytes) continue;
      if (!(Elem<T>::chunk_max(q[j]) >= tf)) continue;
#pragma unroll
      for (int e = 0; e < E; ++e) bits |= (Elem<T>::get(q[j], e) >= tf ? 1u : 0u) << (j * E + e);
    }
    if (__syncthreads_or(bits != 0u)) {
      for (;;) {
        // this thread's next element above the (current) threshold
        bool pr = false;
        uint32_t ky = 0;
        int32_t id = 0;
        while (bits != 0u && !pr) {
          const int idx = __ffs(bits) - 1;
          bits &= bits - 1u;
          ky = key_of(pick(idx, id));
          pr = ky != 0u && comp_of(ky, id) > tau;
        }
        if (!__syncthreads_or(pr)) break;
        offer(pr, ky, id);
      }
    }
  }

  // ---- the few elements outside the 16-byte aligned body
  {
    const bool hv = tid < p.head_n, tv = tid < p.tail_n;
    const float vh = hv ? Elem<T>::load(row + tid) : 0.0f;
    const float vt = tv ? Elem<T>::load(row + p.tail_first + tid) : 0.0f;
    if (hv) lse_one(vh);
    if (tv) lse_one(vt);
    if (n > 0) {
      uint32_t ky = hv ? key_of(vh) : 0u;
      offer(ky != 0u && comp_of(ky, tid) > tau, ky, tid);
      ky = tv ? key_of(vt) : 0u;
      offer(ky != 0u && comp_of(ky, p.tail_first + tid) > tau, ky, p.tail_first + tid);
    }
  }

  // ---- log of the sum: the threads' sums brought to the row's maximum
  float M = lm;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, o));
  if ((tid & 31) == 0) red_m[tid >> 5] = M;
  __syncthreads();
  M = red_m[0];
#pragma unroll
  for (int w = 1; w < kThreads / 32; ++w) M = fmaxf(M, red_m[w]);
  double part = lm > -INFINITY ? ls * exp((double)lm - (double)M) : 0.0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xFFFFFFFFu, part, o);
  if ((tid & 31) == 0) red_s[tid >> 5] = part;
  __syncthreads();
  if (tid == 0) {
    double z = 0.0;
    for (int w = 0; w < kThreads / 32; ++w) z += red_s[w];
    const double lse = (double)M + log(z);  // tools/server_chat.h:422
    s_lse = lse;
    if (a.lse) a.lse[b] = lse;
    if (a.logprob) {
      const int32_t tok = a.token ? a.token[b] : -1;
      if (tok >= a.V) raise_status(a.status, ARCS_ERR_ARG);
      a.logprob[b] = (tok >= 0 && tok < a.V) ? (double)Elem<T>::load(row + tok) - lse : (double)NAN;  // :427
    }
  }
  if (n <= 0) return;
  __syncthreads();
  if (s_cnt > n) sel_prune<1, kThreads>(sel, n, ps, tid);
  __syncthreads();
  // ---- best first: an entry's place is the number of entries above it (composites are unique)
  const int m = min(s_cnt, n);
  const double lse = s_lse;
  for (int i = tid; i < m; i += kThreads) {
    const uint64_t c = comp_of(bkey[i], bid[i]);
    int rank = 0;
    for (int j = 0; j < m; ++j) rank += comp_of(bkey[j], bid[j]) > c;
    a.top_id[(size_t)b * a.top_stride + rank] = bid[i];
    a.top_logprob[(size_t)b * a.top_stride + rank] = (double)value_of(bkey[i]) - lse;
  }
}

}  // namespace arcs

using namespace arcs;

extern "C" int arcs_logprobs_batch(const arcs_logprob_args* g, void* stream) {
  if (int inj = fault_injected()) return inj;
  if (!g || !g->logits || g->B <= 0 || g->V <= 0 || g->row_stride < g->V || (g->dtype != ARCS_F32 && g->dtype != ARCS_BF16))
    return set_error(ARCS_ERR_ARG, "logprobs_batch: bad argument");
  if (g->top_n < 0 || g->top_n > ARCS_KCAP) return set_error(ARCS_ERR_TOPK, "logprobs_batch: top_n must be 0 .. ARCS_KCAP");
  if (g->top_n > 0 && (!g->top_id || !g->top_logprob || g->top_stride < g->top_n))
    return set_error(ARCS_ERR_ARG, "logprobs_batch: top_n given without top_id / top_logprob of at least top_n entries per row");
  if (g->token && !g->logprob) return set_error(ARCS_ERR_ARG, "logprobs_batch: token given without logprob");
  LogprobDev a;
  a.logits = g->logits;
  a.row_stride = g->row_stride;
  a.B = g->B;
  a.V = g->V;
  a.token = g->token;
  a.top_n = g->top_n;
  a.top_stride = g->top_stride;
  a.logprob = g->logprob;
  a.lse = g->lse;
  a.top_id = g->top_id;
  a.top_logprob = g->top_logprob;
  a.status = g->status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define ARCS_LAUNCH(T)                                                                                               \
  do {                                                                                                               \
    cudaError_t e = cudaFuncSetAttribute(logprob_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLpSmem); \
    if (e != cudaSuccess) return set_error(ARCS_ERR_CUDA, cudaGetErrorString(e));                                    \
    logprob_kernel<T><<<(unsigned)g->B, kThreads, kLpSmem, st>>>(a);                                                 \
  } while (0)
  if (g->dtype == ARCS_F32) ARCS_LAUNCH(float);
  else ARCS_LAUNCH(__nv_bfloat16);
#undef ARCS_LAUNCH
  return check_launch("logprobs_batch");
}
