// logprobs_batch: per row the log-softmax of one token and the top_n largest raw logits as log
// probabilities (tools/server_chat.h:417-441; zero/runz.cpp:478-484 scores perplexity with the
// same sum). One launch. A CTA streams one segment of one row once through a ring of bulk-copied
// tiles and keeps
//  - per thread a running (reference value, sum of exponentials relative to it), the sum in fp64;
//  - for the whole CTA a candidate buffer with a rising threshold: the top_n best so far.
// Rows are cut into segments when there are few of them; the CTA that finishes a row last merges
// the segments' results (left in the workspace) and writes the row's output.
#include "plan.h"
#include "select.cuh"
#include "stream.cuh"

namespace arcs {

constexpr int kLpCap = 1024;                  // candidate buffer of a CTA
constexpr int kLpTrig = kLpCap - kThreads;    // prune once it has grown past this
constexpr int kLpPerSm = 3;                   // CTAs per SM the segments are planned for

struct LpPart {      // what a segment leaves for the merge
  double z;          // sum of exp(l - M) over the segment
  float M;           // the segment's maximum (-inf: nothing but NaN or -inf)
  int32_t cnt;       // entries in its candidate list
};

struct LogprobDev {
  const void* logits;
  int64_t row_stride;
  int32_t B, V, nseg, seg_len;
  const int32_t* token;
  int32_t top_n, top_stride;
  double* logprob;
  double* lse;
  int32_t* top_id;
  double* top_logprob;
  unsigned int* ws_ctr;            // [B] segments of the row that have finished, 0 between launches
  LpPart* ws_part;                 // [B][nseg]
  unsigned long long* ws_list;     // [B][nseg][top_n] composites
  int32_t* status;
};

// exp(v - m) for v <= m as 2^((v - m) * log2 e) by the special-function unit. Measured against
// fp64 sums the log of a row's sum comes out within 4e-8 whatever is done about the roundings of
// the difference and of the product (first-order corrections were tried: the unit's own error
// dominates), so nothing is. NaN and -inf give 0.
__device__ __forceinline__ float exp_diff(float v, float m) {
  constexpr float kL2e = 1.44269502162933349609375f;
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(__fmul_rn(__fsub_rn(fmaxf(v, -1e38f), m), kL2e)));
  return e;
}

// Warp-collective append to the candidate buffer; lanes with p set store (key, id). Returns true
// for a lane whose entry found no room (the caller offers it again after the next prune); `hot`
// is set once the buffer has grown past the prune trigger.
__device__ __forceinline__ bool lp_push(const Sel& s, bool p, uint32_t key, int32_t id, bool& hot) {
  const unsigned b = __ballot_sync(0xFFFFFFFFu, p);
  if (b == 0) return false;
  const int lane = threadIdx.x & 31, leader = __ffs(b) - 1;
  int base = 0;
  if (lane == leader) base = (int)sm_atomic_add(s.cnt, (uint32_t)__popc(b));
  base = __shfl_sync(0xFFFFFFFFu, base, leader);
  if (!p) return false;
  const int pos = base + __popc(b & ((1u << lane) - 1u));
  hot = hot || pos + 1 > s.trig;
  if (pos >= s.cap) return true;
  s.key[pos] = key;
  s.id[pos] = id;
  return false;
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
  __shared__ int s_cnt, s_misc[8], s_flag;
  __shared__ uint32_t s_maxkey;
  __shared__ float red_m[kThreads / 32];
  __shared__ double red_s[kThreads / 32], s_lse;
  __shared__ __align__(16) uint32_t s_keys[kThreads];

  constexpr int E = Elem<T>::kPerChunk;
  constexpr int kChunks = kTileBytes / 16 / kThreads;
  static_assert(kChunks * E <= 32, "a thread's elements of one tile are tracked in a 32-bit mask");
  const int tid = threadIdx.x, b = blockIdx.x / a.nseg, seg = blockIdx.x % a.nseg;
  const T* row = reinterpret_cast<const T*>(a.logits) + (size_t)b * a.row_stride;
  const int32_t lo = seg * a.seg_len, hi = min(a.V, lo + a.seg_len);
  const SegPlan p = make_plan(row, lo, hi);
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
  float own = -INFINITY;  // the largest value this thread itself has seen
  unsigned long long tau = 0ull;  // exclusive threshold of the candidate buffer (every thread's copy is current)

  // one more value for the sum
  auto lse_one = [&](float v) {
    own = fmaxf(own, v);
    if (v > lm) {
      ls *= exp((double)lm - (double)v);
      lm = v;
    }
    if (lm > -INFINITY) ls += (double)exp_diff(v, lm);
  };
  // All threads call. The threads' own maxima belong to disjoint sets of elements, so the n-th
  // largest of them is a lower bound of the n-th largest element: the threshold rises to it
  // without a look at the buffer (16-bit key resolution, one warp). The largest of them becomes
  // every thread's reference for its exponentials: a thread then meets a larger value, and pays
  // for the fp64 rescaling of its sum, only where the CTA as a whole does.
  auto share_maxima = [&](bool reference) {
    __syncthreads();  // (s_keys may still be read from the last time)
    s_keys[tid] = own > -INFINITY ? key_of(own) : 0u;
    __syncthreads();
    if (tid < 32) {
      uint32_t mk = 0;
#pragma unroll
      for (int i = 0; i < kThreads / 32; ++i) mk = max(mk, s_keys[i * 32 + tid]);
      mk = __reduce_max_sync(0xFFFFFFFFu, mk);
      const uint32_t k = n > 0 ? warp_kth16<kThreads / 32>(s_keys, n) : 0u;
      const unsigned long long cand = k ? ((unsigned long long)k << 32) - 1ull : 0ull;
      if (tid == 0) {
        s_maxkey = mk;
        if (cand > s_tau) s_tau = cand;
      }
    }
    __syncthreads();
    tau = s_tau;
    if (reference && s_maxkey != 0u) {
      const float top = value_of(s_maxkey);
      if (top > lm) {
        ls *= exp((double)lm - (double)top);
        lm = top;
      }
    }
  };
  // A lane sets the (few) elements it finds above the threshold aside, two at most, and the warp
  // appends what its lanes hold to the buffer in one go, now and then: an append costs the warp
  // a round trip to a shared counter.
  uint32_t sk0 = 0, sk1 = 0;
  int32_t si0 = 0, si1 = 0;
  int ns = 0;
  bool hot = false;
  auto warp_flush = [&]() {
    const bool lost1 = lp_push(sel, ns == 2 && comp_of(sk1, si1) > tau, sk1, si1, hot);
    if (ns == 2 && !lost1) ns = 1;
    const bool lost0 = lp_push(sel, ns == 1 && comp_of(sk0, si0) > tau, sk0, si0, hot);
    if (ns == 1 && !lost0) ns = 0;
  };
  // Every thread calls with the mask of its own elements that may belong to the n best;
  // elem(idx, key, id) names element idx. `flush`: what the lanes hold goes to the buffer before
  // the call returns. When the buffer has grown past the trigger, or had no room for some entry,
  // the CTA keeps the n best, the threshold rises and what was left out is offered again.
  auto push_all = [&](uint32_t bits, bool flush, auto elem) {
    uint32_t again = 0;
    for (;;) {
      while (__any_sync(0xFFFFFFFFu, bits != 0u)) {
        if (__any_sync(0xFFFFFFFFu, bits != 0u && ns == 2)) warp_flush();
        if (bits != 0u) {
          const int idx = __ffs(bits) - 1;
          bits &= bits - 1u;
          if (ns < 2) {
            uint32_t ky = 0;
            int32_t id = 0;
            elem(idx, ky, id);
            if (ky != 0u && comp_of(ky, id) > tau) {
              if (ns == 0) {
                sk0 = ky;
                si0 = id;
              } else {
                sk1 = ky;
                si1 = id;
              }
              ++ns;
            }
          } else {
            again |= 1u << idx;  // (the buffer is full: after the prune)
          }
        }
      }
      if (flush) warp_flush();
      if (!__syncthreads_or(hot || again != 0u || (flush && ns > 0))) break;
      const unsigned long long before = tau;
      sel_prune<1, kThreads>(sel, n, ps, tid);
      if (s_tau < before) {  // (entries still held by lanes were not in the buffer: its n-th best may lie below the threshold)
        __syncthreads();
        if (tid == 0) s_tau = before;
        __syncthreads();
      }
      tau = s_tau;
      hot = false;
      bits = again;
      again = 0;
    }
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
    float cmax[kChunks];
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
      const uint32_t off = (uint32_t)(j * kThreads + tid) * 16u;
      cmax[j] = NAN;  // (a chunk past the end of the tile reaches no threshold, not even -inf)
      if (off >= nbytes) continue;
      const float cm = Elem<T>::chunk_max(q[j]);
      cmax[j] = cm;
      own = fmaxf(own, cm);
      if (cm > lm) {
        ls *= exp((double)lm - (double)cm);
        lm = cm;
      }
      if (lm > -INFINITY) {
        float ev[E];
#pragma unroll
        for (int e = 0; e < E; ++e) ev[e] = exp_diff(Elem<T>::get(q[j], e), lm);
#pragma unroll
        for (int w = E / 2; w > 0; w >>= 1)
#pragma unroll
          for (int e = 0; e < w; ++e) ev[e] += ev[e + w];
        ls += (double)ev[0];
      }
    }
    if (t == 0 || t == 3 || t == 15 || t == 63) share_maxima(true);
    if (n <= 0) continue;

    // ---- the candidates
    const int32_t tile_first = p.body_first + (int32_t)((uint32_t)t * kTileBytes / sizeof(T));
    const uint32_t tkey = (uint32_t)(tau >> 32);
    const float tf = value_of(tkey < 0x007FFFFFu ? 0x007FFFFFu : tkey);  // inclusive value threshold
    // the chunks whose maximum reaches the threshold are few: only they are looked into, in a
    // loop the warp leaves as soon as no lane has one; what passes is set aside by the lane
    uint32_t hotc = 0;
#pragma unroll
    for (int j = 0; j < kChunks; ++j) hotc |= (cmax[j] >= tf ? 1u : 0u) << j;
    uint32_t bits = 0;
    while (__any_sync(0xFFFFFFFFu, hotc != 0u)) {
      if (hotc != 0u) {
        const int j = __ffs(hotc) - 1;
        hotc &= hotc - 1u;
        uint4 c = q[0];
#pragma unroll
        for (int x = 1; x < kChunks; ++x)
          if (j == x) c = q[x];
        const int32_t id0 = tile_first + (int32_t)((uint32_t)(j * kThreads + tid) * 16u / sizeof(T));
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float v = Elem<T>::get(c, e);
          if (v >= tf) {
            const uint32_t ky = key_of(v);
            if (ky != 0u && comp_of(ky, id0 + e) > tau) {
              if (ns == 0) {
                sk0 = ky;
                si0 = id0 + e;
                ns = 1;
              } else if (ns == 1) {
                sk1 = ky;
                si1 = id0 + e;
                ns = 2;
              } else {
                bits |= 1u << (j * E + e);  // (no room in the lane: the general path below)
              }
            }
          }
        }
      }
    }
    push_all(bits, (t & 7) == 7 || t + 1 == p.tiles, [&](int idx, uint32_t& ky, int32_t& id) {
      const int j = idx / E;
      uint4 c = q[0];
#pragma unroll
      for (int x = 1; x < kChunks; ++x)
        if (j == x) c = q[x];
      id = tile_first + (int32_t)((uint32_t)(j * kThreads + tid) * 16u / sizeof(T)) + idx % E;
      ky = key_of(Elem<T>::get(c, idx % E));
    });
  }

  // ---- the few elements outside the 16-byte aligned body
  {
    const bool hv = tid < p.head_n, tv = tid < p.tail_n;
    const float vh = hv ? Elem<T>::load(row + lo + tid) : 0.0f;
    const float vt = tv ? Elem<T>::load(row + p.tail_first + tid) : 0.0f;
    if (hv) lse_one(vh);
    if (tv) lse_one(vt);
    if (n > 0)
      push_all((hv ? 1u : 0u) | (tv ? 2u : 0u), true, [&](int idx, uint32_t& ky, int32_t& id) {
        ky = key_of(idx == 0 ? vh : vt);
        id = idx == 0 ? lo + tid : p.tail_first + tid;
      });
  }

  // the CTA's (maximum, sum of exponentials relative to it) from the threads' pairs; the sum is
  // returned to thread 0
  auto cta_lse = [&](float m_t, double s_t, float& M) -> double {
    M = m_t;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, o));
    __syncthreads();  // (red_m / red_s may still be read from an earlier call)
    if ((tid & 31) == 0) red_m[tid >> 5] = M;
    __syncthreads();
    M = red_m[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) M = fmaxf(M, red_m[w]);
    double part = m_t > -INFINITY ? s_t * exp((double)m_t - (double)M) : 0.0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xFFFFFFFFu, part, o);
    if ((tid & 31) == 0) red_s[tid >> 5] = part;
    __syncthreads();
    double z = 0.0;
    if (tid == 0)
      for (int w = 0; w < kThreads / 32; ++w) z += red_s[w];
    return z;
  };
  float M;
  double z = cta_lse(lm, ls, M);
  // What is left of the buffer once a last threshold (from the threads' own maxima, where the
  // buffer holds this CTA's own elements) has been applied: a little more than n entries as a
  // rule. Where the n best are needed, an entry's place is the number of entries above it
  // (composites are unique).
  auto settle = [&](bool own_elements) -> int {
    if (own_elements) share_maxima(false);
    else __syncthreads();
    const int c0 = min(s_cnt, kLpCap);
    unsigned long long mine[kLpCap / kThreads];
#pragma unroll
    for (int x = 0; x < kLpCap / kThreads; ++x) {
      const int i = tid + x * kThreads;
      mine[x] = i < c0 ? comp_of(bkey[i], bid[i]) : 0ull;
    }
    __syncthreads();
    if (tid == 0) s_cnt = 0;
    __syncthreads();
    bool hot = false;
#pragma unroll
    for (int x = 0; x < kLpCap / kThreads; ++x) lp_push(sel, mine[x] > tau, comp_key(mine[x]), comp_id(mine[x]), hot);
    __syncthreads();
    if (s_cnt > 512) {
      sel_prune<1, kThreads>(sel, n, ps, tid);
      __syncthreads();
    }
    return min(s_cnt, kLpCap);
  };
  auto rank_of = [&](int i, int c) -> int {
    const uint64_t ci = comp_of(bkey[i], bid[i]);
    int rank = 0;
    for (int j = 0; j < c; ++j) rank += comp_of(bkey[j], bid[j]) > ci;
    return rank;
  };

  if (a.nseg > 1) {
    // ---- leave the segment's results; the CTA that finishes the row last merges them
    const size_t slot = (size_t)b * a.nseg + seg;
    const int c = n > 0 ? settle(true) : 0, m = min(c, n);
    for (int i = tid; i < c; i += kThreads) {
      const int rank = rank_of(i, c);
      if (rank < n) a.ws_list[slot * n + rank] = comp_of(bkey[i], bid[i]);
    }
    if (tid == 0) {
      LpPart pt;
      pt.z = z;
      pt.M = M;
      pt.cnt = m;
      a.ws_part[slot] = pt;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      s_flag = atomicAdd(&a.ws_ctr[b], 1u) == (unsigned)a.nseg - 1u;
      if (s_flag) a.ws_ctr[b] = 0u;  // left at zero for the next launch
    }
    __syncthreads();
    if (!s_flag) return;
    __threadfence();
    float pm = -INFINITY;
    double pz = 0.0;
    int pc = 0;
    if (tid < a.nseg) {
      const LpPart* src = &a.ws_part[(size_t)b * a.nseg + tid];
      pz = __ldcg(&src->z);
      pm = __ldcg(&src->M);
      pc = __ldcg(&src->cnt);
    }
    z = cta_lse(pm, pz, M);
    if (n > 0) {
      if (tid == 0) {
        s_cnt = 0;
        s_tau = 0ull;
      }
      __syncthreads();
      tau = 0ull;
      // the segments' lists go through the buffer, kThreads entries at a time
      __shared__ int s_cnts[kMaxSeg];
      if (tid < a.nseg) s_cnts[tid] = pc;
      __syncthreads();
      for (int e0 = 0; e0 < a.nseg * n; e0 += kThreads) {
        const int e = e0 + tid, g = e / n, i = e % n;
        const bool have = e < a.nseg * n && i < s_cnts[g];
        const unsigned long long c = have ? __ldcg(&a.ws_list[((size_t)b * a.nseg + g) * n + i]) : 0ull;
        push_all(have ? 1u : 0u, true, [&](int, uint32_t& ky, int32_t& id) {
          ky = comp_key(c);
          id = comp_id(c);
        });
      }
    }
  }

  // ---- the row's output
  if (tid == 0) {
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
  const int c = settle(a.nseg == 1);  // (its barriers also publish s_lse)
  const double lse = s_lse;
  for (int i = tid; i < c; i += kThreads) {
    const int rank = rank_of(i, c);
    if (rank < n) {
      a.top_id[(size_t)b * a.top_stride + rank] = bid[i];
      a.top_logprob[(size_t)b * a.top_stride + rank] = (double)value_of(bkey[i]) - lse;
    }
  }
}

}  // namespace arcs

using namespace arcs;

static void lp_plan(int32_t B, int32_t V, int* nseg, int* seg_len) { plan_segments(B, V, nseg, seg_len, kLpPerSm); }

extern "C" size_t arcs_logprobs_workspace_bytes(int32_t B, int32_t V, int32_t top_n) {
  if (B <= 0 || V <= 0 || top_n < 0) return 0;
  int nseg, seg_len;
  lp_plan(B, V, &nseg, &seg_len);
  if (nseg == 1) return 16;  // whole rows: nothing is handed over
  return 256 + (((size_t)B * 4 + 255) & ~(size_t)255) + (size_t)B * nseg * sizeof(LpPart) + (size_t)B * nseg * (size_t)top_n * 8;
}

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
  lp_plan(g->B, g->V, &a.nseg, &a.seg_len);
  a.token = g->token;
  a.top_n = g->top_n;
  a.top_stride = g->top_stride;
  a.logprob = g->logprob;
  a.lse = g->lse;
  a.top_id = g->top_id;
  a.top_logprob = g->top_logprob;
  a.status = g->status;
  a.ws_ctr = nullptr;
  a.ws_part = nullptr;
  a.ws_list = nullptr;
  if (a.nseg > 1) {
    if (!g->workspace || g->workspace_bytes < arcs_logprobs_workspace_bytes(g->B, g->V, g->top_n))
      return set_error(ARCS_ERR_WORKSPACE, "logprobs_batch: workspace too small");
    if ((reinterpret_cast<uintptr_t>(g->workspace) & 15u) != 0) return set_error(ARCS_ERR_WORKSPACE, "logprobs_batch: workspace must be 16-byte aligned");
    char* ws = static_cast<char*>(g->workspace);
    a.ws_ctr = reinterpret_cast<unsigned int*>(ws);
    ws += ((size_t)g->B * 4 + 255) & ~(size_t)255;
    a.ws_part = reinterpret_cast<LpPart*>(ws);
    ws += (size_t)g->B * a.nseg * sizeof(LpPart);
    a.ws_list = reinterpret_cast<unsigned long long*>(ws);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)g->B * (unsigned)a.nseg;
#define ARCS_LAUNCH(T)                                                                                               \
  do {                                                                                                               \
    static std::atomic<unsigned long long> attr_done{0};                                                   \
    cudaError_t e = ensure_dynamic_smem(logprob_kernel<T>, (int)kLpSmem, attr_done);                       \
    if (e != cudaSuccess) return set_error(ARCS_ERR_CUDA, cudaGetErrorString(e));                                    \
    logprob_kernel<T><<<grid, kThreads, kLpSmem, st>>>(a);                                                           \
  } while (0)
  if (g->dtype == ARCS_F32) ARCS_LAUNCH(float);
  else ARCS_LAUNCH(__nv_bfloat16);
#undef ARCS_LAUNCH
  return check_launch("logprobs_batch");
}
