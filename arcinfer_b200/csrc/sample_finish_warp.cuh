// finish_row_fast: the common case of the finish step, one warp per row (or, when the rows are
// few, one CTA per row).
//
// A row whose candidates fit a warp's hands - no allowed-token mask, at most 64 candidates kept,
// at most 256 survivors above the last threshold, at most 32 flagged entries, at most 32
// segments, no list of the stream overflowed - is finished without the CTA-wide selection: the
// survivors above the threshold are gathered, the flagged ones settled against the history and
// bias lists (tools/sampler.h:154-174), the rest ranked by counting, and tools/sampler.h:54-77
// followed to the letter (fp64 softmax in candidate order, min-p / top-p cuts, the draw). Any
// other row is left to the CTA-wide path of the finish kernel.
#pragma once
#include "sample_common.cuh"

namespace arcs {


constexpr int kFastK = 64;      // most candidates a row may keep on this path
constexpr int kFastBuf = 256;   // most survivors above the last threshold (one warp)
constexpr int kFastBufCta = 512;  // ... when the whole CTA works on the row
constexpr int kFastFlag = 32;   // most flagged entries
constexpr uint32_t kFlagWaitLimit = 1u << 21;  // bounded wait for an item's release (about a second)

__device__ __forceinline__ int32_t ld_acquire_gpu(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// exp(x) for a float x <= 0 (a softmax term), evaluated in fp64 and rounded to float: the value
// tools/sampler.h:60 stores, std::exp of a float argument. x = n ln 2 + r with |r| <= ln 2 / 2;
// e^r by a degree-11 Taylor polynomial (relative error below 2^-44, so the rounding to float
// differs from that of the exact value for about one argument in a million); times 2^n. Far
// fewer instructions than the general fp64 exponential, on a path where they are a row's latency.
__device__ __forceinline__ float exp_term(float xf) {
  if (!(xf > -104.0f)) return 0.0f;  // (below the smallest float denormal; also -inf)
  const double x = (double)xf;
  const double n = rint(x * 1.4426950408889634);
  const double r = fma(n, -6.93147180369123816490e-01, x);
  const double r2 = fma(n, -1.90821492927058770002e-10, r);
  double p = 2.50521083854417187751e-08;            // 1/11!
  p = fma(p, r2, 2.75573192239858906526e-07);       // 1/10!
  p = fma(p, r2, 2.75573192239858906526e-06);       // 1/9!
  p = fma(p, r2, 2.48015873015873015873e-05);       // 1/8!
  p = fma(p, r2, 1.98412698412698412698e-04);       // 1/7!
  p = fma(p, r2, 1.38888888888888888889e-03);       // 1/6!
  p = fma(p, r2, 8.33333333333333333333e-03);       // 1/5!
  p = fma(p, r2, 4.16666666666666666667e-02);       // 1/4!
  p = fma(p, r2, 1.66666666666666666667e-01);       // 1/3!
  p = fma(p, r2, 0.5);
  p = fma(p, r2, 1.0);
  p = fma(p, r2, 1.0);
  const int ni = (int)n;  // >= -151: the scaling is split so that neither factor underflows
  const int n1 = ni < -1000 ? -1000 : ni, n2 = ni - n1;
  double v = p * __longlong_as_double((long long)(1023 + n1) << 52);
  if (n2 != 0) v *= __longlong_as_double((long long)(1023 + n2) << 52);
  return (float)v;
}

// one warp's scratch (carved out of shared memory by the caller, 8-byte aligned)
template <int BUF>
struct FastScratchT {
  unsigned long long buf[BUF];  // composites of the survivors above the threshold; later the running sums
  float sv[kFastK];
  int32_t sid[kFastK];
  double spr[kFastK + 1];
  uint32_t fkey[kFastFlag];
  int32_t fid[kFastFlag];   // (global id | kOkB)
  int32_t loff[66];         // where each of the row's lists (two a segment) begins in the row's run of entries
  unsigned long long tau;   // the threshold the survivors must exceed
  int32_t rc, m, nf, spill, kB;
};
using FastScratch = FastScratchT<kFastBuf>;
using FastScratchCta = FastScratchT<kFastBufCta>;
static_assert(sizeof(FastScratch) <= 4096, "a warp's scratch fits one of the CTA-wide path's 4 KB arrays");

enum { kFastDone = 0, kFastSlow = 1, kFastLate = 2 };
template <int N>
struct IntTag {
  static constexpr int value = N;
};

// Vocabulary shards: the shards' (max, sum of exp(l - max)) pairs of row b combined by one warp:
// M = max m_g, Z = sum z_g exp(m_g - M).
__device__ __forceinline__ void combine_mz(const SampleDev& a, int b) {
  if (!a.mz_out || !a.merge_mz) return;
  const int lane = threadIdx.x & 31;
  float M = -INFINITY;
  for (int g = lane; g < a.merge_G; g += 32) M = fmaxf(M, __ldg(&a.merge_mz[((size_t)g * a.B + b) * a.merge_mz_stride]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, o));
  double Z = 0.0;
  for (int g = lane; g < a.merge_G; g += 32) {
    const float* mz = &a.merge_mz[((size_t)g * a.B + b) * a.merge_mz_stride];
    const float m = __ldg(&mz[0]), z = __ldg(&mz[1]);
    if (m > -INFINITY) Z += (double)z * exp((double)m - (double)M);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) Z += __shfl_xor_sync(0xFFFFFFFFu, Z, o);
  if (lane == 0) {
    a.mz_out[2 * (size_t)b] = M;
    a.mz_out[2 * (size_t)b + 1] = (float)Z;
  }
}

// NT threads finish row b: one warp (NT == 32, four rows to a CTA), or the whole CTA (NT == 128)
// when the rows are few, which are then cut into many segments with as many loose thresholds:
// the entries are read by all threads, the threshold is tightened from a count of the entries by
// the upper 16 bits of their keys (bins: 256 counters, NT == 128 only) before the survivors are
// kept, and the survivors are ranked by all threads. What one warp can do (settings, headers,
// flagged entries, softmax, cuts, draw) the first warp does. Every thread returns the same code
// up to the last barrier.
template <typename T, int NT>
__device__ __noinline__ int finish_row_fast(const SampleDev& a, int b, FastScratchT<(NT == 128 ? kFastBufCta : kFastBuf)>& fs, uint32_t* bins) {
  constexpr int kBuf = NT == 128 ? kFastBufCta : kFastBuf;
  static_assert(NT == 32 || NT == 128, "one warp or the CTA");
  const int lane = threadIdx.x & 31;
  const int tid = NT == 32 ? lane : (int)threadIdx.x;
  const bool lead = NT == 32 || threadIdx.x < 32;
  const bool merging = a.merge_G > 0;
  auto bar = [&]() {
    if (NT == 32) __syncwarp();
    else __syncthreads();
  };
  // ---- the row's settings and, if it is short, its history: fetched before the row's items are
  // waited for (a CTA of the last rows sits here while the stream kernel runs)
  RowCfg r;
  constexpr int HR = 16;
  int32_t hreg[HR];
  bool hist_in_regs = false, bans = false;
  if (lead) {
    r = row_cfg<false>(a, b);
    hist_in_regs = r.pen_on && r.lists_ok && r.H <= 32 * HR;
#pragma unroll
    for (int x = 0; x < HR; ++x) hreg[x] = hist_in_regs && x * 32 + lane < r.H ? __ldg(&a.hist_ids[r.h0 + x * 32 + lane]) : -1;
    // ---- the row's items: released by the stream kernel (bounded wait), their headers
    unsigned long long tau = 0ull;
    bool over = false, late = false;
    int c0 = 0, c1 = 0;  // (lane g: the list lengths of segment g, for rows of at most 32 segments)
    if (merging) {
      // Vocabulary shards: the row's lists are the shards' candidates, each best first. A shard
      // that sent k entries has k at or above its k-th: nothing below the largest such entry can
      // be among the k best of all.
      combine_mz(a, b);
      for (int i = lane; i < r.NB; i += 32) bans = bans || __ldg(&a.bias_vals[r.q0 + i]) <= ARCS_BANNED;
      const int kth = r.kB - 1;
      if (lane < a.merge_G && kth >= 0 && kth < a.merge_width) {
        const size_t row = ((size_t)lane * a.B + b) * a.merge_stride;
        const int32_t id = (!a.merge_n || kth < __ldg(&a.merge_n[(size_t)lane * a.B + b])) ? __ldg(&a.merge_id[row + kth]) : -1;
        const uint32_t ky = key_of(__ldg(&a.merge_val[row + kth]));
        if (id >= 0 && ky != 0u) tau = comp_of(ky, id) - 1ull;  // (composites are unique: "above tau" keeps the k-th itself)
      }
    }
    for (int g = lane; g < a.nseg && !merging; g += 32) {
      const ItemHdr* hd = item_ws(a, b * a.nseg + g).hdr;
      uint32_t spins = 0;
      while (ld_acquire_gpu(&hd->streamed) == 0) {
        if (++spins > kFlagWaitLimit) {
          late = true;
          break;
        }
        __nanosleep(spins < 64 ? 100 : 400);
      }
      const int n0 = __ldcg(&hd->n_pre), nt = __ldcg(&hd->n_tch), n1 = __ldcg(&hd->n_candB);
      over = over || n1 > kListB || nt > item_pre_cap(a.hash_slots) - n0;
      bans = bans || __ldcg(&hd->bans) != 0;
      const unsigned long long t = __ldcg(&hd->tauB);
      tau = t > tau ? t : tau;
      c0 = n0 + nt;
      c1 = n1;
    }
    __syncwarp();  // (the lanes that waited have acquired the items' lists for the whole warp)
    int rc = kFastDone;
    if (r.kB > kFastK || a.nseg > 32 || a.merge_G > 32) rc = kFastSlow;
    else if (__any_sync(0xFFFFFFFFu, late)) rc = kFastLate;
    else if (__any_sync(0xFFFFFFFFu, over)) rc = kFastSlow;
    tau = warp_max_u64(tau);
    bans = __any_sync(0xFFFFFFFFu, bans);
    // The row's lists (two a segment: what the preparing warps supplied with the flagged entries
    // behind it, and the scanners' survivors) are read as one run of entries: where each begins
    if (a.nseg > 32) c0 = c1 = 0;
    int inc = c0 + c1;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(0xFFFFFFFFu, inc, d);
      if (lane >= d) inc += t;
    }
    if (lane < a.nseg) {
      fs.loff[2 * lane] = inc - c0 - c1;
      fs.loff[2 * lane + 1] = inc - c1;
    }
    if (lane == 31) fs.loff[2 * min(a.nseg, 32)] = inc;
    if (lane == 0) {
      fs.rc = rc;
      fs.tau = tau;
      fs.m = 0;
      fs.nf = 0;
      fs.spill = 0;
      fs.kB = r.kB;
    }
  }
  bar();
  if (fs.rc != kFastDone) return fs.rc;
  const int nl = 2 * a.nseg, total = merging ? a.merge_G * a.merge_width : fs.loff[nl];
  // entry f of the run. A thread's entries come in rising order: the list it stands in (its
  // entries as if the run began at base[0]) is kept from one entry to the next.
  struct Cursor {
    const unsigned long long* base = nullptr;
    int end = 0, lst = -1;
  };
  auto entry = [&](int f, Cursor& c) -> unsigned long long {
    if (merging) {  // entry i of shard g's list, in the lists' own form
      const int g = f / a.merge_width, i = f - g * a.merge_width;
      const size_t row = (size_t)g * a.B + b;
      if (a.merge_n && i >= __ldg(&a.merge_n[row])) return 0ull;
      const int32_t id = __ldg(&a.merge_id[row * a.merge_stride + i]);
      const uint32_t ky = key_of(__ldg(&a.merge_val[row * a.merge_stride + i]));
      if (id < 0 || ky == 0u) return 0ull;
      return (unsigned long long)ky | ((unsigned long long)((uint32_t)id | kOkB) << 32);
    }
    while (f >= c.end) {  // (f < total == loff[nl]: the walk ends inside the table)
      ++c.lst;
      c.end = fs.loff[c.lst + 1];
      const ItemWs w = item_ws(a, b * a.nseg + (c.lst >> 1));
      c.base = ((c.lst & 1) ? w.candB : w.pre) - fs.loff[c.lst];
    }
    return __ldcg(c.base + f);
  };
  constexpr int R = 8;  // entries a thread fetches together: one trip to memory for R * NT entries
  // ---- many entries (NT == 128): a tighter threshold first, read off the counts of the entries by
  // the upper 16 bits of their keys, as the stream kernel does for its own (flagged entries count
  // for nothing: what they are worth is not known yet)
  if (NT == 128 && total > kBuf) {
    for (int i = tid; i < 256; i += NT) bins[i] = 0u;
    bar();
    const unsigned long long tau0 = fs.tau;
    const uint32_t base = (uint32_t)(tau0 >> 48);
    Cursor lst;
    for (int i0 = 0; i0 < total; i0 += R * NT) {
      unsigned long long e[R];
#pragma unroll
      for (int x = 0; x < R; ++x) {
        const int f = i0 + x * NT + tid;
        e[x] = f < total ? entry(f, lst) : 0ull;
      }
#pragma unroll
      for (int x = 0; x < R; ++x) {
        const uint32_t ky = (uint32_t)e[x], y = (uint32_t)(e[x] >> 32);
        if (i0 + x * NT + tid < total && !(y & kTch) && (y & kOkB) && comp_of(ky, (int32_t)(y & kIdMask)) > tau0)
          sm_red_add(&bins[min((ky >> 16) - base, 255u)], 1u);
      }
    }
    bar();
    if (lead) {
      int d, kr;
      bool ex;
      find_bin(bins, fs.kB, d, kr, ex);
      if (d > 0 && lane == 0) {
        const unsigned long long t = (unsigned long long)((base + (uint32_t)d) << 16) << 32;
        if (t > fs.tau) fs.tau = t;
      }
    }
    bar();
  }
  // ---- gather: survivors above the threshold to the buffer, flagged entries to their stage (in
  // any order: the ranking below does not depend on it)
  {
    const unsigned long long tau = fs.tau;
    Cursor lst;
    int m_w = 0, nf_w = 0;
    for (int i0 = 0; i0 < total; i0 += R * NT) {
      unsigned long long e[R];
#pragma unroll
      for (int x = 0; x < R; ++x) {
        const int f = i0 + x * NT + tid;
        e[x] = f < total ? entry(f, lst) : 0ull;
      }
#pragma unroll
      for (int x = 0; x < R; ++x) {
        if (i0 + x * NT >= total) break;
        const bool p = i0 + x * NT + tid < total;
        const uint32_t ky = (uint32_t)e[x], y = (uint32_t)(e[x] >> 32);
        const int32_t id = (int32_t)(y & kIdMask);
        const bool fl = p && (y & kTch);
        const uint64_t cm = comp_of(ky, id);
        const bool keep = p && !fl && (y & kOkB) && cm > tau;
        const unsigned bk = __ballot_sync(0xFFFFFFFFu, keep), bf = __ballot_sync(0xFFFFFFFFu, fl);
        // (one warp counts in registers; the warps of a CTA draw their places from the shared counters)
        int atk = m_w + __popc(bk & ((1u << lane) - 1u)), atf = nf_w + __popc(bf & ((1u << lane) - 1u));
        if (NT != 32) {
          const int lk = __ffs(bk) - 1, lf = __ffs(bf) - 1;
          int bk0 = 0, bf0 = 0;
          if (bk && lane == lk) bk0 = (int)sm_atomic_add(&fs.m, (uint32_t)__popc(bk));
          if (bf && lane == lf) bf0 = (int)sm_atomic_add(&fs.nf, (uint32_t)__popc(bf));
          if (bk) atk += __shfl_sync(0xFFFFFFFFu, bk0, lk);
          if (bf) atf += __shfl_sync(0xFFFFFFFFu, bf0, lf);
        } else {
          m_w += __popc(bk);
          nf_w += __popc(bf);
        }
        if (keep) {
          if (atk < kBuf) fs.buf[atk] = cm;
          else fs.spill = 1;
        }
        if (fl) {
          if (atf < kFastFlag) {
            fs.fkey[atf] = ky;
            fs.fid[atf] = (int32_t)(y & (kIdMask | kOkB));
          } else {
            fs.spill = 1;
          }
        }
      }
    }
    if (NT == 32 && lane == 0) {
      fs.m = m_w;
      fs.nf = nf_w;
    }
  }
  bar();
  if (fs.spill) return kFastSlow;
  // ---- settle the flagged entries (tools/sampler.h:154-174 for them): one in the bias list was
  // evaluated by the preparing warps and is dropped here; one in the history is dropped too when
  // they evaluated the history (table mode), else penalised here; one the filter flagged by
  // accident is an ordinary element.
  if (fs.nf > 0) {
    if (lead) {
      const unsigned long long tau = fs.tau;
      const int nf = fs.nf;
      int m = fs.m;
      const int32_t w0 = window_start(r);
      for (int f = 0; f < nf; ++f) {
        const int32_t idf = fs.fid[f] & (int32_t)kIdMask;
        int cnt = 0;
        bool win = false, inbias = false;
        for (int i = lane; i < r.NB; i += 32) inbias = inbias || a.bias_ids[r.q0 + i] == idf;
        if (r.pen_on) {
          if (hist_in_regs) {
#pragma unroll
            for (int x = 0; x < HR; ++x)
              if (hreg[x] == idf) {
                ++cnt;
                win = win || x * 32 + lane >= w0;
              }
          } else {
            for (int i = lane; i < r.H; i += 32)
              if (__ldg(&a.hist_ids[r.h0 + i]) == idf) {
                ++cnt;
                win = win || i >= w0;
              }
          }
        }
        cnt = (int)__reduce_add_sync(0xFFFFFFFFu, (unsigned)cnt);
        win = __any_sync(0xFFFFFFFFu, win);
        inbias = __any_sync(0xFFFFFFFFu, inbias);
        uint32_t ky = fs.fkey[f];
        bool p = !inbias && (fs.fid[f] & (int32_t)kOkB) != 0;
        if (p && cnt > 0) {
          if (r.touch == kTouchTable) {
            p = false;
          } else {
            ky = key_of(penalise(r, value_of(ky), (uint32_t)cnt, w0 == 0 || win));
            p = ky != 0u;
          }
        }
        const uint64_t cm = comp_of(ky, idf);
        p = p && cm > tau;
        if (p) {  // (warp-uniform: every lane computed the same)
          if (m >= kBuf) {
            if (lane == 0) fs.spill = 1;
            break;
          }
          if (lane == 0) fs.buf[m] = cm;
          ++m;
        }
      }
      if (lane == 0) fs.m = m;
    }
    bar();
    if (fs.spill) return kFastSlow;
  }
  // ---- candidates best first: ranked by counting (composites are unique)
  const int m = fs.m;
  const int nB = min(m, fs.kB);
  auto rank_all = [&](auto per_tag) {
    constexpr int PER = decltype(per_tag)::value;
    unsigned long long mine[PER];
    int rank[PER];
#pragma unroll
    for (int x = 0; x < PER; ++x) {
      mine[x] = x * NT + tid < m ? fs.buf[x * NT + tid] : 0ull;
      rank[x] = 0;
    }
#pragma unroll 4
    for (int i = 0; i < m; ++i) {
      const unsigned long long c = fs.buf[i];
#pragma unroll
      for (int x = 0; x < PER; ++x) rank[x] += c > mine[x];
    }
#pragma unroll
    for (int x = 0; x < PER; ++x)
      if (x * NT + tid < m && rank[x] < nB) {
        fs.sv[rank[x]] = value_of(comp_key(mine[x]));
        fs.sid[rank[x]] = comp_id(mine[x]);
      }
  };
  if (NT == 128) rank_all(IntTag<kFastBufCta / 128>{});
  else if (m <= 64) rank_all(IntTag<2>{});
  else if (m <= 128) rank_all(IntTag<4>{});
  else rank_all(IntTag<kFastBuf / 32>{});
  bar();
  if (!lead) return kFastDone;  // (the rest is one warp's work)
  // ---- tools/sampler.h:54-77
  int nc = nB;
  if (bans)  // :54-55 (every lane walks the same few steps)
    while (nc > 1 && fs.sv[nc - 1] <= ARCS_BANNED) --nc;
  bool tie = false;  // equal logits among the candidates kept: the reference's order there is not defined
  for (int i = lane; i + 1 < nc; i += 32) tie = tie || fs.sv[i] == fs.sv[i + 1];
  const int flags = __any_sync(0xFFFFFFFFu, tie) ? ARCS_FLAG_TIE_TOPK : 0;
  const bool draw = !r.greedy && nc >= 1;
  int token = nc > 0 ? fs.sid[0] : -1, n = nc > 0 ? 1 : 0;
  double* cum = reinterpret_cast<double*>(fs.buf);  // (the buffer is no longer needed)
  if (draw) {
    const float mx = fs.sv[0];
    for (int i = lane; i < nc; i += 32) {
      const float x = __fdiv_rn(__fsub_rn(fs.sv[i], mx), r.prm.temperature);  // :60 float arithmetic
      fs.spr[i] = (double)exp_term(x);                                        // float exp, widened
    }
    __syncwarp();
    double z = 0.0;  // :58-60 in candidate order (every lane adds the same chain)
#pragma unroll 8
    for (int i = 0; i < nc; ++i) z = __dadd_rn(z, fs.spr[i]);
    __syncwarp();
    for (int i = lane; i < nc; i += 32) fs.spr[i] = __ddiv_rn(fs.spr[i], z);  // :64, the same quotients in any order
    __syncwarp();
    // :65-72. The running sums are a chain of roundings in candidate order; where the chain is
    // cut is then found by all lanes.
    if (lane == 0) {
      double c = 0.0;
#pragma unroll 8
      for (int i = 0; i < nc; ++i) {
        c = __dadd_rn(c, fs.spr[i]);
        cum[i] = c;
      }
    }
    __syncwarp();
    const double mp = __dmul_rn((double)r.prm.min_p, fs.spr[0]);
    int n_i = nc;
    for (int i = lane; i < nc; i += 32) {
      int c = 0x7FFFFFFF;
      if (r.prm.min_p > 0.0f && fs.spr[i] < mp) c = max(1, i);   // :65 (tested before the candidate is added)
      else if (cum[i] >= (double)r.prm.top_p) c = i + 1;         // :67
      n_i = min(n_i, c);
    }
    n = (int)__reduce_min_sync(0xFFFFFFFFu, (unsigned)n_i);
    if (lane == 0) {
      const double tot = cum[n - 1];             // the same sum, in the same order, as :70
      double rr = __dmul_rn(a.u[b], tot);        // :71-72
      int pick = -1;
      for (int i = 0; i < n && pick < 0; i += 4) {  // (four steps of the chain at a time: the loads run ahead of it)
        const double p0 = fs.spr[i], p1 = i + 1 < n ? fs.spr[i + 1] : 0.0, p2 = i + 2 < n ? fs.spr[i + 2] : 0.0, p3 = i + 3 < n ? fs.spr[i + 3] : 0.0;
        const double r0 = __dsub_rn(rr, p0), r1 = __dsub_rn(r0, p1), r2 = __dsub_rn(r1, p2), r3 = __dsub_rn(r2, p3);
        if (r0 <= 0.0) pick = i;
        else if (i + 1 < n && r1 <= 0.0) pick = i + 1;
        else if (i + 2 < n && r2 <= 0.0) pick = i + 2;
        else if (i + 3 < n && r3 <= 0.0) pick = i + 3;
        rr = r3;
      }
      if (pick < 0) pick = n - 1;
      token = fs.sid[pick];
    }
  }
  if (lane == 0) {
    if (r.k_bad || !r.lists_ok) token = -1;
    a.token[b] = token;
    if (a.n_cand) a.n_cand[b] = nc;
    if (a.n_kept) a.n_kept[b] = n;
    if (a.flags) a.flags[b] = flags;
  }
  if (a.cand_id || a.cand_val || a.cand_pr) {
    if (lane == 0 && nc > a.cand_width) raise_status(a.status, ARCS_ERR_TOPK);
    for (int i = lane; i < a.cand_width; i += 32) {
      const size_t o = (size_t)b * a.cand_stride + i;
      const bool in = i < nc;
      if (a.cand_id) a.cand_id[o] = in ? fs.sid[i] : -1;
      if (a.cand_val) a.cand_val[o] = in ? fs.sv[i] : 0.0f;
      if (a.cand_pr) a.cand_pr[o] = in ? (draw ? (float)fs.spr[i] : (i == 0 ? 1.0f : 0.0f)) : 0.0f;
    }
  }
  return kFastDone;
}

}  // namespace arcs
