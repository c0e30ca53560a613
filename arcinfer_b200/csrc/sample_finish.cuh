// finish_kernel: from an item's survivors to the row's token.
//
// One CTA of kGroup threads per row. It merges what the prepare kernel supplied (touched tokens
// with their adjusted logits, elements outside the aligned body) with what the stream kernel
// kept, for every segment of the row, selects the k best under (value desc, id asc), and then
// follows tools/sampler.h:54-77 (or :105-143 with an allowed-token mask) to the letter: fp64
// softmax in candidate order, min-p / top-p cuts, the draw.
#pragma once
#include "sample_common.cuh"

namespace arcs {

constexpr int kSortCap = 160;  // a longer buffer is cut to the k best by the radix select before it is ranked by counting

template <typename T, bool MASKED>
__global__ void __launch_bounds__(kGroup) finish_kernel(const SampleDev a) {
  __shared__ unsigned long long s64[8];
  __shared__ double spr[ARCS_KCAP + 1];
  __shared__ __align__(8) uint32_t bkey[kCapB];
  __shared__ int32_t bid[kCapB];
  __shared__ uint32_t akey[MASKED ? kCapA : 1];
  __shared__ int32_t aid[MASKED ? kCapA : 1];
  __shared__ uint32_t hist[512];
  __shared__ uint32_t tk[kTmpCap];
  __shared__ int32_t ti[kTmpCap];
  __shared__ float sv[ARCS_KCAP];
  __shared__ int32_t sid[ARCS_KCAP];
  __shared__ int misc[8];
  __shared__ int sh[8];
  __shared__ int seg_n[3][kMaxSeg];
  enum { L_TAU_B = 0, L_TAU_A, L_PRUNE_MIN, L_TOP, L_LOW };
  enum { S_CNT_B = 0, S_CNT_A, S_FLAGS, S_NCAND, S_BANS };

  const int gt = threadIdx.x;
  const int b = blockIdx.x;
  const int32_t Vg = a.v_global > 0 ? a.v_global : a.V;
  TR(8);
  const RowCfg r = row_cfg<MASKED>(a, b);
#ifdef ARCS_TRACE
  if (r.H > 100000) return;
#endif
  TR(9);
  const PruneScratch psF{hist, tk, ti, misc, &s64[L_PRUNE_MIN]};
  const Sel selB{bkey, bid, &sh[S_CNT_B], &s64[L_TAU_B], r.kB, kCapB - kGroup, kCapB};  // (pruned only when the buffer is nearly full)
  const Sel selA{akey, aid, &sh[S_CNT_A], &s64[L_TAU_A], ARCS_HEAD, 1024, kCapA};
  if (gt == 0) {
    sh[S_CNT_B] = 0;
    sh[S_CNT_A] = 0;
    sh[S_FLAGS] = 0;
    sh[S_BANS] = 0;
    s64[L_TAU_B] = 0ull;
    s64[L_TAU_A] = 0ull;
  }
  __syncthreads();

  bool hot = false;
  // called by the whole group after a barrier behind which nobody pushes
  auto maybe_prune = [&]() {
    const bool pb = *selB.cnt > selB.trig, pa = MASKED && *selA.cnt > selA.trig;
    group_sync<2>();
    if (pb) sel_prune<2>(selB, selB.k, psF, gt);
    if (pa) sel_prune<2>(selA, selA.k, psF, gt);
  };
  // one list of entries (key | word y << 32) into the selections, a round of kGroup at a time;
  // the entries of several rounds are fetched together
  auto take = [&](const unsigned long long* list, int n, bool toB, bool toA) {
    constexpr int R = 4;
    for (int i0 = 0; i0 < n; i0 += R * kGroup) {
      unsigned long long e[R];
#pragma unroll
      for (int x = 0; x < R; ++x) {
        const int i = i0 + x * kGroup + gt;
        e[x] = i < n ? __ldcg(&list[i]) : 0ull;
      }
#pragma unroll
      for (int x = 0; x < R; ++x) {
        if (i0 + x * kGroup >= n) break;
        const bool p = i0 + x * kGroup + gt < n;
        const uint32_t ky = (uint32_t)e[x], y = (uint32_t)(e[x] >> 32);
        const int32_t id = (int32_t)(y & kIdMask);
        const uint64_t cm = comp_of(ky, id);
        if (toB) sel_push(selB, p && (y & kOkB) && cm > *selB.tau, ky, id, hot, a.status);
        if (MASKED && toA) sel_push(selA, p && cm > *selA.tau, ky, id, hot, a.status);
        // at most kGroup pushes on top of a buffer at or below its trigger: inside its capacity
        if (group_sync_or<2>(hot)) {
          maybe_prune();
          hot = false;
        }
      }
    }
  };
  // what the segments' headers say, fetched together. Nothing at or below the largest threshold a
  // segment's stream ended on can be among the k best: that segment alone holds k above it.
  for (int g = gt; g < a.nseg; g += kGroup) {
    const ItemHdr* hd = item_ws(a, b * a.nseg + g).hdr;
    seg_n[0][g] = __ldcg(&hd->n_pre);
    seg_n[1][g] = __ldcg(&hd->n_candB);
    seg_n[2][g] = MASKED ? __ldcg(&hd->n_candA) : 0;
    if (__ldcg(&hd->bans) != 0) atomicOr(&sh[S_BANS], 1);
    atomicMax(&s64[L_TAU_B], __ldcg(&hd->tauB));
    if (MASKED) atomicMax(&s64[L_TAU_A], __ldcg(&hd->tauA));
  }
  __syncthreads();
  const bool bans = sh[S_BANS] != 0;
  for (int g = 0; g < a.nseg; ++g) {
    const ItemWs w = item_ws(a, b * a.nseg + g);
    take(w.pre, seg_n[0][g], true, true);
    take(w.candB, seg_n[1][g], true, false);
    if (MASKED) take(w.candA, seg_n[2][g], false, true);
  }
  group_sync<2>();
  TR(10);
  if (MASKED) sel_prune<2>(selA, selA.k, psF, gt);

  // ---- candidates best first. A short buffer is ranked by counting, which selects the k best
  // and sorts them in one step; a longer one is cut to the k best by the radix select first.
  const int sort_cap = max(kSortCap, selB.k + 64);
  if (*selB.cnt > sort_cap) sel_prune<2>(selB, selB.k, psF, gt);
  group_sync<2>();
  const int nbuf = min(*selB.cnt, sort_cap);
  const int nB = min(nbuf, selB.k);
  for (int i = gt; i < nbuf; i += kGroup) {
    const uint32_t ky = selB.key[i];
    const int32_t id = selB.id[i];
    const uint64_t c = comp_of(ky, id);
    int rank = 0;
    for (int x = 0; x < nbuf; ++x) rank += comp_of(selB.key[x], selB.id[x]) > c;
    if (rank < nB) {
      sv[rank] = value_of(ky);
      sid[rank] = id;
    }
  }
  if (gt == 0) {
    s64[L_TOP] = 0ull;                    // best composite among head entries that are not skipped as banned
    s64[L_LOW] = 0xFFFFFFFFFFFFFFFFull;   // smallest composite of the head
  }
  group_sync<2>();
  TR(11);
  // ---- tools/sampler.h:54-77 (or :105-143)
  int flags = 0, nc = nB;
  if (MASKED) {
    const int nA = min(*selA.cnt, ARCS_HEAD);
    for (int i = gt; i < nA; i += kGroup) {
      const uint64_t c = comp_of(selA.key[i], selA.id[i]);
      if (!(bans && value_of(selA.key[i]) <= ARCS_BANNED)) atomicMax(&s64[L_TOP], (unsigned long long)c);
      atomicMin(&s64[L_LOW], (unsigned long long)c);
    }
    group_sync<2>();
    if (gt == 0) {
      const uint64_t top = s64[L_TOP], low = s64[L_LOW];
      if (top != 0ull && (nB == 0 || comp_of(key_of(sv[0]), sid[0]) != top)) flags |= ARCS_FLAG_FIRST_REFUSED;
      if (Vg > ARCS_HEAD && nA == ARCS_HEAD) {  // the scan reaches rank 512 (tools/sampler.h:106-116)
        int nh = 0;
        while (nh < nB && comp_of(key_of(sv[nh]), sid[nh]) >= low) ++nh;
        if (nh < selB.k) {
          const float l512 = value_of(comp_key(low));
          if (!r.greedy && nh > 0 && __fdiv_rn(__fsub_rn(sv[0], l512), r.prm.temperature) > 20.0f) {  // :111
            nc = nh;
            flags |= ARCS_FLAG_TAIL_SKIPPED;
          } else {
            flags |= ARCS_FLAG_TAIL_USED;
          }
        }
      }
      sh[S_NCAND] = nc;
      sh[S_FLAGS] = flags;
    }
    group_sync<2>();
    nc = sh[S_NCAND];
  } else {
    if (gt == 0) {
      if (bans)  // tools/sampler.h:54-55
        while (nc > 1 && sv[nc - 1] <= ARCS_BANNED) --nc;
      sh[S_NCAND] = nc;
    }
    group_sync<2>();
    nc = sh[S_NCAND];
  }
  {  // equal logits among the candidates kept: the reference's order there is not defined
    bool tie = false;
    for (int i = gt; i + 1 < nc; i += kGroup) tie = tie || sv[i] == sv[i + 1];
    if (tie) atomicOr(&sh[S_FLAGS], ARCS_FLAG_TIE_TOPK);
  }
  TR(12);
  const bool draw = (!r.greedy && nc > 1) || (!MASKED && !r.greedy && nc == 1);
  if (draw) {
    const float mx = sv[0];
    for (int i = gt; i < nc; i += kGroup) {
      const float x = __fdiv_rn(__fsub_rn(sv[i], mx), r.prm.temperature);  // :60 float arithmetic
      spr[i] = (double)(float)exp((double)x);                              // float exp, widened
    }
    group_sync<2>();
    if (gt == 0) {
      double z = 0.0;
      for (int i = 0; i < nc; ++i) z = __dadd_rn(z, spr[i]);  // :58-60 in candidate order
      spr[ARCS_KCAP] = z;
    }
    group_sync<2>();
    const double z = spr[ARCS_KCAP];
    for (int i = gt; i < nc; i += kGroup) spr[i] = __ddiv_rn(spr[i], z);  // :64, the same quotients in any order
  }
  group_sync<2>();
  TR(13);
  // :65-72. The running sums are a chain of roundings in candidate order (one thread); where the
  // chain is cut is then found by all threads.
  double* cum = reinterpret_cast<double*>(bkey);  // (the buffer is no longer needed: 256 doubles fit)
  if (gt == 0) {
    sh[S_NCAND] = nc;  // n: candidates left after the cuts
    if (draw) {
      double c = 0.0;
      for (int i = 0; i < nc; ++i) {
        c = __dadd_rn(c, spr[i]);
        cum[i] = c;
      }
    }
  }
  group_sync<2>();
  if (draw) {
    const double mp = __dmul_rn((double)r.prm.min_p, spr[0]);
    for (int i = gt; i < nc; i += kGroup) {
      int n_i = 0x7FFFFFFF;
      if (r.prm.min_p > 0.0f && spr[i] < mp) n_i = max(1, i);   // :65 (tested before the candidate is added)
      else if (cum[i] >= (double)r.prm.top_p) n_i = i + 1;      // :67
      if (n_i != 0x7FFFFFFF) atomicMin(&sh[S_NCAND], n_i);
    }
  }
  group_sync<2>();
  if (gt == 0) {
    int token = nc > 0 ? sid[0] : -1, n = nc > 0 ? 1 : 0;
    if (draw) {
      n = sh[S_NCAND];
      const double tot = cum[n - 1];                                            // the same sum, in the same order, as :70
      double rr = __dmul_rn(a.u[b], tot);                                       // :71-72
      int pick = n - 1;
      for (int i = 0; i < n; ++i) {
        rr = __dsub_rn(rr, spr[i]);
        if (rr <= 0.0) { pick = i; break; }
      }
      token = sid[pick];
    }
    if (r.k_bad || !r.lists_ok) token = -1;
    a.token[b] = token;
    if (a.n_cand) a.n_cand[b] = nc;
    if (a.n_kept) a.n_kept[b] = n;
  }
  group_sync<2>();
  TR(14);
  if (gt == 0 && a.flags) a.flags[b] = sh[S_FLAGS];
  for (int i = gt; i < a.cand_stride && (a.cand_id || a.cand_val || a.cand_pr); i += kGroup) {
    const size_t o = (size_t)b * a.cand_stride + i;
    const bool in = i < nc;
    if (a.cand_id) a.cand_id[o] = in ? sid[i] : -1;
    if (a.cand_val) a.cand_val[o] = in ? sv[i] : 0.0f;
    if (a.cand_pr) a.cand_pr[o] = in ? (draw ? (float)spr[i] : (i == 0 ? 1.0f : 0.0f)) : 0.0f;
  }
}

}  // namespace arcs
