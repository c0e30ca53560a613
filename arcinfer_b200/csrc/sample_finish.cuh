// finish_kernel: from an item's survivors to the row's token.
//
// It runs beside the stream kernel: a row is taken when that kernel has released every item of
// it. The common case of a row is finished by one warp (sample_finish_warp.cuh), four rows to a
// CTA, or by all warps of a CTA together when the rows are few (a row is then cut into many
// segments, whose lists all have to be merged); what follows here is the general path, which all threads of the CTA walk together for a
// row the warp path left (an allowed-token mask, many candidates, lists that overflowed): it merges what the preparing warps supplied (touched
// tokens with their adjusted logits, elements outside the aligned body) with what the scanners
// kept, for every segment of the row, selects the k best under (value desc, id asc), and then
// follows tools/sampler.h:54-77 (or :105-143 with an allowed-token mask) to the letter: fp64
// softmax in candidate order, min-p / top-p cuts, the draw.
#pragma once
#include "sample_finish_warp.cuh"

namespace arcs {

constexpr int kStage = 1024;   // flagged entries settled together
constexpr int kSortCap = 160;  // a longer buffer is cut to the k best by the radix select before it is ranked by counting
template <typename T, bool MASKED, int G>
__global__ void __launch_bounds__(G, 5) finish_kernel(const SampleDev a) {  // (at most 96 registers: one CTA fits beside the stream kernel's)
  __shared__ unsigned long long s64[8];
  __shared__ double spr[ARCS_KCAP + 1];
  __shared__ __align__(16) uint32_t bkey[kCapB];
  __shared__ int32_t bid[kCapB];
  __shared__ uint32_t akey[MASKED ? kCapA : 1];
  __shared__ int32_t aid[MASKED ? kCapA : 1];
  __shared__ uint32_t hist[512];
  __shared__ uint32_t tk[kTmpCap];
  __shared__ int32_t ti[kTmpCap];
  __shared__ float sv[ARCS_KCAP];
  __shared__ int32_t sid[ARCS_KCAP];
  __shared__ int misc[8];
  __shared__ int sh[12];
  __shared__ int seg_n[4][kMaxSeg];  // per segment: entries of the prepare kernel (+ flagged ones of the stream), survivors B, A, overflowed
  __shared__ __align__(16) uint32_t fl_all[3 * kStage];  // (one array, so that the CTA-wide fast path can take it whole as its scratch)
  uint32_t* const fl_key = fl_all;                                              // hot elements the filter flagged, waiting to be settled
  int32_t* const fl_id = reinterpret_cast<int32_t*>(fl_all + kStage);            // (global id | kOkB)
  uint32_t* const fl_cnt = fl_all + 2 * kStage;                                 // occurrences in the history | in the repeat window << 31 | in the bias list << 30
  enum { L_TAU_B = 0, L_TAU_A, L_PRUNE_MIN, L_TOP, L_LOW };
  enum { S_CNT_B = 0, S_CNT_A, S_FLAGS, S_NCAND, S_BANS, S_NFLAG, S_NLIST, S_NLISTA, S_OVER, S_NPRE };

  const int gt = threadIdx.x;
  const int32_t Vg = a.v_global > 0 ? a.v_global : a.V;
  const bool merging = a.merge_G > 0;
  // ---- rows of this CTA: the warp path first, every warp its own row
  const int kRows = MASKED ? 1 : a.rows_per_cta;  // (at most G / 32)
  static_assert(G == 128 && kStage * 4 >= (int)sizeof(FastScratch) && kCapB * 4 >= (int)sizeof(FastScratch), "the warps' scratch lies in four of the arrays above");
  static_assert(3 * kStage * 4 >= (int)sizeof(FastScratchCta), "the CTA-wide fast path's scratch is the three stage arrays together");
  __shared__ int row_rc[G / 32];
  const int b_first = (int)blockIdx.x * kRows;
  if (!MASKED) {
    const int w = gt >> 5, bw = b_first + w;
    int rc = kFastSlow;
    if (kRows == 1) {  // few rows: the whole CTA on one
      rc = finish_row_fast<T, G>(a, b_first, *reinterpret_cast<FastScratchCta*>(fl_all), hist);
      if (w > 0) rc = kFastDone;
    } else if (w >= kRows || bw >= a.B) {
      rc = kFastDone;
    } else {
      void* scratch = w == 0 ? (void*)fl_key : w == 1 ? (void*)fl_id : w == 2 ? (void*)fl_cnt : (void*)bkey;
      rc = finish_row_fast<T, 32>(a, bw, *reinterpret_cast<FastScratch*>(scratch), nullptr);
    }
    if ((gt & 31) == 0) row_rc[w] = rc;
    __syncthreads();
  }
  for (int rr = 0; rr < kRows; ++rr) {
  const int b = b_first + rr;
  if (b >= a.B) break;
  if (!MASKED) {
    if (row_rc[rr] == kFastDone) continue;
    if (row_rc[rr] == kFastLate) {
      if (gt == 0) {
        raise_status(a.status, ARCS_ERR_TIMEOUT);
        a.token[b] = -1;
      }
      continue;
    }
  }
  __syncthreads();  // (the row before is through with the shared arrays)
  if (gt == 0) {
    sh[S_CNT_B] = 0;
    sh[S_CNT_A] = 0;
    sh[S_FLAGS] = 0;
    sh[S_BANS] = 0;
    sh[S_NFLAG] = 0;
    sh[S_NLIST] = 0;
    sh[S_NLISTA] = 0;
    sh[S_OVER] = 0;
    sh[S_NPRE] = 0;
    s64[L_TAU_B] = 0ull;
    s64[L_TAU_A] = 0ull;
  }
  __syncthreads();
  // The stream kernel's lists and headers are read from here on. That kernel may still be running
  // (this one is launched behind it with programmatic stream serialization and does not wait for
  // its end): a row is taken when all its items have been released. The wait is bounded.
  if (!merging) {
    bool late = false;
    for (int g = gt; g < a.nseg; g += G) {
      const int32_t* flag = &item_ws(a, b * a.nseg + g).hdr->streamed;
      uint32_t spins = 0;
      while (ld_acquire_gpu(flag) == 0) {
        if (++spins > kFlagWaitLimit) {
          late = true;
          break;
        }
        __nanosleep(spins < 64 ? 100 : 400);
      }
    }
    if (__syncthreads_or(late)) {
      if (gt == 0) {
        raise_status(a.status, ARCS_ERR_TIMEOUT);
        a.token[b] = -1;
      }
      continue;
    }
  }
  // what the segments' headers say (fetched together with the row's settings). Nothing at or
  // below the largest threshold a segment's stream ended on can be among the k best: that
  // segment alone holds k above it.
  const RowCfg r = row_cfg<MASKED>(a, b);  // (its loads travel together with the headers')
  if (merging && gt < 32) combine_mz(a, b);
  if (merging) {  // the banned-tail rule needs to know whether the row's bias list bans anything (tools/sampler.h:34)
    bool any = false;
    for (int i = gt; i < r.NB; i += G) any = any || a.bias_vals[r.q0 + i] <= -100.0f;
    if (any) sm_red_or(&sh[S_BANS], 1u);
    if (gt == 0) sh[S_NLIST] = a.merge_G * a.merge_stride;
  }
  for (int g = gt; g < a.nseg && !merging; g += G) {
    const ItemHdr* hd = item_ws(a, b * a.nseg + g).hdr;
    int n0 = __ldcg(&hd->n_pre);
    const int nt = __ldcg(&hd->n_tch);
    int n1 = __ldcg(&hd->n_candB), n2 = MASKED ? __ldcg(&hd->n_candA) : 0;
    // a list of the stream that overflowed was only counted: the segment is read again below
    const bool over = n1 > kListB || n2 > kListA || nt > item_pre_cap(a.hash_slots) - n0;
    if (over) n1 = n2 = 0;
    else n0 += nt;  // (the stream kernel appends right behind the prepare kernel's entries)
    seg_n[0][g] = n0;
    seg_n[1][g] = n1;
    seg_n[2][g] = n2;
    seg_n[3][g] = over;
    if (over) sm_red_or(&sh[S_OVER], 1u);
    sm_red_add(&sh[S_NLIST], (uint32_t)(n0 + n1));
    sm_red_add(&sh[S_NPRE], (uint32_t)n0);  // (only these entries can be flagged)
    if (MASKED) sm_red_add(&sh[S_NLISTA], (uint32_t)(n0 + n2));
    if (__ldcg(&hd->bans) != 0) sm_red_or(&sh[S_BANS], 1u);
    sm_red_max_u64(&s64[L_TAU_B], __ldcg(&hd->tauB));
    if (MASKED) sm_red_max_u64(&s64[L_TAU_A], __ldcg(&hd->tauA));
  }
  __syncthreads();
  const bool bans = sh[S_BANS] != 0;
  // barriers between the rounds of pushes are needed only when a buffer or the stage could overflow
  const bool careful = sh[S_OVER] != 0 || sh[S_NLIST] > kCapB || (MASKED && sh[S_NLISTA] > kCapA) || sh[S_NPRE] > kStage;
  const PruneScratch psF{hist, tk, ti, misc, &s64[L_PRUNE_MIN]};
  // (a buffer is pruned only when it is nearly full: looked at after every four rounds of G pushes)
  const Sel selB{bkey, bid, &sh[S_CNT_B], &s64[L_TAU_B], r.kB, kCapB - 4 * G, kCapB};
  const Sel selA{akey, aid, &sh[S_CNT_A], &s64[L_TAU_A], ARCS_HEAD, kCapA - 4 * G, kCapA};

  bool hot = false;
  // called by the whole group after a barrier behind which nobody pushes
  auto maybe_prune = [&]() {
    const bool pb = *selB.cnt > selB.trig, pa = MASKED && *selA.cnt > selA.trig;
    group_sync<2, G>();
    if (pb) sel_prune<2, G>(selB, selB.k, psF, gt);
    if (pa) sel_prune<2, G>(selA, selA.k, psF, gt);
  };
  const uint32_t* mrow = MASKED ? a.mask + (size_t)(a.mask_row ? a.mask_row[b] : b) * a.mask_stride : nullptr;
  // after a round of pushes: prune when a buffer has grown past its trigger
  // (at most G pushes on top of a buffer at or below its trigger: inside its capacity)
  auto after_push = [&]() {
    if (group_sync_or<2, G>(hot)) {
      maybe_prune();
      hot = false;
    }
  };
  // Settle the staged flagged entries (tools/sampler.h:154-174 for them): one in the bias list
  // was evaluated by the prepare kernel and is dropped here; one in the history is dropped too
  // when the prepare kernel evaluated the history (table mode), else penalised here; one the
  // filter flagged by accident is an ordinary element.
  auto settle = [&]() {
    group_sync<2, G>();
    const int nF = min(sh[S_NFLAG], kStage);
    if (nF == 0) return;
    for (int f = gt; f < nF; f += G) fl_cnt[f] = 0u;
    group_sync<2, G>();
    const int32_t w0 = window_start(r);
    for (int i = gt; i < r.NB; i += G) {
      const int32_t t = a.bias_ids[r.q0 + i];
      for (int f = 0; f < nF; ++f)
        if ((fl_id[f] & (int32_t)kIdMask) == t) sm_red_or(&fl_cnt[f], 1u << 30);
    }
    if (r.pen_on) {
      for (int i = gt; i < r.H; i += G) {
        const int32_t t = __ldg(&a.hist_ids[r.h0 + i]);
        for (int f = 0; f < nF; ++f)
          if ((fl_id[f] & (int32_t)kIdMask) == t) {
            sm_red_add(&fl_cnt[f], 1u);
            if (i >= w0) sm_red_or(&fl_cnt[f], 1u << 31);
          }
      }
    }
    group_sync<2, G>();
    for (int f0 = 0; f0 < nF; f0 += G) {
      const int f = f0 + gt;
      bool p = f < nF;
      uint32_t ky = 0u;
      int32_t id = 0;
      bool okB = false;
      if (p) {
        const uint32_t info = fl_cnt[f], cnt = info & 0x3FFFFFFFu;
        ky = fl_key[f];
        id = fl_id[f] & (int32_t)kIdMask;
        okB = (fl_id[f] & (int32_t)kOkB) != 0;
        if ((info >> 30) & 1u) {
          p = false;
        } else if (cnt > 0) {
          if (r.touch == kTouchTable) {
            p = false;
          } else {
            const float v = penalise(r, value_of(ky), cnt, w0 == 0 || (info >> 31));
            ky = key_of(v);
            p = ky != 0u;
            if (MASKED) okB = ((__ldg(&mrow[id >> 5]) >> (id & 31)) & 1u) && !(bans && v + 0.0f <= ARCS_BANNED);  // tools/sampler.h:118-119
          }
        }
      }
      const uint64_t cm = comp_of(ky, id);
      sel_push(selB, p && okB && cm > *selB.tau, ky, id, hot, a.status);
      if (MASKED) sel_push(selA, p && cm > *selA.tau, ky, id, hot, a.status);
      after_push();
    }
    if (gt == 0) sh[S_NFLAG] = 0;
    group_sync<2, G>();
  };
  // Two lists of entries (key | word y << 32) into the selections, a round of G at a time:
  // `first` feeds both selections, `second` only one (the selection proper, or with toA the
  // constrained head ranking). The entries of several rounds are fetched together; flagged
  // entries are staged.
  auto take = [&](const unsigned long long* first, int n1, const unsigned long long* second, int n2, bool toA) {
    constexpr int R = 8;
    const int n = n1 + n2;
    for (int i0 = 0; i0 < n; i0 += R * G) {
      unsigned long long e[R];
#pragma unroll
      for (int x = 0; x < R; ++x) {
        const int i = i0 + x * G + gt;
        e[x] = i < n1 ? __ldcg(&first[i]) : i < n ? __ldcg(&second[i - n1]) : 0ull;
      }
#pragma unroll
      for (int x = 0; x < R; ++x) {
        if (i0 + x * G >= n) break;
        const int i = i0 + x * G + gt;
        const bool p = i < n, one = i < n1;
        const uint32_t ky = (uint32_t)e[x], y = (uint32_t)(e[x] >> 32);
        const int32_t id = (int32_t)(y & kIdMask);
        const bool fl = p && (y & kTch);
        const uint64_t cm = comp_of(ky, id);
        sel_push(selB, p && !fl && (one || !toA) && (y & kOkB) && cm > *selB.tau, ky, id, hot, a.status);
        if (MASKED) sel_push(selA, p && !fl && (one || toA) && cm > *selA.tau, ky, id, hot, a.status);
        const unsigned bf = __ballot_sync(0xFFFFFFFFu, fl);
        if (bf) {
          const int lane = gt & 31, leader = __ffs(bf) - 1;
          int base = 0;
          if (lane == leader) base = (int)sm_atomic_add(&sh[S_NFLAG], (uint32_t)__popc(bf));
          base = __shfl_sync(0xFFFFFFFFu, base, leader);
          if (fl) {
            const int pos = base + __popc(bf & ((1u << lane) - 1u));  // (inside the stage: it is emptied below before a round could overflow it)
            fl_key[pos] = ky;
            fl_id[pos] = (int32_t)(y & (kIdMask | kOkB));
          }
        }
        if (careful && ((x & 3) == 3 || i0 + (x + 1) * G >= n)) {
          after_push();
          if (sh[S_NFLAG] > kStage - 4 * G) settle();
        }
      }
    }
  };
  // A segment whose lists overflowed is read again here, element by element, against the
  // thresholds known by now (slow, and rare: ascending data, masses of equal logits).
  auto rescan = [&](int g) {
    constexpr int E = Elem<T>::kPerChunk;
    const Item<T> it = item_of<T>(a, b * a.nseg + g);
    const ItemWs w = item_ws(a, b * a.nseg + g);
    const int bw = bloom_words_of(a.hash_slots);
    const int nchunk = it.p.body_bytes / 16;
    for (int c0 = 0; c0 < nchunk; c0 += G) {
      const int ci = c0 + gt;
      const uint4 q = ci < nchunk ? ldg128_stream(it.p.body + (size_t)ci * 16) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float v = Elem<T>::get(q, e);
        const int32_t id = it.p.body_first + ci * E + e + a.id_base;
        const uint32_t ky = key_of(v);
        const uint64_t cm = comp_of(ky, id);
        bool p = ci < nchunk && ky != 0u && (cm > *selB.tau || (MASKED && cm > *selA.tau));
        bool fl = false;
        if (p && r.touch != kTouchNone) {
          fl = bloom_has([&](uint32_t wi) { return __ldg(&w.bloom[wi]); }, bw, id - a.id_base);
        }
        bool okB = true;
        if (MASKED && p) okB = ((__ldg(&mrow[id >> 5]) >> (id & 31)) & 1u) && !(bans && v + 0.0f <= ARCS_BANNED);  // tools/sampler.h:118-119
        sel_push(selB, p && !fl && okB && cm > *selB.tau, ky, id, hot, a.status);
        if (MASKED) sel_push(selA, p && !fl && cm > *selA.tau, ky, id, hot, a.status);
        const unsigned bf = __ballot_sync(0xFFFFFFFFu, p && fl);
        if (bf) {
          const int lane = gt & 31, leader = __ffs(bf) - 1;
          int base = 0;
          if (lane == leader) base = (int)sm_atomic_add(&sh[S_NFLAG], (uint32_t)__popc(bf));
          base = __shfl_sync(0xFFFFFFFFu, base, leader);
          if (p && fl) {
            const int pos = base + __popc(bf & ((1u << lane) - 1u));
            fl_key[pos] = ky;
            fl_id[pos] = (int32_t)((uint32_t)id | (okB ? kOkB : 0u));
          }
        }
        after_push();
        if (sh[S_NFLAG] > kStage - G) settle();
      }
    }
  };
  if (!merging) {
    for (int g = 0; g < a.nseg; ++g) {
      const ItemWs w = item_ws(a, b * a.nseg + g);
      take(w.pre, seg_n[0][g], w.candB, seg_n[1][g], false);
      if (MASKED) take(nullptr, 0, w.candA, seg_n[2][g], true);
      if (seg_n[3][g]) rescan(g);
    }
  } else {
    // the shards' lists: each already holds that shard's k best under the same order
    for (int g = 0; g < a.merge_G; ++g) {
      const size_t row = (size_t)g * a.B + b;
      const int n = a.merge_n ? min(__ldg(&a.merge_n[row]), a.merge_width) : a.merge_width;  // (without lengths a list ends at its first negative id)
      for (int i0 = 0; i0 < n; i0 += G) {
        const int i = i0 + gt;
        const bool p = i < n;
        const float v = p ? __ldg(&a.merge_val[row * a.merge_stride + i]) : 0.0f;
        const int32_t id = p ? __ldg(&a.merge_id[row * a.merge_stride + i]) : 0;
        const uint32_t ky = key_of(v);
        sel_push(selB, p && id >= 0 && ky != 0u && comp_of(ky, id) > *selB.tau, ky, id, hot, a.status);
        if (careful) after_push();
      }
    }
  }
  settle();
  group_sync<2, G>();
  if (MASKED) sel_prune<2, G>(selA, selA.k, psF, gt);
  if (MASKED && a.head_id) {
    // the ranked head: the (at most) 512 best of all tokens, banned ones included, best first
    // (composites are unique, so counting the larger ones ranks them)
    const int nA = min(*selA.cnt, ARCS_HEAD);
    for (int i = gt; i < ARCS_HEAD; i += G) {
      if (i < nA) {
        const uint64_t c = comp_of(selA.key[i], selA.id[i]);
        int rank = 0;
        for (int x = 0; x < nA; ++x) rank += comp_of(selA.key[x], selA.id[x]) > c;
        a.head_id[(size_t)b * ARCS_HEAD + rank] = selA.id[i];
        a.head_val[(size_t)b * ARCS_HEAD + rank] = value_of(selA.key[i]);
      } else {
        a.head_id[(size_t)b * ARCS_HEAD + i] = -1;
        a.head_val[(size_t)b * ARCS_HEAD + i] = 0.0f;
      }
    }
    if (gt == 0) a.n_head[b] = nA;
  }

  // ---- candidates best first. A short buffer is ranked by counting, which selects the k best
  // and sorts them in one step; a longer one is cut to the k best by the radix select first.
  const int sort_cap = max(kSortCap, selB.k + 64);
  if (*selB.cnt > sort_cap) sel_prune<2, G>(selB, selB.k, psF, gt);
  group_sync<2, G>();
  const int nbuf = min(*selB.cnt, sort_cap);
  const int nB = min(nbuf, selB.k);
  for (int i = gt; i < nbuf; i += G) {
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
  group_sync<2, G>();
  // ---- tools/sampler.h:54-77 (or :105-143)
  int flags = 0, nc = nB;
  if (MASKED) {
    const int nA = min(*selA.cnt, ARCS_HEAD);
    for (int i = gt; i < nA; i += G) {
      const uint64_t c = comp_of(selA.key[i], selA.id[i]);
      if (!(bans && value_of(selA.key[i]) <= ARCS_BANNED)) sm_red_max_u64(&s64[L_TOP], (unsigned long long)c);
      sm_red_min_u64(&s64[L_LOW], (unsigned long long)c);
    }
    group_sync<2, G>();
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
    group_sync<2, G>();
    nc = sh[S_NCAND];
  } else {
    if (gt == 0) {
      if (bans)  // tools/sampler.h:54-55
        while (nc > 1 && sv[nc - 1] <= ARCS_BANNED) --nc;
      sh[S_NCAND] = nc;
    }
    group_sync<2, G>();
    nc = sh[S_NCAND];
  }
  {  // equal logits among the candidates kept: the reference's order there is not defined
    bool tie = false;
    for (int i = gt; i + 1 < nc; i += G) tie = tie || sv[i] == sv[i + 1];
    if (tie) sm_red_or(&sh[S_FLAGS], (uint32_t)ARCS_FLAG_TIE_TOPK);
  }
  const bool draw = (!r.greedy && nc > 1) || (!MASKED && !r.greedy && nc == 1);
  if (draw) {
    const float mx = sv[0];
    for (int i = gt; i < nc; i += G) {
      const float x = __fdiv_rn(__fsub_rn(sv[i], mx), r.prm.temperature);  // :60 float arithmetic
      spr[i] = (double)(float)exp((double)x);                              // float exp, widened
    }
    group_sync<2, G>();
    if (gt == 0) {
      double z = 0.0;
#pragma unroll 8
      for (int i = 0; i < nc; ++i) z = __dadd_rn(z, spr[i]);  // :58-60 in candidate order
      spr[ARCS_KCAP] = z;
    }
    group_sync<2, G>();
    const double z = spr[ARCS_KCAP];
    for (int i = gt; i < nc; i += G) spr[i] = __ddiv_rn(spr[i], z);  // :64, the same quotients in any order
  }
  group_sync<2, G>();
  // :65-72. The running sums are a chain of roundings in candidate order (one thread); where the
  // chain is cut is then found by all threads.
  double* cum = reinterpret_cast<double*>(bkey);  // (the buffer is no longer needed: 256 doubles fit)
  if (gt == 0) {
    sh[S_NCAND] = nc;  // n: candidates left after the cuts
    if (draw) {
      double c = 0.0;
#pragma unroll 8
      for (int i = 0; i < nc; ++i) {
        c = __dadd_rn(c, spr[i]);
        cum[i] = c;
      }
    }
  }
  group_sync<2, G>();
  if (draw) {
    const double mp = __dmul_rn((double)r.prm.min_p, spr[0]);
    for (int i = gt; i < nc; i += G) {
      int n_i = 0x7FFFFFFF;
      if (r.prm.min_p > 0.0f && spr[i] < mp) n_i = max(1, i);   // :65 (tested before the candidate is added)
      else if (cum[i] >= (double)r.prm.top_p) n_i = i + 1;      // :67
      if (n_i != 0x7FFFFFFF) sm_red_min_s32(&sh[S_NCAND], n_i);
    }
  }
  group_sync<2, G>();
  if (gt == 0) {
    int token = nc > 0 ? sid[0] : -1, n = nc > 0 ? 1 : 0;
    if (draw) {
      n = sh[S_NCAND];
      const double tot = cum[n - 1];                                            // the same sum, in the same order, as :70
      double rr = __dmul_rn(a.u[b], tot);                                       // :71-72
      int pick = -1;
      for (int i = 0; i < n && pick < 0; i += 4) {  // (four steps of the chain at a time: the loads run ahead of it)
        const double p0 = spr[i], p1 = i + 1 < n ? spr[i + 1] : 0.0, p2 = i + 2 < n ? spr[i + 2] : 0.0, p3 = i + 3 < n ? spr[i + 3] : 0.0;
        const double r0 = __dsub_rn(rr, p0), r1 = __dsub_rn(r0, p1), r2 = __dsub_rn(r1, p2), r3 = __dsub_rn(r2, p3);
        if (r0 <= 0.0) pick = i;
        else if (i + 1 < n && r1 <= 0.0) pick = i + 1;
        else if (i + 2 < n && r2 <= 0.0) pick = i + 2;
        else if (i + 3 < n && r3 <= 0.0) pick = i + 3;
        rr = r3;
      }
      if (pick < 0) pick = n - 1;
      token = sid[pick];
    }
    if (r.k_bad || !r.lists_ok) token = -1;
    a.token[b] = token;
    if (a.n_cand) a.n_cand[b] = nc;
    if (a.n_kept) a.n_kept[b] = n;
  }
  group_sync<2, G>();
  if (gt == 0 && a.flags) a.flags[b] = sh[S_FLAGS];
  if (gt == 0 && nc > a.cand_width && (a.cand_id || a.cand_val || a.cand_pr)) raise_status(a.status, ARCS_ERR_TOPK);
  for (int i = gt; i < a.cand_width && (a.cand_id || a.cand_val || a.cand_pr); i += G) {
    const size_t o = (size_t)b * a.cand_stride + i;
    const bool in = i < nc;
    if (a.cand_id) a.cand_id[o] = in ? sid[i] : -1;
    if (a.cand_val) a.cand_val[o] = in ? sv[i] : 0.0f;
    if (a.cand_pr) a.cand_pr[o] = in ? (draw ? (float)spr[i] : (i == 0 ? 1.0f : 0.0f)) : 0.0f;
  }
  }  // (rows of this CTA)
}

}  // namespace arcs
