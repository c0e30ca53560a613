// prepare_kernel: everything about an item that does not need the pass over its logits.
//
// One CTA of kGroup threads per item (a row, or a segment of a row). It writes to the item's
// block of the workspace:
//  - a filter over the columns a penalty or a bias touches (tools/sampler.h:154-174), which the
//    stream kernel consults for its hot elements;
//  - entries with final values for the tokens it evaluates itself, with the exact fp32
//    arithmetic of Sampler::adjusted: the bias tokens, and - when some penalty can raise a
//    logit, so that a token may matter although its raw logit is not hot - every history token;
//  - the few elements outside the item's 16-byte aligned body;
//  - a first threshold read off a short prefix of the item.
#pragma once
#include "sample_common.cuh"

namespace arcs {

constexpr int kBootKeys = 1024;  // piece maxima the first threshold is read off

static size_t prep_smem_bytes(int hash_slots) {
  return 16 + (size_t)hash_slots * 8 + 2 * (size_t)kBootKeys * 4 + (size_t)bloom_words_of(hash_slots) * 4 + 16 * 4;
}

template <typename T, bool MASKED>
__global__ void __launch_bounds__(kGroup) prepare_kernel(const SampleDev a) {
  extern __shared__ __align__(128) char smem[];
  const int bw = bloom_words_of(a.hash_slots);
  unsigned long long* m64 = reinterpret_cast<unsigned long long*>(smem);      // [2]
  uint32_t* hk = reinterpret_cast<uint32_t*>(m64 + 2);                         // [hash_slots] token columns (table mode)
  uint32_t* hi_ = hk + a.hash_slots;                                           // [hash_slots] what applies to them
  uint32_t* ptk = hi_ + a.hash_slots;                                          // [kBootKeys] maxima over pieces of the prefix
  uint32_t* ptk2 = ptk + kBootKeys;                                            // [kBootKeys] ... over their allowed elements only
  uint32_t* bl = ptk2 + kBootKeys;                                             // [bw] the item's filter
  int* pmisc = reinterpret_cast<int*>(bl + bw);
  int* n_pre = pmisc + 0;
  int* n_extra = pmisc + 1;

  constexpr int E = Elem<T>::kPerChunk;
  const int gt = threadIdx.x, lane = gt & 31;
  const int item = blockIdx.x;
  const int32_t Vg = a.v_global > 0 ? a.v_global : a.V;
  pdl_trigger();  // (the stream kernel may move in as CTAs of this one retire; it waits before it reads their output)
  const Item<T> it = item_of<T>(a, item);
  const RowCfg r = row_cfg<MASKED>(a, it.b);
  const ItemWs w = item_ws(a, item);
  const uint32_t* mrow = MASKED ? a.mask + (size_t)(a.mask_row ? a.mask_row[it.b] : it.b) * a.mask_stride : nullptr;

  if (gt == 0) {
    if (r.k_bad) raise_status(a.status, ARCS_ERR_TOPK);
    if (!r.lists_ok) raise_status(a.status, ARCS_ERR_LIST);
    *n_pre = 0;
    *n_extra = 0;
  }
  // the prefix is fetched first: its latency hides behind the list work
  const int nchunk = min(it.p.body_bytes, MASKED ? 2 * 8192 : kBootBytes) / 16;
  const int32_t c_lo = it.p.body_first, c_hi = it.p.body_first + nchunk * E;  // columns of the prefix
  constexpr int kPer = kBootBytes / 16 / kGroup;               // chunks of the prefix per thread
  constexpr int kMaxima = kBootKeys / kGroup;                   // maxima each thread keeps (1024 pieces in all)
  constexpr int kPiece = kPer / kMaxima > 0 ? kPer / kMaxima : 1;  // chunks per piece
  float pm[kMaxima];
  bool pany[kMaxima];
#pragma unroll
  for (int i = 0; i < kMaxima; ++i) {
    pm[i] = -INFINITY;
    pany[i] = false;
  }
  if (!MASKED) {
    // the maxima of the thread's pieces of the prefix (disjoint pieces of kPiece chunks), the
    // chunks fetched eight at a time
    constexpr int kBatch = kPer < 8 ? kPer : 8;
#pragma unroll
    for (int x0 = 0; x0 < kPer; x0 += kBatch) {
      uint4 q[kBatch];
#pragma unroll
      for (int x = 0; x < kBatch; ++x) {
        const int ci = gt + (x0 + x) * kGroup;
        q[x] = ci < nchunk ? ldg128_stream(it.p.body + (size_t)ci * 16) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int x = 0; x < kBatch; ++x) {
        const int ci = gt + (x0 + x) * kGroup;
        if (ci < nchunk) {
          const int pi = ((x0 + x) / kPiece) % kMaxima;
          pm[pi] = fmaxf(pm[pi], Elem<T>::chunk_max(q[x]));
          pany[pi] = true;
        }
      }
    }
  }

  bool bans = false;  // Sampler::bans_: any bias entry <= -100, in range or not (tools/sampler.h:34)
  for (int i = gt; i < r.NB && r.lists_ok; i += kGroup) bans = bans || a.bias_vals[r.q0 + i] <= -100.0f;
  bans = __syncthreads_or(bans) != 0;

  // column of a listed id inside this item, -1 when it is not this item's
  auto col_of = [&](int32_t t) -> int32_t {
    if (t < 0 || t >= Vg) return -1;
    const int32_t c = t - a.id_base;
    return (c < it.lo || c >= it.hi) ? -1 : c;
  };
  // one more column for the filter
  auto bloom_add = [&](bool valid, int32_t c) {
    if (!valid) return;
    const uint32_t b1 = bloom_bit1(c, bw), b2 = bloom_bit2(c, bw);
    sm_red_or(&bl[b1 >> 5], 1u << (b1 & 31));
    sm_red_or(&bl[b2 >> 5], 1u << (b2 & 31));
  };
  // one more entry for the finish kernel (called by whole warps; lanes with `valid` supply):
  // v is the logit of column c, final unless the entry is flagged for the finish kernel to settle
  auto supply = [&](bool valid, float v, int32_t c, bool flagged) {
    const uint32_t ky = key_of(v);
    valid = valid && ky != 0u;
    const unsigned bal = __ballot_sync(0xFFFFFFFFu, valid);
    if (bal == 0u) return;
    const int leader = __ffs(bal) - 1;
    int base = 0;
    if (lane == leader) base = (int)sm_atomic_add(n_pre, (uint32_t)__popc(bal));
    base = __shfl_sync(0xFFFFFFFFu, base, leader);
    if (!valid) return;
    const int32_t g = c + a.id_base;
    bool okB = true;
    if (MASKED) okB = ((__ldg(&mrow[g >> 5]) >> (g & 31)) & 1u) && !(bans && v + 0.0f <= ARCS_BANNED);  // tools/sampler.h:118-119
    w.pre[base + __popc(bal & ((1u << lane) - 1u))] =
        (unsigned long long)ky | ((unsigned long long)((uint32_t)g | (okB ? kOkB : 0u) | (flagged ? kTch : 0u)) << 32);
  };

  int extra = 0;  // listed columns inside the prefix: they may own a maximum there without counting
  if (r.touch != kTouchNone) {
    for (int i = gt; i < bw; i += kGroup) bl[i] = 0u;
    __syncthreads();
  }
  if (r.touch == kTouchLight) {
    // ---- the filter over every listed column; the bias tokens evaluated here
    constexpr int R = 4;  // ids fetched together: one trip to memory per batch, not per id
    if (r.pen_on) {
      for (int i0 = 0; i0 < r.H; i0 += R * kGroup) {
        int32_t t[R];
#pragma unroll
        for (int x = 0; x < R; ++x) {
          const int i = i0 + x * kGroup + gt;
          t[x] = i < r.H ? __ldg(&a.hist_ids[r.h0 + i]) : -1;
        }
#pragma unroll
        for (int x = 0; x < R; ++x) {
          const int32_t c = col_of(t[x]);
          extra += c >= c_lo && c < c_hi;
          bloom_add(c >= 0, c);
        }
      }
    }
    if (r.NB > 0) {
      const int32_t w0 = window_start(r);
      for (int i0 = 0; i0 < r.NB; i0 += kGroup) {  // (one round: the list is short in this mode)
        const int i = i0 + gt;
        const int32_t t = i < r.NB ? a.bias_ids[r.q0 + i] : -1;
        const int32_t c = col_of(t);
        bool first = c >= 0;  // evaluated once, at the id's first entry
        for (int j = 0; j < i && first; ++j) first = a.bias_ids[r.q0 + j] != t;
        extra += first && c >= c_lo && c < c_hi;
        bloom_add(first, c);
        float v = 0.0f;
        if (first) {
          v = Elem<T>::load(it.row + c);
          bool ban = false;
          for (int j = i; j < r.NB; ++j) {  // :154-155 in list order, duplicates add again
            if (a.bias_ids[r.q0 + j] != t) continue;
            const float bv = a.bias_vals[r.q0 + j];
            if (bv > -100.0f) v = __fadd_rn(v, bv);
            else ban = true;
          }
          if (r.pen_on) {
            uint32_t cnt = 0;
            bool in_win = false;
            for (int h = 0; h < r.H; ++h)
              if (__ldg(&a.hist_ids[r.h0 + h]) == t) {
                ++cnt;
                in_win = in_win || h >= w0;
              }
            if (cnt > 0) v = penalise(r, v, cnt, in_win);
          }
          if (ban) v = ARCS_BANNED;                                                                    // :174
        }
        supply(first, v, c, false);
      }
    }
  } else if (r.touch == kTouchTable) {
    // ---- every listed token evaluated here: a table of the distinct columns first
    for (int i = gt; i < a.hash_slots; i += kGroup) {
      hk[i] = kEmpty;
      hi_[i] = 0;
    }
    __syncthreads();
    auto insert = [&](int32_t t) -> int {  // global id -> slot (| 0x40000000 when it was there), -1 when it is not this item's
      const int32_t c = col_of(t);
      if (c < 0) return -1;
      uint32_t h = hash_of(c, a.hash_shift);
      for (int probe = 0; probe < a.hash_slots; ++probe) {
        const uint32_t old = sm_atomic_cas(&hk[h], kEmpty, (uint32_t)c);
        if (old == kEmpty) return (int)h;                                      // first occurrence
        if (old == (uint32_t)c) return (int)h | 0x40000000;                    // seen before
        h = (h + 1) & (uint32_t)(a.hash_slots - 1);
      }
      return -1;
    };
    // the bias list goes in first: a slot that carries a bias flag was opened by it, any other by the history
    for (int i = gt; i < r.NB; i += kGroup) {
      const int s = insert(a.bias_ids[r.q0 + i]);
      if (s >= 0) sm_red_or(&hi_[s & 0x3FFFFFFF], a.bias_vals[r.q0 + i] > -100.0f ? kInfoBias : kInfoBan);
    }
    __syncthreads();
    const int32_t w0 = window_start(r);
    if (r.pen_on) {
      for (int i = gt; i < r.H; i += kGroup) {
        // one atomic per id, more only for a repeated id (its count is 1 + the additions) and
        // for a window shorter than the history
        const int s = insert(a.hist_ids[r.h0 + i]);
        if (s >= 0 && (s & 0x40000000)) sm_red_add(&hi_[s & 0x3FFFFFFF], 1u);
        if (s >= 0 && w0 > 0 && i >= w0) sm_red_or(&hi_[s & 0x3FFFFFFF], kInfoWindow);
      }
    }
    __syncthreads();
    constexpr int R = 4;  // table slots per thread per batch: their logits are fetched together
    for (int s0 = 0; s0 < a.hash_slots; s0 += R * kGroup) {
      uint32_t ck[R], info[R];
      float raw[R];
#pragma unroll
      for (int x = 0; x < R; ++x) {
        const int s = s0 + x * kGroup + gt;
        ck[x] = s < a.hash_slots ? hk[s] : kEmpty;
        info[x] = ck[x] != kEmpty ? hi_[s] : 0u;
        raw[x] = ck[x] != kEmpty ? Elem<T>::load(it.row + (int32_t)ck[x]) : 0.0f;
      }
#pragma unroll
      for (int x = 0; x < R; ++x) {
        const bool valid = ck[x] != kEmpty;
        float v = raw[x];
        if (valid) {
          extra += (int32_t)ck[x] >= c_lo && (int32_t)ck[x] < c_hi;
          const uint32_t cnt = (info[x] & kInfoCount) + ((info[x] & (kInfoBias | kInfoBan)) ? 0u : 1u);  // (the id that opened a slot is not added)
          if (info[x] & kInfoBias) {  // :154-155 in list order, duplicates add again
            const int32_t g = (int32_t)ck[x] + a.id_base;
            for (int i = 0; i < r.NB; ++i)
              if (a.bias_ids[r.q0 + i] == g && a.bias_vals[r.q0 + i] > -100.0f) v = __fadd_rn(v, a.bias_vals[r.q0 + i]);
          }
          if (r.pen_on && cnt > 0) v = penalise(r, v, cnt, w0 == 0 || (info[x] & kInfoWindow));
          if (info[x] & kInfoBan) v = ARCS_BANNED;                                                      // :174
        }
        bloom_add(valid, (int32_t)ck[x]);
        supply(valid, v, (int32_t)ck[x], false);
      }
    }
  }
  if (extra) sm_red_add(n_extra, (uint32_t)extra);
  __syncthreads();
  // ---- the item's filter goes out
  if (r.touch != kTouchNone)
    for (int i = gt; i < bw; i += kGroup) w.bloom[i] = bl[i];
  // the scalar elements before the first and after the last 16-byte boundary; one the filter
  // knows is flagged, like a hot element of the stream, for the finish kernel to settle
  if (gt < 64) {  // (two whole warps: the first takes the head, the second the tail)
    const bool head = gt < 32;
    const bool valid = head ? lane < it.p.head_n : lane < it.p.tail_n;
    const int32_t c = head ? it.lo + lane : it.p.tail_first + lane;
    bool flagged = false;
    if (valid && r.touch != kTouchNone) {
      flagged = bloom_has([&](uint32_t wi) { return bl[wi]; }, bw, c);
    }
    supply(valid, valid ? Elem<T>::load(it.row + c) : 0.0f, c, flagged);
  }
  __syncthreads();

  // first threshold: the k-th largest of up to 1024 maxima over disjoint pieces
  // of the prefix is a lower bound of the k-th best element; listed columns inside the prefix
  // may own a maximum without counting, so that many more are skipped
  const int kth = (MASKED ? ARCS_HEAD : r.kB) + *n_extra;
  unsigned long long tau0B = 0ull, tau0A = 0ull;
  if (!MASKED) {
    // (pieces are merged four and four when 256 maxima are enough: the search is a quarter the work)
    const bool fine = kth > 2 * kGroup;
    if (fine) {
#pragma unroll
      for (int i = 0; i < kMaxima; ++i) ptk[i * kGroup + gt] = pany[i] ? key_of(pm[i]) : 0u;
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float m = -INFINITY;
        bool any = false;
#pragma unroll
        for (int i = h * (kMaxima / 2); i < (h + 1) * (kMaxima / 2); ++i) {
          m = fmaxf(m, pm[i]);
          any = any || pany[i];
        }
        ptk[h * kGroup + gt] = any ? key_of(m) : 0u;
      }
    }
    __syncthreads();
    if (kth <= min(nchunk / (fine ? kPiece : kPiece * (kMaxima / 2)), fine ? kBootKeys : 2 * kGroup)) {
      if (gt < 32)
        m64[1] = (unsigned long long)(fine ? warp_kth16<kBootKeys / 32>(ptk, kth) : warp_kth16<2 * kGroup / 32>(ptk, kth)) << 32;  // keeps ties with it
      __syncthreads();
      tau0B = m64[1];
    }
  } else {
    // constrained rows rank the whole vocabulary's best 512: k-th largest of up to 1024 chunk
    // maxima; and the selection proper gets its first threshold from the maxima over the allowed
    // elements of the same chunks (without one, every allowed token of a dense mask would be listed)
    if (nchunk <= kBootKeys) {
      for (int ci = gt; ci < kBootKeys; ci += kGroup) {
        uint32_t kA = 0u, kB = 0u;
        if (ci < nchunk) {
          const uint4 q = ldg128_stream(it.p.body + (size_t)ci * 16);
          kA = key_of(Elem<T>::chunk_max(q));
          const int32_t gid = it.p.body_first + ci * E + a.id_base;
          uint32_t bits = __ldg(&mrow[gid >> 5]) >> (gid & 31);
          if ((gid & 31) + E > 32) bits |= __ldg(&mrow[(gid >> 5) + 1]) << (32 - (gid & 31));
          float mB = -INFINITY;
          bool anyB = false;
#pragma unroll
          for (int e = 0; e < E; ++e)
            if ((bits >> e) & 1u) {
              const float v = Elem<T>::get(q, e);
              if (!(v != v)) {  // (a NaN is never selected)
                mB = fmaxf(mB, v);
                anyB = true;
              }
            }
          if (anyB) kB = key_of(mB);
        }
        ptk[ci] = kA;
        ptk2[ci] = kB;
      }
      __syncthreads();
      const int kthB = r.kB + *n_extra;
      if (gt < 32) {
        if (kth <= nchunk) m64[1] = (unsigned long long)warp_kth16<kBootKeys / 32>(ptk, kth) << 32;  // keeps ties with it
      } else if (gt < 64) {
        if (kthB <= nchunk) m64[0] = (unsigned long long)warp_kth16<kBootKeys / 32>(ptk2, kthB) << 32;
      }
      __syncthreads();
      if (kth <= nchunk) tau0A = m64[1];
      if (kthB <= nchunk) tau0B = m64[0];
    }
  }
  // ---- the item's header
  if (gt == 0) {
    ItemHdr h;
    h.tau0B = tau0B;
    h.tau0A = tau0A;
    h.tauB = tau0B;
    h.tauA = tau0A;
    h.K = r.kB;
    h.touched = r.touch;
    h.bans = bans;
    h.baseB = (int32_t)(tau0B >> 48);
    h.baseA = (int32_t)(tau0A >> 48);
    h.n_pre = *n_pre;
    h.n_tch = 0;
    h.n_candB = 0;
    h.n_candA = 0;
    for (int i = 0; i < 7; ++i) h.pad[i] = 0;
    *w.hdr = h;
  }
}

}  // namespace arcs
