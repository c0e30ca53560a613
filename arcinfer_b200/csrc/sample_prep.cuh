// prep_item: everything about an item that does not need the pass over its logits, done by a
// small group of warps of the stream kernel ahead of the stream.
//
// For one item (a row, or a segment of a row) the group builds, in the shared-memory set of
// per-item state the scanners will read:
//  - a filter over the columns a penalty or a bias touches (tools/sampler.h:154-174), which the
//    scanners consult for their hot elements;
//  - the item's header (how many candidates the row keeps, how touched tokens are handled), and
//    one bit per 16-byte chunk of the item's first tiles that holds a listed column (those chunks
//    are left out when the item's first threshold is read off these tiles);
// and writes to the item's block of the workspace entries with final values for the tokens it
// evaluates itself, with the exact fp32 arithmetic of Sampler::adjusted: the bias tokens, and -
// when some penalty can raise a logit, so that a token may matter although its raw logit is not
// hot - every history token; and the few elements outside the item's 16-byte aligned body.
#pragma once
#include "sample_common.cuh"

namespace arcs {

static_assert(kPrepG >= 64, "two whole warps take the scalar elements at either end of an item");

// indices into the group's small scratch
enum { P_NPRE = 0, P_CMD = 1, P_END = 4 };

// hk / hi_: [hash_slots] table of the distinct listed columns (table mode only); bl: the set's
// filter; skip: the set's [kBootSkipWords] chunk bits; shdr: the set's header; pmisc: [P_END].
// Called by all kPrepG threads (gt = index in the group).
template <typename T, bool MASKED>
__device__ __forceinline__ void prep_item(const SampleDev& a, int item, ItemHdr* shdr, uint32_t* bl, uint32_t* skip, uint32_t* hk,
                                          uint32_t* hi_, int* pmisc, int gt) {
  constexpr int G = kPrepG;
  const int bw = bloom_words_of(a.hash_slots);
  const int lane = gt & 31;
  const int32_t Vg = a.v_global > 0 ? a.v_global : a.V;
  const Item<T> it = item_of<T>(a, item);
  const RowCfg r = row_cfg<MASKED>(a, it.b);
  const ItemWs w = item_ws(a, item);
  const uint32_t* mrow = MASKED ? a.mask + (size_t)(a.mask_row ? a.mask_row[it.b] : it.b) * a.mask_stride : nullptr;

  if (gt == 0) {
    if (r.k_bad) raise_status(a.status, ARCS_ERR_TOPK);
    if (!r.lists_ok) raise_status(a.status, ARCS_ERR_LIST);
  }
  if (gt == 0) pmisc[P_NPRE] = 0;
  for (int i = gt; i < kBootSkipWords; i += G) skip[i] = 0u;
  bool bans = false;  // Sampler::bans_: any bias entry <= -100, in range or not (tools/sampler.h:34)
  for (int i = gt; i < r.NB && r.lists_ok; i += G) bans = bans || a.bias_vals[r.q0 + i] <= -100.0f;
  bans = group_sync_or<3, G>(bans);

  // column of a listed id inside this item, -1 when it is not this item's
  auto col_of = [&](int32_t t) -> int32_t {
    if (t < 0 || t >= Vg) return -1;
    const int32_t c = t - a.id_base;
    return (c < it.lo || c >= it.hi) ? -1 : c;
  };
  // A listed column inside the item's first kBootTiles tiles marks its 16-byte chunk: the chunk's
  // maximum may be that token's raw logit, which counts for no threshold.
  auto count_window = [&](bool valid, int32_t c) {
    if (!valid) return;
    const int32_t rel = c - it.p.body_first;
    if (rel >= 0 && rel < kBootBytes / (int)sizeof(T)) {
      const int ch = rel / (16 / (int)sizeof(T));
      sm_red_or(&skip[ch % kPrepG], 1u << (ch / kPrepG));
    }
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
    if (lane == leader) base = (int)sm_atomic_add(&pmisc[P_NPRE], (uint32_t)__popc(bal));
    base = __shfl_sync(0xFFFFFFFFu, base, leader);
    if (!valid) return;
    const int32_t g = c + a.id_base;
    bool okB = true;
    if (MASKED) okB = ((__ldg(&mrow[g >> 5]) >> (g & 31)) & 1u) && !(bans && v + 0.0f <= ARCS_BANNED);  // tools/sampler.h:118-119
    w.pre[base + __popc(bal & ((1u << lane) - 1u))] =
        (unsigned long long)ky | ((unsigned long long)((uint32_t)g | (okB ? kOkB : 0u) | (flagged ? kTch : 0u)) << 32);
  };

  if (r.touch != kTouchNone) {
    for (int i = gt; i < bw; i += G) bl[i] = 0u;
    group_sync<3, G>();
  }
  if (r.touch == kTouchLight) {
    // ---- the filter over every listed column; the bias tokens evaluated here
    constexpr int R = 4;  // ids fetched together: one trip to memory per batch, not per id
    if (r.pen_on) {
      for (int i0 = 0; i0 < r.H; i0 += R * G) {
        int32_t t[R];
#pragma unroll
        for (int x = 0; x < R; ++x) {
          const int i = i0 + x * G + gt;
          t[x] = i < r.H ? __ldg(&a.hist_ids[r.h0 + i]) : -1;
        }
#pragma unroll
        for (int x = 0; x < R; ++x) {
          const int32_t c = col_of(t[x]);
          count_window(c >= 0, c);
          bloom_add(c >= 0, c);
        }
      }
    }
    if (r.NB > 0) {
      const int32_t w0 = window_start(r);
      for (int i0 = 0; i0 < r.NB; i0 += G) {  // (one round: the list is short in this mode)
        const int i = i0 + gt;
        const int32_t t = i < r.NB ? a.bias_ids[r.q0 + i] : -1;
        const int32_t c = col_of(t);
        bool first = c >= 0;  // evaluated once, at the id's first entry
        for (int j = 0; j < i && first; ++j) first = a.bias_ids[r.q0 + j] != t;
        count_window(first, c);
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
    for (int i = gt; i < a.hash_slots; i += G) {
      hk[i] = kEmpty;
      hi_[i] = 0;
    }
    group_sync<3, G>();
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
      return -1;  // (not reachable: rows whose lists exceed half the table are refused, row_cfg)
    };
    // the bias list goes in first: a slot that carries a bias flag was opened by it, any other by the history
    for (int i = gt; i < r.NB; i += G) {
      const int s = insert(a.bias_ids[r.q0 + i]);
      if (s >= 0) sm_red_or(&hi_[s & 0x3FFFFFFF], a.bias_vals[r.q0 + i] > -100.0f ? kInfoBias : kInfoBan);
    }
    group_sync<3, G>();
    const int32_t w0 = window_start(r);
    if (r.pen_on) {
      for (int i = gt; i < r.H; i += G) {
        // one atomic per id, more only for a repeated id (its count is 1 + the additions) and
        // for a window shorter than the history
        const int s = insert(a.hist_ids[r.h0 + i]);
        if (s >= 0 && (s & 0x40000000)) sm_red_add(&hi_[s & 0x3FFFFFFF], 1u);
        if (s >= 0 && w0 > 0 && i >= w0) sm_red_or(&hi_[s & 0x3FFFFFFF], kInfoWindow);
      }
    }
    group_sync<3, G>();
    constexpr int R = 4;  // table slots per thread per batch: their logits are fetched together
    for (int s0 = 0; s0 < a.hash_slots; s0 += R * G) {
      uint32_t ck[R], info[R];
      float raw[R];
#pragma unroll
      for (int x = 0; x < R; ++x) {
        const int s = s0 + x * G + gt;
        ck[x] = s < a.hash_slots ? hk[s] : kEmpty;
        info[x] = ck[x] != kEmpty ? hi_[s] : 0u;
        raw[x] = ck[x] != kEmpty ? Elem<T>::load(it.row + (int32_t)ck[x]) : 0.0f;
      }
#pragma unroll
      for (int x = 0; x < R; ++x) {
        const bool valid = ck[x] != kEmpty;
        float v = raw[x];
        if (valid) {
          const uint32_t cnt = (info[x] & kInfoCount) + ((info[x] & (kInfoBias | kInfoBan)) ? 0u : 1u);  // (the id that opened a slot is not added)
          if (info[x] & kInfoBias) {  // :154-155 in list order, duplicates add again
            const int32_t g = (int32_t)ck[x] + a.id_base;
            for (int i = 0; i < r.NB; ++i)
              if (a.bias_ids[r.q0 + i] == g && a.bias_vals[r.q0 + i] > -100.0f) v = __fadd_rn(v, a.bias_vals[r.q0 + i]);
          }
          if (r.pen_on && cnt > 0) v = penalise(r, v, cnt, w0 == 0 || (info[x] & kInfoWindow));
          if (info[x] & kInfoBan) v = ARCS_BANNED;                                                      // :174
        }
        count_window(valid, (int32_t)ck[x]);
        bloom_add(valid, (int32_t)ck[x]);
        supply(valid, v, (int32_t)ck[x], false);
      }
    }
  }
  group_sync<3, G>();  // the filter is complete
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
  group_sync<3, G>();
  // ---- the item's header
  if (gt == 0) {
    shdr->tauB = 0ull;
    shdr->tauA = 0ull;
    shdr->K = r.kB;
    shdr->touched = r.touch;
    shdr->bans = bans;
    shdr->n_pre = pmisc[P_NPRE];
    shdr->n_tch = 0;
    shdr->n_candB = 0;
    shdr->n_candA = 0;
    shdr->streamed = 0;
  }
  group_sync<3, G>();
}

}  // namespace arcs
