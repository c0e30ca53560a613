// prepare_kernel: everything about an item that does not need the pass over its logits.
//
// One CTA of kGroup threads per item (a row, or a segment of a row). It builds the table of the
// tokens the stream must not supply (every id of the history a penalty applies to, every id of
// the bias list: tools/sampler.h:154-174), evaluates those tokens itself with the exact fp32
// arithmetic of Sampler::adjusted, adds the few elements outside the item's 16-byte aligned
// body, and reads a first threshold off a short prefix of the item. Results go to the item's
// block of the workspace.
#pragma once
#include "sample_common.cuh"

namespace arcs {

static size_t prep_smem_bytes(int hash_slots) {
  return (size_t)hash_slots * 8 + kBloomWords * 4 + 512 * 4 + (size_t)kTmpCap * 8 + 16 * 4 + 16;
}

template <typename T, bool MASKED>
__global__ void __launch_bounds__(kGroup) prepare_kernel(const SampleDev a) {
  extern __shared__ __align__(128) char smem[];
  unsigned long long* m64 = reinterpret_cast<unsigned long long*>(smem);      // [2]
  uint32_t* hk = reinterpret_cast<uint32_t*>(m64 + 2);                         // [hash_slots] token columns
  uint32_t* hi_ = hk + a.hash_slots;                                           // [hash_slots] what applies to them
  uint32_t* bloom = hi_ + a.hash_slots;                                        // [kBloomWords]
  uint32_t* phist = bloom + kBloomWords;                                       // [512]
  uint32_t* ptk = phist + 512;                                                 // [kTmpCap]
  int32_t* pti = reinterpret_cast<int32_t*>(ptk + kTmpCap);                    // [kTmpCap]
  int* pmisc = reinterpret_cast<int*>(pti + kTmpCap);                          // [8] select scratch, [8..] counters
  int* n_pre = pmisc + 8;
  int* n_extra = pmisc + 9;

  constexpr int E = Elem<T>::kPerChunk;
  const int gt = threadIdx.x;
  const int item = blockIdx.x;
  const int32_t Vg = a.v_global > 0 ? a.v_global : a.V;
  const PruneScratch psP{phist, ptk, pti, pmisc, &m64[0]};
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
  // the prefix is fetched first: its latency hides behind the table work
  const int nchunk = min(it.p.body_bytes, MASKED ? 2 * kBootBytes : kBootBytes) / 16;
  float m0 = -INFINITY, m1 = -INFINITY;
  bool any0 = false, any1 = false;
  if (!MASKED) {
    // two maxima per thread, each over every other one of the thread's chunks of the prefix
    for (int ci = gt; ci < nchunk; ci += 2 * kGroup) {
      m0 = fmaxf(m0, Elem<T>::chunk_max(ldg128_stream(it.p.body + (size_t)ci * 16)));
      any0 = true;
      if (ci + kGroup < nchunk) {
        m1 = fmaxf(m1, Elem<T>::chunk_max(ldg128_stream(it.p.body + (size_t)(ci + kGroup) * 16)));
        any1 = true;
      }
    }
  }

  bool bans = false;  // Sampler::bans_: any bias entry <= -100, in range or not (tools/sampler.h:34)
  for (int i = gt; i < r.NB && r.lists_ok; i += kGroup) bans = bans || a.bias_vals[r.q0 + i] <= -100.0f;
  if (r.touched_on) {
    for (int i = gt; i < a.hash_slots; i += kGroup) {
      hk[i] = kEmpty;
      hi_[i] = 0;
    }
    for (int i = gt; i < kBloomWords; i += kGroup) bloom[i] = 0u;
    __syncthreads();
    auto insert = [&](int32_t t) -> int {  // global id -> slot, -1 when it is not this item's
      if (t < 0 || t >= Vg) return -1;
      const int32_t c = t - a.id_base;
      if (c < it.lo || c >= it.hi) return -1;
      uint32_t h = hash_of(c, a.hash_shift);
      for (int probe = 0; probe < a.hash_slots; ++probe) {
        const uint32_t old = atomicCAS(&hk[h], kEmpty, (uint32_t)c);
        if (old == kEmpty) atomicOr(&bloom[bloom_bit(c) >> 5], 1u << (bloom_bit(c) & 31));
        if (old == kEmpty || old == (uint32_t)c) return (int)h;
        h = (h + 1) & (uint32_t)(a.hash_slots - 1);
      }
      return -1;
    };
    if (r.pen_on) {
      const int32_t nwin = r.prm.repeat_last_n < 0 ? r.H : min(r.H, r.prm.repeat_last_n);  // tools/sampler.h:163
      for (int i = gt; i < r.H; i += kGroup) {
        const int s = insert(a.hist_ids[r.h0 + i]);
        if (s >= 0) atomicAdd(&hi_[s], 1u);
        if (s >= 0 && i >= r.H - nwin) atomicOr(&hi_[s], kInfoWindow);
      }
    }
    for (int i = gt; i < r.NB; i += kGroup) {
      const int s = insert(a.bias_ids[r.q0 + i]);
      if (s >= 0) atomicOr(&hi_[s], a.bias_vals[r.q0 + i] > -100.0f ? kInfoBias : kInfoBan);
    }
  }
  bans = __syncthreads_or(bans) != 0;

  // one more entry for the finish kernel: v is the final (adjusted) logit of column c
  auto supply = [&](float v, int32_t c) {
    const uint32_t ky = key_of(v);
    if (ky == 0u) return;
    const int32_t g = c + a.id_base;
    bool okB = true;
    if (MASKED) okB = ((__ldg(&mrow[g >> 5]) >> (g & 31)) & 1u) && !(bans && v + 0.0f <= ARCS_BANNED);  // tools/sampler.h:118-119
    const int pos = atomicAdd(n_pre, 1);
    w.pre[pos] = (unsigned long long)ky | ((unsigned long long)((uint32_t)g | (okB ? kOkB : 0u)) << 32);
  };
  auto is_touched = [&](int32_t c) -> bool {
    uint32_t h = hash_of(c, a.hash_shift);
    for (int probe = 0; probe < a.hash_slots; ++probe) {
      const uint32_t kx = hk[h];
      if (kx == kEmpty) return false;
      if (kx == (uint32_t)c) return true;
      h = (h + 1) & (uint32_t)(a.hash_slots - 1);
    }
    return false;
  };

  // touched tokens: exact fp32 arithmetic of Sampler::adjusted, a few tokens per thread, their
  // logits fetched together
  int extra = 0;  // touched tokens inside the prefix: they may own a maximum there without counting
  if (r.touched_on) {
    constexpr int R = 4;
    const int32_t c_lo = it.p.body_first, c_hi = it.p.body_first + nchunk * E;
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
        if (ck[x] == kEmpty) continue;
        extra += (int32_t)ck[x] >= c_lo && (int32_t)ck[x] < c_hi;
        float v = raw[x];
        const uint32_t cnt = info[x] & kInfoCount;
        if (info[x] & kInfoBias) {  // :154-155 in list order, duplicates add again
          const int32_t g = (int32_t)ck[x] + a.id_base;
          for (int i = 0; i < r.NB; ++i)
            if (a.bias_ids[r.q0 + i] == g && a.bias_vals[r.q0 + i] > -100.0f) v = __fadd_rn(v, a.bias_vals[r.q0 + i]);
        }
        if (r.pen_on && cnt > 0) {
          if (r.fp_on) v = __fsub_rn(v, __fmul_rn(r.prm.frequency_penalty, (float)cnt));             // :160
          if (r.rp_on && (info[x] & kInfoWindow))
            v = v > 0.0f ? __fdiv_rn(v, r.prm.repeat_penalty) : __fmul_rn(v, r.prm.repeat_penalty);   // :166
          if (r.pp_on) v = __fsub_rn(v, r.prm.presence_penalty);                                      // :171
        }
        if (info[x] & kInfoBan) v = ARCS_BANNED;                                                      // :174
        supply(v, (int32_t)ck[x]);
      }
    }
    if (extra) atomicAdd(n_extra, extra);
  }
  // the scalar elements before the first and after the last 16-byte boundary
  if (gt < it.p.head_n) {
    const int32_t c = it.lo + gt;
    if (!(r.touched_on && is_touched(c))) supply(Elem<T>::load(it.row + c), c);
  }
  if (gt >= 32 && gt - 32 < it.p.tail_n) {
    const int32_t c = it.p.tail_first + gt - 32;
    if (!(r.touched_on && is_touched(c))) supply(Elem<T>::load(it.row + c), c);
  }
  __syncthreads();

  // first threshold: the k-th largest of 256 (or, constrained, 1024) maxima over disjoint pieces
  // of the prefix is a lower bound of the k-th best element; touched tokens inside the prefix
  // may own a maximum without counting, so that many more are skipped
  const int kth = (MASKED ? ARCS_HEAD : r.kB) + *n_extra;
  unsigned long long tau0B = 0ull, tau0A = 0ull;
  if (!MASKED) {
    ptk[gt] = any0 ? key_of(m0) : 0u;
    ptk[kGroup + gt] = any1 ? key_of(m1) : 0u;
    __syncthreads();
    if (kth <= min(nchunk, 2 * kGroup)) tau0B = (unsigned long long)group_kth_key<1>(ptk, 2 * kGroup, kth, psP, gt) << 32;  // keeps ties with it
  } else {
    // constrained rows rank the whole vocabulary's best 512: k-th largest of up to 1024 chunk maxima
    constexpr int kKeys = 2 * kTmpCap;  // ptk and pti lie back to back
    if (kth <= nchunk && nchunk <= kKeys) {
      for (int ci = gt; ci < kKeys; ci += kGroup)
        ptk[ci] = ci < nchunk ? key_of(Elem<T>::chunk_max(ldg128_stream(it.p.body + (size_t)ci * 16))) : 0u;
      __syncthreads();
      tau0A = (unsigned long long)group_kth_key<1>(ptk, kKeys, kth, psP, gt) << 32;  // keeps ties with it
    }
  }
  // ---- the item's block
  if (gt == 0) {
    ItemHdr h;
    h.tau0B = tau0B;
    h.tau0A = tau0A;
    h.K = r.kB;
    h.touched = r.touched_on;
    h.bans = bans;
    h.baseB = (int32_t)(tau0B >> 48);
    h.baseA = (int32_t)(tau0A >> 48);
    h.n_pre = *n_pre;
    h.n_candB = 0;
    h.n_candA = 0;
    h.pad[0] = h.pad[1] = h.pad[2] = h.pad[3] = 0;
    *w.hdr = h;
  }
  if (r.touched_on) {
    for (int i = gt; i < kBloomWords; i += kGroup) w.bloom[i] = bloom[i];
    for (int i = gt; i < a.hash_slots; i += kGroup) w.hkey[i] = hk[i];
  }
}

}  // namespace arcs
