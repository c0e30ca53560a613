// Exact top-k selection in shared memory over 64-bit (key, ~id) composites: a candidate
// buffer with a rising threshold, pruned by an 8-bit radix select. Two forms: one run by a
// single warp on a buffer only that warp touches, one run by a helper group of warps that
// synchronises on a named barrier (the other warps of the CTA keep streaming meanwhile).
#pragma once
#include "common.cuh"

namespace arcs {

constexpr int kTmpCap = ARCS_HEAD;  // most entries a prune keeps (the constrained head select keeps 512)
constexpr int kGroup = 128;         // threads of each helper group (one prepares items, one finishes them)

// named-barrier synchronisation of one helper group (BAR: barrier number, kGroup threads)
template <int BAR, int G = kGroup>
__device__ __forceinline__ void group_sync() { asm volatile("bar.sync %0, %1;" ::"n"(BAR), "n"(G) : "memory"); }
template <int BAR, int G = kGroup>
__device__ __forceinline__ bool group_sync_or(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, %2, %3, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred), "n"(BAR), "n"(G)
      : "memory");
  return r != 0;
}

// One running selection of the k best entries seen so far under (value desc, id asc), i.e. the
// k largest composites. Invariant: every entry seen whose composite exceeds *tau is in the
// buffer; *tau is 0 until something has been dropped, then a composite no kept entry is below.
struct Sel {
  uint32_t* key;             // [cap]
  int32_t* id;               // [cap]
  int* cnt;                  // entries in the buffer (owner's copy may live in a register)
  unsigned long long* tau;   // exclusive threshold composite
  int k, trig, cap;
};

struct PruneScratch {
  uint32_t* hist;            // [2][256]
  uint32_t* tk;              // [kTmpCap]
  int32_t* ti;               // [kTmpCap]
  int* misc;                 // [8]: digit, remaining, exact, out count
  unsigned long long* m64;   // [1]: smallest composite kept
};

// Group-wide append (every lane of a warp of the group calls it together); lanes with p set
// store (key, id). Sets `hot` when the buffer has grown past the prune trigger.
__device__ __forceinline__ void sel_push(const Sel& s, bool p, uint32_t key, int32_t id, bool& hot, int32_t* status) {
  const unsigned b = __ballot_sync(0xFFFFFFFFu, p);
  if (b == 0) return;
  const int lane = threadIdx.x & 31, leader = __ffs(b) - 1;
  int base = 0;
  if (lane == leader) base = (int)sm_atomic_add(s.cnt, (uint32_t)__popc(b));
  base = __shfl_sync(0xFFFFFFFFu, base, leader);
  if (p) {
    const int pos = base + __popc(b & ((1u << lane) - 1u));
    if (pos < s.cap) {
      s.key[pos] = key;
      s.id[pos] = id;
    } else {
      raise_status(status, ARCS_ERR_ARG);  // cannot happen: cap >= trig + entries per round
    }
    hot = hot || pos + 1 > s.trig;
  }
}

// Which of the 256 bins holds the `krem`-th entry counted from the top bin down. Called by one
// full warp; lane l owns bins [8l, 8l+8). Returns through all lanes: the bin, the rank wanted
// inside that bin, and whether the bin is taken whole.
__device__ __forceinline__ void find_bin(const uint32_t* h, int krem, int& digit, int& krem_out, bool& exact) {
  const int lane = threadIdx.x & 31;
  uint32_t loc[8], sum = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    loc[j] = h[8 * lane + j];
    sum += loc[j];
  }
  uint32_t incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_down_sync(0xFFFFFFFFu, incl, o);
    if (lane + o < 32) incl += t;
  }
  uint32_t run = incl - sum;  // entries in bins above this lane's
  int d = -1, kr = 0;
  bool ex = false;
#pragma unroll
  for (int j = 7; j >= 0; --j) {
    if (run < (uint32_t)krem && (uint32_t)krem <= run + loc[j]) {
      d = 8 * lane + j;
      kr = krem - (int)run;
      ex = loc[j] == (uint32_t)kr;
    }
    run += loc[j];
  }
  const unsigned fb = __ballot_sync(0xFFFFFFFFu, d >= 0);
  if (fb == 0) {  // fewer than krem entries in all bins (not reachable): take everything
    digit = 0;
    krem_out = krem;
    exact = true;
    return;
  }
  const int src = __ffs(fb) - 1;
  digit = __shfl_sync(0xFFFFFFFFu, d, src);
  krem_out = __shfl_sync(0xFFFFFFFFu, kr, src);
  exact = __shfl_sync(0xFFFFFFFFu, (int)ex, src) != 0;
}

// Keep exactly the k best entries of the buffer. Called by all kGroup threads of the
// finishing group (gt = thread index inside the group) with the buffer quiescent. Radix
// select, most significant byte first, over the composite (key << 32 | ~id): composites are
// unique, so the k-th is found exactly, ties included.
template <int BAR, int G = kGroup>
__device__ __noinline__ void sel_prune(const Sel& s, int k, const PruneScratch& ps, int gt) {
  const int n = min(*s.cnt, s.cap);
  if (n <= k) return;
  for (int i = gt; i < 512; i += G) ps.hist[i] = 0;
  if (gt == 0) {
    ps.misc[3] = 0;
    *ps.m64 = 0xFFFFFFFFFFFFFFFFull;
  }
  group_sync<BAR, G>();
  uint64_t prefix = 0, mask = 0;
  int krem = k;
  for (int pass = 0; pass < 8; ++pass) {
    const int shift = 56 - 8 * pass;
    uint32_t* h = ps.hist + (pass & 1) * 256;
    for (int i = gt; i < n; i += G) {
      const uint64_t c = comp_of(s.key[i], s.id[i]);
      if ((c & mask) == prefix) sm_red_add(&h[(uint32_t)(c >> shift) & 255u], 1u);
    }
    for (int i = gt; i < 256; i += G) ps.hist[((pass + 1) & 1) * 256 + i] = 0;
    group_sync<BAR, G>();
    if (gt < 32) {
      int d, kr;
      bool ex;
      find_bin(h, krem, d, kr, ex);
      if (gt == 0) {
        ps.misc[0] = d;
        ps.misc[1] = kr;
        ps.misc[2] = ex;
      }
    }
    group_sync<BAR, G>();
    const int d = ps.misc[0];
    krem = ps.misc[1];
    const bool exact = ps.misc[2] != 0;
    prefix |= (uint64_t)d << shift;
    mask |= 0xFFull << shift;
    if (exact) break;
  }
  for (int i = gt; i < n; i += G) {
    const uint32_t ky = s.key[i];
    const uint64_t c = comp_of(ky, s.id[i]);
    if ((c & mask) >= prefix) {
      const int pos = (int)sm_atomic_add(&ps.misc[3], 1u);
      if (pos < kTmpCap) {
        ps.tk[pos] = ky;
        ps.ti[pos] = s.id[i];
      }
      sm_red_min_u64(ps.m64, (unsigned long long)c);
    }
  }
  group_sync<BAR, G>();
  const int m = min(ps.misc[3], kTmpCap);
  for (int i = gt; i < m; i += G) {
    s.key[i] = ps.tk[i];
    s.id[i] = ps.ti[i];
  }
  if (gt == 0) {
    *s.cnt = m;
    *s.tau = *ps.m64 - 1ull;  // exclusive: the smallest kept composite itself still passes
  }
  group_sync<BAR, G>();
}


// The kth largest (1-based) of the n keys in keys[] (n a multiple of kGroup, at most 8 * kGroup),
// found by the whole group with a 4-pass radix select on the 32-bit keys. Every thread returns
// the same value.
template <int BAR>
__device__ __noinline__ uint32_t group_kth_key(const uint32_t* keys, int n, int kth, const PruneScratch& ps, int gt) {
  uint32_t prefix = 0, mask = 0;
  int krem = kth;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = gt; i < 256; i += kGroup) ps.hist[i] = 0;
    group_sync<BAR>();
    for (int i = gt; i < n; i += kGroup) {
      const uint32_t my = keys[i];
      if ((my & mask) == prefix) sm_red_add(&ps.hist[(my >> shift) & 255u], 1u);
    }
    group_sync<BAR>();
    if (gt < 32) {
      int d, kr;
      bool ex;
      find_bin(ps.hist, krem, d, kr, ex);
      if (gt == 0) {
        ps.misc[0] = d;
        ps.misc[1] = kr;
      }
    }
    group_sync<BAR>();
    prefix |= (uint32_t)ps.misc[0] << shift;
    mask |= 0xFFu << shift;
    krem = ps.misc[1];
  }
  group_sync<BAR>();
  return prefix;
}

// The same selection run by ONE warp on a buffer only that warp touches (the examiner warp
// while a row streams). n: entries in the buffer; returns the new count and publishes *s.tau.
// hist: 256 words, tk / ti: kTmpCap entries, all private to the calling warp.
__device__ __noinline__ int sel_prune_warp(const Sel& s, int n, int k, uint32_t* hist, uint32_t* tk, int32_t* ti) {
  const int lane = threadIdx.x & 31;
  if (n <= k) return n;
  uint64_t prefix = 0, mask = 0;
  int krem = k;
  for (int pass = 0; pass < 8; ++pass) {
    const int shift = 56 - 8 * pass;
#pragma unroll
    for (int j = 0; j < 8; ++j) hist[j * 32 + lane] = 0;
    __syncwarp();
    for (int i = lane; i < n; i += 32) {
      const uint64_t c = comp_of(s.key[i], s.id[i]);
      if ((c & mask) == prefix) sm_red_add(&hist[(uint32_t)(c >> shift) & 255u], 1u);
    }
    __syncwarp();
    int d, kr;
    bool ex;
    find_bin(hist, krem, d, kr, ex);
    krem = kr;
    prefix |= (uint64_t)d << shift;
    mask |= 0xFFull << shift;
    __syncwarp();
    if (ex) break;
  }
  int out = 0;
  uint64_t cmin = 0xFFFFFFFFFFFFFFFFull;
  for (int i0 = 0; i0 < n; i0 += 32) {
    const int i = i0 + lane;
    uint32_t ky = 0;
    int32_t id = 0;
    bool keep = false;
    if (i < n) {
      ky = s.key[i];
      id = s.id[i];
      const uint64_t c = comp_of(ky, id);
      keep = (c & mask) >= prefix;
      if (keep && c < cmin) cmin = c;
    }
    const unsigned b = __ballot_sync(0xFFFFFFFFu, keep);
    const int pos = out + __popc(b & ((1u << lane) - 1u));
    if (keep && pos < kTmpCap) {
      tk[pos] = ky;
      ti[pos] = id;
    }
    out += __popc(b);
  }
  out = min(out, kTmpCap);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const uint64_t w = __shfl_xor_sync(0xFFFFFFFFu, cmin, o);
    cmin = w < cmin ? w : cmin;
  }
  __syncwarp();
  for (int i = lane; i < out; i += 32) {
    s.key[i] = tk[i];
    s.id[i] = ti[i];
  }
  if (lane == 0) sm_red_max_u64(s.tau, cmin - 1ull);  // exclusive threshold; never lowered (another warp raises it too)
  __syncwarp();
  return out;
}


// Bin of a key in the coarse histogram an owner warp keeps beside its buffer: the key's upper
// 16 bits (bf16 resolution) relative to `base`, the last bin taking everything above.
__device__ __forceinline__ uint32_t coarse_bin(uint32_t key, uint32_t base) {
  const uint32_t b = (key >> 16) - base;
  return b < 255u ? b : 255u;
}

// Cheap threshold raise for a buffer one warp owns. hist[256] counts the buffer's entries by
// coarse_bin. The bin holding the k-th best entry is found, its lower edge becomes the
// threshold (so every entry of that bin stays: at least k remain) and the entries below are
// dropped in place. Returns the new count; n > k on entry.
__device__ __forceinline__ int sel_raise_warp(const Sel& s, int n, int k, uint32_t* hist, uint32_t base) {
  const int lane = threadIdx.x & 31;
  int d, kr;
  bool ex;
  find_bin(hist, k, d, kr, ex);
  if (d <= 0) return n;  // the k-th best lies in the lowest bin: nothing can be dropped this way
  const uint64_t tc = (uint64_t)((base + (uint32_t)d) << 16) << 32;  // comp > tc  <=>  key >= edge of bin d
  int out = 0;
  for (int i0 = 0; i0 < n; i0 += 32) {
    const int i = i0 + lane;
    uint32_t ky = 0;
    int32_t id = 0;
    bool keep = false;
    if (i < n) {
      ky = s.key[i];
      id = s.id[i];
      keep = comp_of(ky, id) > tc;
    }
    const unsigned b = __ballot_sync(0xFFFFFFFFu, keep);  // (every lane has read its entry before any write below)
    if (keep) {
      const int pos = out + __popc(b & ((1u << lane) - 1u));
      s.key[pos] = ky;
      s.id[pos] = id;
    }
    out += __popc(b);
    __syncwarp();
  }
#pragma unroll
  for (int j = 0; j < 8; ++j)
    if (j * 32 + lane < d) hist[j * 32 + lane] = 0;
  if (lane == 0 && tc > *s.tau) *reinterpret_cast<volatile unsigned long long*>(s.tau) = tc;
  __syncwarp();
  return out;
}

// rebuild the coarse histogram of a buffer after its entries changed wholesale
__device__ __forceinline__ void sel_rehist_warp(const Sel& s, int n, uint32_t* hist, uint32_t base) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int j = 0; j < 8; ++j) hist[j * 32 + lane] = 0;
  __syncwarp();
  for (int i = lane; i < n; i += 32) sm_red_add(&hist[coarse_bin(s.key[i], base)], 1u);
  __syncwarp();
}

}  // namespace arcs
