// Exact top-k selection in shared memory over 64-bit (key, ~id) composites: a candidate
// buffer with a rising threshold, pruned by an 8-bit radix select run by the whole CTA
// (synchronised on a named barrier), and the coarse histogram binning the stream kernel uses.
#pragma once
#include "common.cuh"

namespace arcs {

constexpr int kTmpCap = ARCS_HEAD;  // most entries a prune keeps (the constrained head select keeps 512)
constexpr int kGroup = 128;         // threads of the small per-item / per-row CTAs (prepare and finish kernels)

// named-barrier synchronisation of G threads (BAR: barrier number)
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

// Keep exactly the k best entries of the buffer. Called by all G threads of the CTA (gt = thread
// index) with the buffer quiescent. Radix
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


// A lower bound of the kth largest (1-based) of 32 * PER keys held PER to a lane, found by ONE
// warp with a search on the keys' upper 16 bits, two bits a round (bf16 resolution; exact for
// bf16 data): the largest t with at least kth keys >= t. No shared-memory traffic.
template <int PER>
__device__ __forceinline__ uint32_t warp_kth16_regs(const uint32_t (&k)[PER], int kth) {
  uint32_t t = 0;
#pragma unroll 1
  for (int bit = 14; bit >= 0; bit -= 2) {
    const uint32_t c1 = (t | (1u << bit)) << 16, c2 = (t | (2u << bit)) << 16, c3 = (t | (3u << bit)) << 16;
    int n1 = 0, n2 = 0, n3 = 0;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      n1 += k[i] >= c1;
      n2 += k[i] >= c2;
      n3 += k[i] >= c3;
    }
    // three counts (each at most 32 * PER <= 1024) in one word, one reduction
    const uint32_t all = __reduce_add_sync(0xFFFFFFFFu, (uint32_t)n1 | ((uint32_t)n2 << 11) | ((uint32_t)n3 << 22));
    const int a1 = (int)(all & 0x7FFu), a2 = (int)((all >> 11) & 0x7FFu), a3 = (int)(all >> 22);
    t |= (a3 >= kth ? 3u : a2 >= kth ? 2u : a1 >= kth ? 1u : 0u) << bit;
  }
  return t << 16;
}
// The kth largest (1-based, kth <= 32) of one key per lane, ties counted: the largest key t with at
// least kth lanes holding a key >= t. A handful of warp-wide maxima, no search over bits.
__device__ __forceinline__ uint32_t warp_kth_lane(uint32_t key, int kth) {
  uint32_t t = 0u;
  int taken = 0;
  bool in = true;
#pragma unroll 1
  while (taken < kth) {
    t = __reduce_max_sync(0xFFFFFFFFu, in ? key : 0u);
    if (t == 0u) break;  // fewer than kth keys above zero
    const bool hit = in && key == t;
    taken += __popc(__ballot_sync(0xFFFFFFFFu, hit));
    in = in && !hit;
  }
  return taken >= kth ? t : 0u;
}
// the same with the keys in shared memory (32 * PER of them, 16-byte aligned)
template <int PER>
__device__ __forceinline__ uint32_t warp_kth16(const uint32_t* keys, int kth) {
  const int lane = threadIdx.x & 31;
  uint32_t k[PER];
#pragma unroll
  for (int i = 0; i < PER / 4; ++i) {
    const uint4 q = reinterpret_cast<const uint4*>(keys)[i * 32 + lane];
    k[4 * i] = q.x;
    k[4 * i + 1] = q.y;
    k[4 * i + 2] = q.z;
    k[4 * i + 3] = q.w;
  }
  return warp_kth16_regs<PER>(k, kth);
}

// Bin of a key in an item's coarse histogram: the key's upper 16 bits (bf16 resolution) relative
// to `base`, the last bin taking everything above.
__device__ __forceinline__ uint32_t coarse_bin(uint32_t key, uint32_t base) {
  const uint32_t b = (key >> 16) - base;
  return b < 255u ? b : 255u;
}

}  // namespace arcs
