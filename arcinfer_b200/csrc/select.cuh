// Exact streaming top-k selection in shared memory: a candidate buffer with a rising
// threshold, pruned by an 8-bit radix select over 64-bit (key, ~id) composites.
#pragma once
#include "common.cuh"

namespace arcs {

constexpr int kTmpCap = ARCS_HEAD;  // most entries a prune keeps (the constrained head select keeps 512)

// One running selection of the k best (value desc, id asc) entries seen so far.
// Invariants between prunes: every entry seen with key >= *tau_key is in the buffer;
// *tau_key is 0 (nothing dropped yet) or 1 + the smallest key kept by the last prune.
struct Sel {
  uint32_t* key;      // [cap]
  int32_t* id;        // [cap]
  int* cnt;           // entries in the buffer
  uint32_t* tau_key;  // inclusive threshold for elements that arrive in increasing id order
  int k, trig, cap;
};

struct PruneScratch {
  uint32_t* hist;  // [2][256]
  uint32_t* tk;    // [kTmpCap]
  int32_t* ti;     // [kTmpCap]
  int* misc;       // [8]: digit, remaining, exact, out count, min key kept
};

// Warp-wide append: every lane of the warp calls it; lanes with p set store (key, id).
// Sets `hot` when the buffer has grown past the prune trigger.
__device__ __forceinline__ void sel_push(const Sel& s, bool p, uint32_t key, int32_t id, bool& hot, int32_t* status) {
  const unsigned b = __ballot_sync(0xFFFFFFFFu, p);
  if (b == 0) return;
  const int lane = threadIdx.x & 31, leader = __ffs(b) - 1;
  int base = 0;
  if (lane == leader) base = atomicAdd(s.cnt, __popc(b));
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

// Keep exactly the k best entries of the buffer. Called by all threads of the CTA with the
// buffer quiescent. Radix select, most significant byte first, over the composite
// (key << 32 | ~id): composites are unique, so the k-th is found exactly, ties included.
__device__ __forceinline__ void sel_prune(const Sel& s, int k, const PruneScratch& ps) {
  const int tid = threadIdx.x;
  const int n = min(*s.cnt, s.cap);
  if (n <= k) return;
  ps.hist[tid] = 0;
  ps.hist[256 + tid] = 0;
  if (tid == 0) {
    ps.misc[3] = 0;
    ps.misc[4] = (int)0xFFFFFFFFu;
  }
  __syncthreads();
  uint64_t prefix = 0, mask = 0;
  int krem = k;
  for (int pass = 0; pass < 8; ++pass) {
    const int shift = 56 - 8 * pass;
    uint32_t* h = ps.hist + (pass & 1) * 256;
    for (int i = tid; i < n; i += kThreads) {
      const uint64_t c = comp_of(s.key[i], s.id[i]);
      if ((c & mask) == prefix) atomicAdd(&h[(uint32_t)(c >> shift) & 255u], 1u);
    }
    ps.hist[((pass + 1) & 1) * 256 + tid] = 0;
    __syncthreads();
    if (tid < 32) {
      uint32_t loc[8], sum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        loc[j] = h[8 * tid + j];
        sum += loc[j];
      }
      uint32_t incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_down_sync(0xFFFFFFFFu, incl, o);
        if (tid + o < 32) incl += t;
      }
      uint32_t run = incl - sum;  // entries in bins above this lane's
      if (tid == 0) {  // defaults, overwritten by the lane that finds the bin
        ps.misc[0] = 0;
        ps.misc[1] = krem;
        ps.misc[2] = 1;
      }
      __syncwarp();
#pragma unroll
      for (int j = 7; j >= 0; --j) {
        if (run < (uint32_t)krem && (uint32_t)krem <= run + loc[j]) {
          ps.misc[0] = 8 * tid + j;
          ps.misc[1] = krem - (int)run;
          ps.misc[2] = loc[j] == (uint32_t)krem - run;
        }
        run += loc[j];
      }
    }
    __syncthreads();
    const int d = ps.misc[0];
    krem = ps.misc[1];
    const bool exact = ps.misc[2] != 0;
    prefix |= (uint64_t)d << shift;
    mask |= 0xFFull << shift;
    if (exact) break;
  }
  for (int i = tid; i < n; i += kThreads) {
    const uint32_t ky = s.key[i];
    const uint64_t c = comp_of(ky, s.id[i]);
    if ((c & mask) >= prefix) {
      const int pos = atomicAdd(&ps.misc[3], 1);
      if (pos < kTmpCap) {
        ps.tk[pos] = ky;
        ps.ti[pos] = s.id[i];
      }
      atomicMin(reinterpret_cast<unsigned int*>(&ps.misc[4]), ky);
    }
  }
  __syncthreads();
  const int m = min(ps.misc[3], kTmpCap);
  for (int i = tid; i < m; i += kThreads) {
    s.key[i] = ps.tk[i];
    s.id[i] = ps.ti[i];
  }
  if (tid == 0) {
    *s.cnt = m;
    const uint32_t kmin = (uint32_t)ps.misc[4];
    *s.tau_key = kmin == 0xFFFFFFFFu ? kmin : kmin + 1u;
  }
  __syncthreads();
}

// Sort the n (<= kThreads * 2) buffer entries best first into (out_val, out_id) by counting ranks.
__device__ __forceinline__ void sel_sort(const Sel& s, int n, float* out_val, int32_t* out_id) {
  for (int i = threadIdx.x; i < n; i += kThreads) {
    const uint32_t ky = s.key[i];
    const int32_t id = s.id[i];
    const uint64_t c = comp_of(ky, id);
    int rank = 0;
    for (int j = 0; j < n; ++j) rank += comp_of(s.key[j], s.id[j]) > c;
    out_val[rank] = value_of(ky);
    out_id[rank] = id;
  }
}

}  // namespace arcs
