// Row-segment streaming through a ring of shared-memory tiles filled by 1-D bulk copies.
#pragma once
#include "common.cuh"

namespace arcs {

// How one CTA walks the elements [lo, hi) of a row: a few scalar elements up to the first
// 16-byte boundary, then whole 16-byte chunks fetched by bulk copies in tiles of kTileBytes,
// then the scalar remainder. Works for any row alignment (rows need only element alignment).
struct SegPlan {
  const char* body;   // first 16-byte aligned address of the segment
  int32_t lo, hi;     // element range of the segment
  int32_t head_n;     // scalar elements before the body
  int32_t body_first; // element index of the first body element
  int32_t body_bytes; // multiple of 16
  int32_t tail_first, tail_n;
  int32_t tiles;
};

template <typename T>
__device__ __forceinline__ SegPlan make_plan(const T* row, int32_t lo, int32_t hi) {
  SegPlan p;
  p.lo = lo;
  p.hi = hi;
  const uintptr_t a_lo = reinterpret_cast<uintptr_t>(row + lo), a_hi = reinterpret_cast<uintptr_t>(row + hi);
  uintptr_t a0 = (a_lo + 15) & ~(uintptr_t)15, a1 = a_hi & ~(uintptr_t)15;
  if (a0 > a_hi) a0 = a_hi;
  if (a1 < a0) a1 = a0;
  p.body = reinterpret_cast<const char*>(a0);
  p.head_n = (int32_t)((a0 - a_lo) / sizeof(T));
  p.body_first = lo + p.head_n;
  p.body_bytes = (int32_t)(a1 - a0);
  p.tail_first = p.body_first + p.body_bytes / (int32_t)sizeof(T);
  p.tail_n = hi - p.tail_first;
  p.tiles = (p.body_bytes + kTileBytes - 1) / kTileBytes;
  return p;
}

__device__ __forceinline__ uint32_t tile_bytes(const SegPlan& p, int t) {
  const int32_t rem = p.body_bytes - t * kTileBytes;
  return (uint32_t)(rem < kTileBytes ? rem : kTileBytes);
}
// called by one thread: arm the slot's barrier and start the copy of tile t into it
__device__ __forceinline__ void issue_tile(const SegPlan& p, int t, char* stage, uint64_t* bars) {
  const int slot = t % kStages;
  const uint32_t n = tile_bytes(p, t);
  mbar_expect_tx(&bars[slot], n);
  bulk_load(stage + (size_t)slot * kTileBytes, p.body + (size_t)t * kTileBytes, n, &bars[slot]);
}

// After a failed wait: give the copies still in flight a bounded chance to land before the
// CTA's shared memory is released.
__device__ __forceinline__ void drain_tiles(const SegPlan& p, int from_tile, uint64_t* bars) {
  const int last = (from_tile + kStages < p.tiles) ? from_tile + kStages : p.tiles;
  for (int t = from_tile; t < last; ++t) mbar_wait(&bars[t % kStages], (uint32_t)((t / kStages) & 1));
}

}  // namespace arcs
