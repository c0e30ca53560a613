// Vocabulary-wide constraint mask: every token's byte string is walked through a byte-level
// automaton from a start state; the result is one allowed-token bit per token, packed.
#include "common.cuh"
#include "plan.h"

#include <algorithm>

namespace arcs {

constexpr int kMaskThreads = 256;
constexpr int kMaskInRegs = 16;  // bytes of a token held in registers (longer tokens read the rest from memory)

// One thread per token, all start states in turn: the token's offsets and bytes are fetched once
// and walked from every start state. The table is read through the read-only cache: its lookups
// are random 2-byte reads, one cache sector a lane, and that traffic bounds the kernel (a copy of
// the table in shared memory was measured slower: rows 512 bytes apart put the bytes of ordinary
// text on a few banks).
__global__ void __launch_bounds__(kMaskThreads) dfa_mask_kernel(const uint16_t* __restrict__ table, int32_t n_table_states,
                                                                int32_t dead, const int32_t* __restrict__ states, int32_t n_states,
                                                                const uint32_t* __restrict__ byte_off,
                                                                const uint8_t* __restrict__ bytes,
                                                                const uint8_t* __restrict__ special, int32_t special_ok,
                                                                int32_t V, uint32_t* __restrict__ out, int64_t out_stride) {
  auto next = [&](int32_t s, uint32_t c) -> int32_t { return (int32_t)__ldg(&table[(size_t)s * 256 + c]); };
  // (a state number outside the table, which only a malformed table holds, counts as dead: no lookup leaves the table)
  auto alive = [&](int32_t s) { return s != dead && (uint32_t)s < (uint32_t)n_table_states; };
  for (int32_t t0 = (int32_t)blockIdx.x * kMaskThreads; t0 < V; t0 += (int32_t)gridDim.x * kMaskThreads) {
    const int32_t t = t0 + (int32_t)threadIdx.x;
    uint32_t b0 = 0, len = 0;
    bool piece_ok = false;
    uint8_t by[kMaskInRegs];
    if (t < V) {
      b0 = __ldg(&byte_off[t]);
      const uint32_t b1 = __ldg(&byte_off[t + 1]);
      len = b1 > b0 ? b1 - b0 : 0u;
      // an empty piece is never allowed; a control token only where the caller says so
      piece_ok = len > 0 && !(special && __ldg(&special[t]) && !special_ok);
    }
#pragma unroll
    for (int i = 0; i < kMaskInRegs; ++i) by[i] = piece_ok && (uint32_t)i < len ? __ldg(&bytes[b0 + i]) : (uint8_t)0;
    for (int32_t si = 0; si < n_states; ++si) {
      const int32_t start = __ldg(&states[si]);
      int32_t s = start;
      bool ok = piece_ok && alive(start);
#pragma unroll
      for (int i = 0; i < kMaskInRegs; ++i)
        if (ok && (uint32_t)i < len) {
          s = next(s, by[i]);
          ok = alive(s);
        }
      for (uint32_t i = kMaskInRegs; ok && i < len; ++i) {
        s = next(s, __ldg(&bytes[b0 + i]));
        ok = alive(s);
      }
      const unsigned w = __ballot_sync(0xFFFFFFFFu, ok);
      if ((threadIdx.x & 31) == 0 && t < V) out[(size_t)si * out_stride + (t >> 5)] = w;
    }
  }
}

}  // namespace arcs

extern "C" int arcs_dfa_mask(const uint16_t* table, int32_t n_table_states, int32_t dead, const int32_t* states,
                             int32_t n_states, const uint32_t* byte_off, const uint8_t* bytes,
                             const uint8_t* special, int32_t special_ok, int32_t V, uint32_t* out,
                             int64_t out_stride, void* stream) {
  using namespace arcs;
  if (int inj = fault_injected()) return inj;
  if (!table || !states || !byte_off || !bytes || !out || n_table_states <= 0 || n_states <= 0 || V <= 0 ||
      n_states > 65535 || out_stride < (V + 31) / 32)
    return set_error(ARCS_ERR_ARG, "dfa_mask: bad argument");
  const unsigned blocks = (unsigned)((V + kMaskThreads - 1) / kMaskThreads);
  dfa_mask_kernel<<<std::min(blocks, (unsigned)kSmCount * 8u), kMaskThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      table, n_table_states, dead, states, n_states, byte_off, bytes, special, special_ok, V, out, out_stride);
  return check_launch("dfa_mask");
}
