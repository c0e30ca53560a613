// Vocabulary-wide constraint mask: every token's byte string is walked through a byte-level
// automaton from a start state; the result is one allowed-token bit per token, packed.
#include "common.cuh"
#include "plan.h"

namespace arcs {

__global__ void __launch_bounds__(256) dfa_mask_kernel(const uint16_t* __restrict__ table, int32_t dead,
                                                       const int32_t* __restrict__ states,
                                                       const uint32_t* __restrict__ byte_off,
                                                       const uint8_t* __restrict__ bytes,
                                                       const uint8_t* __restrict__ special, int32_t special_ok,
                                                       int32_t V, uint32_t* __restrict__ out, int64_t out_stride) {
  const int32_t t = blockIdx.x * 256 + threadIdx.x;
  const int32_t start = states[blockIdx.y];
  bool ok = false;
  if (t < V) {
    const uint32_t b0 = byte_off[t], b1 = byte_off[t + 1];
    // an empty piece is never allowed; a control token only where the caller says so
    ok = b1 > b0 && start != dead && !(special && special[t] && !special_ok);
    int32_t s = start;
    for (uint32_t i = b0; ok && i < b1; ++i) {
      s = __ldg(&table[(size_t)s * 256 + __ldg(&bytes[i])]);
      ok = s != dead;
    }
    ok = ok && s != dead;
  }
  const unsigned w = __ballot_sync(0xFFFFFFFFu, ok);
  if ((threadIdx.x & 31) == 0 && t < V) out[(size_t)blockIdx.y * out_stride + (t >> 5)] = w;
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
  const dim3 grid((unsigned)((V + 255) / 256), (unsigned)n_states);
  dfa_mask_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(table, dead, states, byte_off, bytes, special,
                                                                      special_ok, V, out, out_stride);
  return check_launch("dfa_mask");
}
