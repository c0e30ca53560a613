// Batched first-maximum (greedy selection), optional (max, sum exp) per row, and the greedy
// draft-acceptance count per slot. One launch: every CTA streams one segment of one row, folds
// its (value, id) into a 64-bit atomic max per row, and the CTA that finishes last decodes the
// rows and walks the slots.
#include <mutex>

#include "plan.h"
#include "stream.cuh"

namespace arcs {

struct ArgmaxDev {
  const void* logits;
  int64_t row_stride;
  int32_t R, V, nseg, seg_len;
  int32_t* argmax;
  float* max_sumexp;
  int32_t slots;
  const int32_t* row_off;
  const int32_t* draft;
  const int32_t* draft_off;
  int32_t* accepted;
  int32_t* next;
  unsigned int* ws_done;          // one counter
  unsigned long long* ws_best;    // [R] composite (key << 32 | ~id), 0 between launches
  float2* ws_part;                // [R][nseg] partial (max, sum exp)
  int32_t* status;
};

// online (max, sum exp(x - max)) update with one value
__device__ __forceinline__ void lse_add(float& m, float& s, float x) {
  if (x > m) {
    s = s * expf(m - x) + 1.0f;  // expf(-inf) = 0 covers the first value
    m = x;
  } else if (x == x && m > -INFINITY) {
    s += expf(x - m);
  }
}
__device__ __forceinline__ void lse_merge(float& m, float& s, float m2, float s2) {
  if (s2 == 0.0f) return;
  if (s == 0.0f) { m = m2; s = s2; return; }
  if (m2 > m) { s = s * expf(m - m2) + s2; m = m2; }
  else s += s2 * expf(m2 - m);
}

template <typename T, bool LSE>
__global__ void __launch_bounds__(kThreads) argmax_kernel(const ArgmaxDev a) {
  extern __shared__ __align__(128) char stage[];  // kStages * kTileBytes
  __shared__ __align__(8) uint64_t bars[kStages];
  __shared__ unsigned long long red_c[kThreads / 32];
  __shared__ float red_m[kThreads / 32], red_s[kThreads / 32];
  __shared__ int s_flag;

  constexpr int E = Elem<T>::kPerChunk;
  const int tid = threadIdx.x, seg = blockIdx.x % a.nseg, r = blockIdx.x / a.nseg;
  const T* row = reinterpret_cast<const T*>(a.logits) + (size_t)r * a.row_stride;
  const int32_t lo = seg * a.seg_len, hi = min(a.V, lo + a.seg_len);
  const SegPlan p = make_plan(row, lo, hi);

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) mbar_init(&bars[i], 1);
    mbar_init_fence();
    s_flag = 0;
  }
  __syncthreads();
  if (tid == 0)
    for (int t = 0; t < p.tiles && t < kStages; ++t) issue_tile(p, t, stage, bars);

  float bv = -INFINITY;   // best value so far in this thread; strict > keeps the lowest id
  int32_t bi = -1;
  float lm = -INFINITY, ls = 0.0f;

  auto scalar = [&](int32_t id) {
    const float v = Elem<T>::load(row + id);
    if (v > bv || (bi < 0 && v == v)) { bv = v; bi = id; }
    if (LSE) lse_add(lm, ls, v);
  };
  if (tid < p.head_n) scalar(lo + tid);

  bool failed = false;
  for (int t = 0; t < p.tiles; ++t) {
    const int slot = t % kStages;
    if (!mbar_wait(&bars[slot], (uint32_t)((t / kStages) & 1))) failed = true;
    const uint32_t nbytes = tile_bytes(p, t);
    constexpr int kChunks = kTileBytes / 16 / kThreads;
    uint4 q[kChunks];
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
      const uint32_t off = (uint32_t)(j * kThreads + tid) * 16u;
      q[j] = off < nbytes && !failed ? lds128(stage + (size_t)slot * kTileBytes + off) : make_uint4(0, 0, 0, 0);
    }
    // every thread has taken its chunks: the slot can be refilled
    if (__syncthreads_or(failed)) {
      // A bounded wait ran out: the status word marks the call's results invalid. The CTA still
      // takes part in the count below, so that the last CTA leaves the scratch clean for the next call.
      if (tid == 0) {
        raise_status(a.status, ARCS_ERR_TIMEOUT);
        drain_tiles(p, t, bars);
      }
      __syncthreads();
      break;
    }
    if (tid == 0 && t + kStages < p.tiles) issue_tile(p, t + kStages, stage, bars);
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {  // a thread's chunks come in increasing id order
      const uint32_t off = (uint32_t)(j * kThreads + tid) * 16u;
      if (off >= nbytes) continue;
      const float m = Elem<T>::chunk_max(q[j]);
      if (m > bv || bi < 0) {
        const int32_t id0 = p.body_first + (int32_t)(((uint32_t)t * kTileBytes + off) / sizeof(T));
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float v = Elem<T>::get(q[j], e);
          if (v > bv || (bi < 0 && v == v)) { bv = v; bi = id0 + e; }
        }
      }
      if (LSE) {
        if (m > lm) { ls *= expf(lm - m); lm = m; }
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float v = Elem<T>::get(q[j], e);
          if (v == v && lm > -INFINITY) ls += expf(v - lm);
        }
      }
    }
  }
  if (tid < p.tail_n) scalar(p.tail_first + tid);

  // CTA reduction: composite max; lowest id wins among equal values
  uint64_t c = bi >= 0 ? comp_of(key_of(bv), bi) : 0ull;
  c = warp_max_u64(c);
  if (LSE) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xFFFFFFFFu, lm, o), s2 = __shfl_xor_sync(0xFFFFFFFFu, ls, o);
      lse_merge(lm, ls, m2, s2);
    }
  }
  if ((tid & 31) == 0) {
    red_c[tid >> 5] = c;
    if (LSE) { red_m[tid >> 5] = lm; red_s[tid >> 5] = ls; }
  }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < kThreads / 32; ++w) {
      c = red_c[w] > c ? red_c[w] : c;
      if (LSE) lse_merge(lm, ls, red_m[w], red_s[w]);
    }
    if (c) atomicMax(&a.ws_best[r], (unsigned long long)c);
    if (LSE) a.ws_part[(size_t)r * a.nseg + seg] = make_float2(lm, ls);
    __threadfence();
    const unsigned int total = (unsigned int)a.nseg * (unsigned int)a.R;
    s_flag = atomicAdd(a.ws_done, 1u) == total - 1u;
  }
  __syncthreads();
  if (!s_flag) return;

  // ---- last CTA of the launch: decode rows, reset the scratch for the next launch
  __threadfence();
  for (int i = tid; i < a.R; i += kThreads) {
    const unsigned long long b = __ldcg(&a.ws_best[i]);
    a.argmax[i] = b ? comp_id(b) : 0;  // a row without any number: index 0, as a first-maximum scan gives
    a.ws_best[i] = 0ull;
    if (LSE) {
      float m = -INFINITY, s = 0.0f;
      for (int g = 0; g < a.nseg; ++g) {
        const float2 pr = __ldcg(&a.ws_part[(size_t)i * a.nseg + g]);
        lse_merge(m, s, pr.x, pr.y);
        // leave zeros behind: a later launch of another shape may keep a row's maximum here
        a.ws_part[(size_t)i * a.nseg + g] = make_float2(0.0f, 0.0f);
      }
      a.max_sumexp[2 * i] = m;
      a.max_sumexp[2 * i + 1] = s;
    }
  }
  if (tid == 0) *a.ws_done = 0u;
  __syncthreads();
  // greedy acceptance per slot: leading drafts equal to the row's selection, then the bonus token
  for (int s = tid; s < a.slots; s += kThreads) {
    const int32_t r0 = a.row_off[s], rows = a.row_off[s + 1] - r0;
    const int32_t* d = a.draft + a.draft_off[s];
    int32_t nd = a.draft_off[s + 1] - a.draft_off[s];
    if (nd > rows - 1) nd = rows - 1;  // a draft needs a row after it for the bonus token
    int32_t acc = 0, nx = a.argmax[r0];
    while (acc < nd && nx == d[acc]) {
      ++acc;
      nx = a.argmax[r0 + acc];
    }
    a.accepted[s] = acc;
    a.next[s] = nx;
  }
}

// The same walk over tokens chosen by any means (sampled ones: tools/server_chat.h:578-591)
__global__ void accept_kernel(const int32_t* __restrict__ token, const int32_t* __restrict__ row_off, const int32_t* __restrict__ draft,
                              const int32_t* __restrict__ draft_off, int32_t slots, int32_t* __restrict__ accepted, int32_t* __restrict__ next) {
  const int s = (int)(blockIdx.x * blockDim.x + threadIdx.x);
  if (s >= slots) return;
  const int32_t r0 = row_off[s], rows = row_off[s + 1] - r0;
  const int32_t* d = draft + draft_off[s];
  int32_t nd = draft_off[s + 1] - draft_off[s];
  if (nd > rows - 1) nd = rows - 1;  // a draft needs a row after it for the bonus token
  int32_t acc = 0, nx = rows > 0 ? token[r0] : -1;
  while (acc < nd && nx == d[acc]) {
    ++acc;
    nx = token[r0 + acc];
  }
  accepted[s] = acc;
  next[s] = nx;
}

}  // namespace arcs

using namespace arcs;

extern "C" int arcs_accept_batch(const int32_t* token, const int32_t* row_off, const int32_t* draft, const int32_t* draft_off,
                                 int32_t slots, int32_t* accepted, int32_t* next, void* stream) {
  if (int inj = fault_injected()) return inj;
  if (!token || !row_off || !draft_off || !draft || !accepted || !next || slots <= 0) return set_error(ARCS_ERR_ARG, "accept_batch: bad argument");
  accept_kernel<<<(unsigned)((slots + 127) / 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(token, row_off, draft, draft_off, slots, accepted, next);
  return check_launch("accept_batch");
}

extern "C" size_t arcs_argmax_workspace_bytes(int32_t R, int32_t V) {
  if (R <= 0 || V <= 0) return 0;
  int nseg, seg_len;
  plan_segments(R, V, &nseg, &seg_len);
  return 256 + (size_t)R * 8 + (size_t)R * nseg * 8;
}

extern "C" int arcs_argmax_batch(const arcs_argmax_args* g, void* stream) {
  if (int inj = fault_injected()) return inj;
  if (!g || !g->logits || !g->argmax || g->R <= 0 || g->V <= 0 || g->row_stride < g->V ||
      (g->dtype != ARCS_F32 && g->dtype != ARCS_BF16))
    return set_error(ARCS_ERR_ARG, "argmax_batch: bad argument");
  if (g->slots < 0 || (g->slots > 0 && (!g->row_off || !g->draft_off || !g->draft || !g->accepted || !g->next)))
    return set_error(ARCS_ERR_ARG, "argmax_batch: slots given without row_off/draft/draft_off/accepted/next");
  if (!g->workspace || g->workspace_bytes < arcs_argmax_workspace_bytes(g->R, g->V))
    return set_error(ARCS_ERR_WORKSPACE, "argmax_batch: workspace too small");
  ArgmaxDev a;
  a.logits = g->logits;
  a.row_stride = g->row_stride;
  a.R = g->R;
  a.V = g->V;
  plan_segments(g->R, g->V, &a.nseg, &a.seg_len);
  a.argmax = g->argmax;
  a.max_sumexp = g->max_sumexp;
  a.slots = g->slots;
  a.row_off = g->row_off;
  a.draft = g->draft;
  a.draft_off = g->draft_off;
  a.accepted = g->accepted;
  a.next = g->next;
  char* ws = static_cast<char*>(g->workspace);
  a.ws_done = reinterpret_cast<unsigned int*>(ws);
  a.ws_best = reinterpret_cast<unsigned long long*>(ws + 256);
  a.ws_part = reinterpret_cast<float2*>(ws + 256 + (size_t)g->R * 8);
  a.status = g->status;
  const dim3 grid((unsigned)a.nseg * (unsigned)a.R);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool lse = g->max_sumexp != nullptr;
  constexpr int smem = kStages * kTileBytes;
#define ARCS_LAUNCH(T, L)                                                                                  \
  do {                                                                                                     \
    static std::atomic<unsigned long long> attr_done{0};                                                   \
    cudaError_t e = ensure_dynamic_smem(argmax_kernel<T, L>, smem, attr_done);                             \
    if (e != cudaSuccess) return set_error(ARCS_ERR_CUDA, cudaGetErrorString(e));                          \
    argmax_kernel<T, L><<<grid, kThreads, smem, st>>>(a);                                                  \
  } while (0)
  if (g->dtype == ARCS_F32) {
    if (lse) ARCS_LAUNCH(float, true);
    else ARCS_LAUNCH(float, false);
  } else {
    if (lse) ARCS_LAUNCH(__nv_bfloat16, true);
    else ARCS_LAUNCH(__nv_bfloat16, false);
  }
#undef ARCS_LAUNCH
  return check_launch("argmax_batch");
}

// ---------------------------------------------------------------------------------------------
// arcs_argmax_batch_static: the same launch with its scratch in a fixed device array.
// ---------------------------------------------------------------------------------------------
// Some callers of this library must not allocate device memory: a serving loop that has handed
// the whole of HBM to its own pool (weights, KV cache) and runs with the allocator closed, or
// code running where an allocation would synchronise the device (between the kernels of a
// latency-critical step). For them the scratch lives here, once per GPU that loads the library,
// until the process exits.
constexpr size_t kStaticScratchBytes = 1u << 20;  // 1 MiB: e.g. 1024 rows x 64 segments
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
void* g_static_ptr[kMaxDevices];           // device address of g_static_scratch, per device
std::mutex g_static_mu;                    // guards the per-device set-up
}  // namespace

extern "C" size_t arcs_argmax_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int arcs_argmax_batch_static(const arcs_argmax_args* g, void* stream) {
  if (!g || g->R <= 0 || g->V <= 0) return set_error(ARCS_ERR_ARG, "argmax_batch_static: bad argument");
  const size_t need = arcs_argmax_workspace_bytes(g->R, g->V);
  if (need > kStaticScratchBytes) {
    snprintf(error_buffer(), 256, "argmax_batch_static: %d rows x %d columns need %zu bytes of scratch, the fixed array holds %zu",
             g->R, g->V, need, kStaticScratchBytes);
    return ARCS_ERR_WORKSPACE;
  }
  // The array that is used is the one of the device the stream belongs to, which must be the
  // current device (a launch on another device's stream fails anyway).
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_error(ARCS_ERR_CUDA, cudaGetErrorString(e));
  if (stream) {
    int sdev = dev;
    e = cudaStreamGetDevice(static_cast<cudaStream_t>(stream), &sdev);
    if (e != cudaSuccess) return set_error(ARCS_ERR_CUDA, cudaGetErrorString(e));
    if (sdev != dev) return set_error(ARCS_ERR_ARG, "argmax_batch_static: the stream belongs to another device than the current one");
  }
  if (dev < 0 || dev >= kMaxDevices) return set_error(ARCS_ERR_ARG, "argmax_batch_static: device index out of range");
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptr[dev]) {
      // Set-up, once per device, with that device current: in host code the array's name is only a
      // handle; the address a kernel can use comes from the runtime. The array is cleared here
      // (one thread at a time does this, so the clearing is enqueued once) because the kernels
      // rely on finding, and leaving, their counters at zero.
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess || !p) return set_error(ARCS_ERR_CUDA, e != cudaSuccess ? cudaGetErrorString(e) : "no address for the scratch array");
      e = cudaMemsetAsync(p, 0, kStaticScratchBytes, static_cast<cudaStream_t>(stream));
      if (e != cudaSuccess) return set_error(ARCS_ERR_CUDA, cudaGetErrorString(e));
      g_static_ptr[dev] = p;
    }
    scratch = g_static_ptr[dev];
  }
  arcs_argmax_args a = *g;
  a.workspace = scratch;
  a.workspace_bytes = kStaticScratchBytes;
  return arcs_argmax_batch(&a, stream);
}
