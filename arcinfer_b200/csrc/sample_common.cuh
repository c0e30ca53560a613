// What the three kernels of sample_batch share: the argument block, the work items, the
// per-item block of the workspace through which the kernels hand their results on, and the
// row settings of tools/sampler.h.
//
//   prepare_kernel  one small CTA per item: table of the tokens a penalty or a bias touches,
//                   their adjusted logits (exact fp32 arithmetic of Sampler::adjusted), a first
//                   threshold from a short prefix of the item;
//   stream_kernel   one persistent CTA per SM: the single pass over the logits, which keeps
//                   what can still be among the k best of an item;
//   finish_kernel   one small CTA per row: final order, fp64 softmax, cuts, draw.
#pragma once
#include "plan.h"
#include "select.cuh"
#include "stream.cuh"

namespace arcs {

constexpr uint32_t kIdMask = 0x3FFFFFFFu;  // entry word y: id | eligible for the selection proper << 30 | parity << 31
constexpr uint32_t kOkB = 1u << 30;
constexpr int kCapB = 1024;   // candidate buffer: prune trigger (<= 512) + one round of pushes
constexpr int kCapA = 1152;   // constrained head select (k = 512): fill limit 1024 + one step / round of 128
constexpr int kBootBytes = 8192;  // prefix of an item read ahead to seed its threshold
constexpr uint32_t kEmpty = 0xFFFFFFFFu;
// per touched token: occurrences in the history (low 20 bits) and what applies to it
constexpr uint32_t kInfoCount = 0xFFFFFu, kInfoWindow = 1u << 31, kInfoBias = 1u << 30, kInfoBan = 1u << 29;
constexpr int kMaxScalars = 16;   // elements of an item outside its 16-byte aligned body (fewer than 8 at either end)

struct SampleDev {
  const void* logits;
  int64_t row_stride;
  int32_t B, V, nseg, seg_len;
  const arcs_row_params* params;
  const int32_t* hist_off;
  const int32_t* hist_ids;
  const int32_t* bias_off;
  const int32_t* bias_ids;
  const float* bias_vals;
  const double* u;
  const uint32_t* mask;
  const int32_t* mask_row;
  int64_t mask_stride;
  int32_t id_base, v_global;
  int32_t hash_slots, hash_shift;  // power of two, 32 - log2
  int32_t max_hist, max_bias;
  int32_t* token;
  int32_t* n_cand;
  int32_t* n_kept;
  int32_t* flags;
  int32_t* cand_id;
  float* cand_val;
  float* cand_pr;
  int32_t cand_stride;
  char* ws_items;           // [B * nseg] blocks of item_block bytes
  int64_t item_block;
  int32_t* status;
};

// ---- one item's block of the workspace
// [ItemHdr][table columns hash_slots words]   <- copied to shared memory by the stream kernel
// [entries the prepare kernel supplies: hash_slots + kMaxScalars]        (key | word y << 32)
// [survivors of the stream, selection proper: kCapB][constrained head ranking: kCapA when masked]
struct ItemHdr {
  unsigned long long tau0B, tau0A;  // first thresholds (exclusive composites)
  int32_t K;                        // entries the selection proper keeps
  int32_t touched, bans;            // the table is in use; a bias entry <= -100 exists (tools/sampler.h:34)
  int32_t baseB, baseA;             // upper 16 key bits the coarse histograms start at
  int32_t n_pre;                    // entries supplied by the prepare kernel
  int32_t n_candB, n_candA;         // survivors written by the stream kernel
  unsigned long long tauB, tauA;    // last thresholds of the stream: at least K (512) eligible elements of the item lie above
};
static_assert(sizeof(ItemHdr) == 64, "ItemHdr is copied as 64 bytes");

__host__ __device__ inline int32_t item_tab_bytes(int hash_slots) { return (int32_t)sizeof(ItemHdr) + hash_slots * 4; }
__host__ __device__ inline int64_t item_block_bytes(bool masked, int hash_slots) {
  return (int64_t)item_tab_bytes(hash_slots) + (int64_t)(hash_slots + kMaxScalars) * 8 + (int64_t)kCapB * 8 + (masked ? (int64_t)kCapA * 8 : 0);
}
struct ItemWs {
  ItemHdr* hdr;
  uint32_t* hkey;
  unsigned long long* pre;
  unsigned long long* candB;
  unsigned long long* candA;
};
__device__ __forceinline__ ItemWs item_ws(const SampleDev& a, int item) {
  char* p = a.ws_items + (size_t)item * a.item_block;
  ItemWs w;
  w.hdr = reinterpret_cast<ItemHdr*>(p);
  w.hkey = reinterpret_cast<uint32_t*>(p + sizeof(ItemHdr));
  w.pre = reinterpret_cast<unsigned long long*>(w.hkey + a.hash_slots);
  w.candB = w.pre + a.hash_slots + kMaxScalars;
  w.candA = w.candB + kCapB;
  return w;
}

#ifdef ARCS_TRACE
__device__ long long g_trace[64];
#define TR(i) do { if (blockIdx.x == 300 && threadIdx.x == 0) g_trace[i] = clock64(); } while (0)
__device__ long long g_trace2[8 * 16];
#define TS(ev, j) do { if (blockIdx.x == 0 && (j) < 16) g_trace2[(ev) * 16 + (j)] = clock64(); } while (0)
#else
#define TR(i)
#define TS(ev, j)
#endif
__device__ __forceinline__ uint32_t hash_of(int32_t id, int shift) { return ((uint32_t)id * 2654435761u) >> shift; }

// what every kernel derives from an item number
template <typename T>
struct Item {
  int32_t b, seg, lo, hi;
  const T* row;
  SegPlan p;
};
template <typename T>
__device__ __forceinline__ Item<T> item_of(const SampleDev& a, int item) {
  Item<T> it;
  it.b = item / a.nseg;
  it.seg = item % a.nseg;
  it.row = reinterpret_cast<const T*>(a.logits) + (size_t)it.b * a.row_stride;
  it.lo = it.seg * a.seg_len;
  it.hi = min(a.V, it.lo + a.seg_len);
  it.p = make_plan(it.row, it.lo, it.hi);
  return it;
}

// a row's settings as tools/sampler.h reads them
struct RowCfg {
  arcs_row_params prm;
  int kB;
  bool greedy, k_bad, fp_on, rp_on, pp_on, pen_on, lists_ok, touched_on;
  int32_t h0, H, q0, NB;
};
template <bool MASKED>
__device__ __forceinline__ RowCfg row_cfg(const SampleDev& a, int b) {
  const int32_t Vg = a.v_global > 0 ? a.v_global : a.V;
  RowCfg r;
  r.prm = a.params[b];
  r.greedy = r.prm.temperature <= 0.0f;
  if (MASKED) r.kB = r.greedy ? 1 : (r.prm.top_k > 0 ? min(r.prm.top_k, Vg) : 40);     // `need`, tools/sampler.h:86
  else r.kB = r.greedy ? 1 : min(r.prm.top_k > 0 ? min(r.prm.top_k, Vg) : 256, Vg);    // tools/sampler.h:38-40
  r.k_bad = r.kB > ARCS_KCAP;
  if (r.k_bad) r.kB = ARCS_KCAP;
  r.fp_on = r.prm.frequency_penalty != 0.0f;
  r.rp_on = r.prm.repeat_penalty != 1.0f && r.prm.repeat_penalty > 0.0f && r.prm.repeat_last_n != 0;
  r.pp_on = r.prm.presence_penalty != 0.0f;
  r.h0 = a.hist_off ? a.hist_off[b] : 0;
  r.H = a.hist_off ? a.hist_off[b + 1] - r.h0 : 0;
  r.q0 = a.bias_off ? a.bias_off[b] : 0;
  r.NB = a.bias_off ? a.bias_off[b + 1] - r.q0 : 0;
  r.pen_on = (r.fp_on || r.rp_on || r.pp_on) && r.H > 0;
  r.lists_ok = r.H <= a.max_hist && r.NB <= a.max_bias;
  r.touched_on = (r.pen_on || r.NB > 0) && r.lists_ok;
  return r;
}

}  // namespace arcs
