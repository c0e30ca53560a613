// What the two kernels of sample_batch share: the argument block, the work items, the per-item
// block of the workspace through which they hand their results on, and the row settings of
// tools/sampler.h.
//
//   stream_kernel   one persistent CTA per SM: the single pass over the logits, which keeps what
//                   can still be among the k best of an item. Two of its warps prepare the items
//                   ahead of the stream (table of the tokens a penalty or a bias touches, their
//                   adjusted logits with the exact fp32 arithmetic of Sampler::adjusted);
//   finish_kernel   one small CTA per row: final order, fp64 softmax, cuts, draw. It is launched
//                   behind the stream kernel, runs beside it, and takes a row as soon as the stream
//                   has released the row's items.
#pragma once
#include "plan.h"
#include "select.cuh"
#include "stream.cuh"

namespace arcs {

constexpr uint32_t kIdMask = 0x1FFFFFFFu;  // entry word y: id | flagged by the filter << 29 | eligible for the selection proper << 30 | parity << 31
constexpr uint32_t kTch = 1u << 29, kOkB = 1u << 30;
constexpr int kCapB = 1024;   // finish kernel's candidate buffer: prune trigger + one round of pushes
constexpr int kCapA = 1280;   // ... for the constrained head select (k = 512): trigger 768 + four rounds of 128
constexpr int kListB = 4096;  // survivors of the stream an item's block holds: selection proper (typically k * (1 + ln(V / 4096)))
constexpr int kListA = 8192;  // ... constrained head ranking
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
  int32_t cand_width;       // entries written per row of the candidate outputs (<= cand_stride)
  int32_t* head_id;         // [B][ARCS_HEAD] ranked head of a constrained row (optional)
  float* head_val;
  int32_t* n_head;
  char* ws_items;           // [B * nseg] blocks of item_block bytes
  int64_t item_block;
  int32_t* status;
  // merge mode of the finish kernel (vocabulary shards): the candidates come from gathered per-shard lists
  int32_t merge_G, merge_stride;
  const int32_t* merge_id;   // [G][B][merge_stride] global ids, best first
  const float* merge_val;    // [G][B][merge_stride] adjusted logits
  const int32_t* merge_n;    // [G][B] entries per list
  int32_t merge_width;       // entries per gathered list (<= merge_stride)
  const float* merge_mz;     // [G][B] (max, sum exp) pairs of the shards, merge_mz_stride floats apart (optional)
  int32_t merge_mz_stride;
  float* mz_out;             // [B][2] the pairs combined (optional)
  int32_t rows_per_cta;      // finish kernel without a mask: rows a CTA takes, one a warp (4; 1 when the rows are few)
};

// ---- geometry of the stream (shared with the preparing warps, which count the listed columns
// that fall into an item's first tiles)
constexpr int kScanW = 16;                   // scanner warps
constexpr int kShare = 2;                    // scanner warps that split one tile between them
constexpr int kTeams = kScanW / kShare;      // teams: team x takes the tiles whose running number is x modulo kTeams
constexpr int kSTile = 8192;                 // bytes per tile (512 chunks of 16 bytes)
constexpr int kMine = kSTile / 16 / kShare;  // chunks of a tile per scanner warp
constexpr int kBootTiles = 2;                // first tiles of an item its first threshold is read off
constexpr int kBootBytes = kBootTiles * kSTile;
constexpr int kPrepW = 4;                    // preparing warps of the stream kernel
constexpr int kPrepG = kPrepW * 32;          // ... threads (named barrier 3)
// One bit per 16-byte chunk of those tiles: the chunk holds a listed column. Chunk c is bit
// c / kPrepG of word c % kPrepG: the chunks one preparing thread looks at share a word.
constexpr int kBootSkipWords = kPrepG;
static_assert(kBootBytes / 16 / kPrepG <= 32, "a preparing thread's chunks of the first tiles fit one word of bits");

// ---- one item's block of the workspace
// [ItemHdr][filter bloom_words words: written only when a list of the stream overflowed]
// [entries with final values, from the preparing warps, then hot elements the filter flagged, from
//  the scanners, raw: hash_slots + kMaxScalars]                        (key | word y << 32)
// [survivors of the stream, selection proper: kListB][constrained head ranking: kListA when masked]
struct ItemHdr {
  unsigned long long tauB, tauA;    // last thresholds of the stream: at least K (512) eligible elements of the item lie above
  int32_t K;                        // entries the selection proper keeps
  int32_t touched;                  // kTouchNone / kTouchLight / kTouchTable
  int32_t bans;                     // a bias entry <= -100 exists (tools/sampler.h:34)
  int32_t n_pre;                    // entries supplied by the preparing warps
  int32_t n_tch;                    // flagged hot elements appended by the scanners
  int32_t n_candB, n_candA;         // survivors written by the scanners
  int32_t streamed;                 // 1 (released at gpu scope) once everything above and the lists are final
  int32_t pad[12];
};
static_assert(sizeof(ItemHdr) == 96, "ItemHdr is 96 bytes");
// How an item's penalised / biased tokens reach the finish kernel.
//  light: penalties can only lower a logit, so a history token matters only if its raw logit is
//         hot: the stream flags hot elements the filter knows and the finish kernel adjusts them;
//         the (few) bias tokens are evaluated by the prepare kernel.
//  table: some penalty can raise a logit, or the bias list is long: the prepare kernel evaluates
//         every touched token; flagged hot elements that are touched are dropped later.
constexpr int kTouchNone = 0, kTouchLight = 1, kTouchTable = 2;
constexpr int kLightBias = 64;  // longest bias list handled without the table

// filter size: 64 bits per listed id while the lists are short (two bits set per id: about one false
// alarm in a thousand lookups), at most 1024 words: longer lists only raise the false-alarm rate,
// and a false alarm costs one more entry for the finish kernel to settle
constexpr int kMaxTableSlots = 2048;  // most distinct listed tokens x 2 the on-chip table holds
__host__ __device__ inline int32_t bloom_words_of(int hash_slots) { return hash_slots < 256 ? 256 : hash_slots > 1024 ? 1024 : hash_slots; }
__host__ __device__ inline int32_t item_tab_bytes(int hash_slots) { return (int32_t)sizeof(ItemHdr) + bloom_words_of(hash_slots) * 4; }
// (in shared memory a set of per-item state also carries kBootSkipWords words behind the filter)
__host__ __device__ inline int32_t item_pre_cap(int hash_slots) { return hash_slots + kMaxScalars; }
__host__ __device__ inline int64_t item_block_bytes(bool masked, int hash_slots) {
  return (int64_t)item_tab_bytes(hash_slots) + (int64_t)item_pre_cap(hash_slots) * 8 + (int64_t)kListB * 8 + (masked ? (int64_t)kListA * 8 : 0);
}
struct ItemWs {
  ItemHdr* hdr;
  uint32_t* bloom;
  unsigned long long* pre;
  unsigned long long* candB;
  unsigned long long* candA;
};
__device__ __forceinline__ ItemWs item_ws(const SampleDev& a, int item) {
  char* p = a.ws_items + (size_t)item * a.item_block;
  ItemWs w;
  w.hdr = reinterpret_cast<ItemHdr*>(p);
  w.bloom = reinterpret_cast<uint32_t*>(p + sizeof(ItemHdr));
  w.pre = reinterpret_cast<unsigned long long*>(w.bloom + bloom_words_of(a.hash_slots));
  w.candB = w.pre + item_pre_cap(a.hash_slots);
  w.candA = w.candB + kListB;
  return w;
}
// the two bits of a column in an item's filter (bits: 32 * bloom_words, a power of two)
__device__ __forceinline__ uint32_t bloom_bit1(int32_t c, int bloom_words) { return (((uint32_t)c * 0x9E3779B1u) >> 8) & (uint32_t)(bloom_words * 32 - 1); }
__device__ __forceinline__ uint32_t bloom_bit2(int32_t c, int bloom_words) { return (((uint32_t)c * 0x85EBCA6Bu) >> 7) & (uint32_t)(bloom_words * 32 - 1); }
template <typename LOAD>
__device__ __forceinline__ bool bloom_has(LOAD load, int bloom_words, int32_t c) {
  const uint32_t b1 = bloom_bit1(c, bloom_words), b2 = bloom_bit2(c, bloom_words);
  return ((load(b1 >> 5) >> (b1 & 31)) & (load(b2 >> 5) >> (b2 & 31)) & 1u) != 0u;
}

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
  int touch;  // kTouchNone / kTouchLight / kTouchTable
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
  const bool lowering = (!r.rp_on || r.prm.repeat_penalty >= 1.0f) && !(r.prm.frequency_penalty < 0.0f) && !(r.prm.presence_penalty < 0.0f);
  r.touch = !r.touched_on ? kTouchNone : ((r.pen_on && !lowering) || r.NB > kLightBias) ? kTouchTable : kTouchLight;
  // the table holds every listed token of the row: a row whose lists are longer than it is refused
  // (rows in light mode, whose penalties only lower logits, take histories of any length)
  if (r.touch == kTouchTable && (r.pen_on ? r.H : 0) + r.NB > a.hash_slots / 2) {
    r.lists_ok = false;
    r.touched_on = false;
    r.touch = kTouchNone;
  }
  return r;
}

// tools/sampler.h:160-171 for a token that occurs cnt (> 0) times in the history; in_window: one
// of the occurrences lies inside the repeat window
__device__ __forceinline__ float penalise(const RowCfg& r, float v, uint32_t cnt, bool in_window) {
  if (r.fp_on) v = __fsub_rn(v, __fmul_rn(r.prm.frequency_penalty, (float)cnt));                         // :160
  if (r.rp_on && in_window) v = v > 0.0f ? __fdiv_rn(v, r.prm.repeat_penalty) : __fmul_rn(v, r.prm.repeat_penalty);  // :166
  if (r.pp_on) v = __fsub_rn(v, r.prm.presence_penalty);                                                 // :171
  return v;
}
// first history index inside the repeat window (tools/sampler.h:163)
__device__ __forceinline__ int32_t window_start(const RowCfg& r) {
  const int32_t nwin = r.prm.repeat_last_n < 0 ? r.H : min(r.H, r.prm.repeat_last_n);
  return r.H - nwin;
}

}  // namespace arcs
