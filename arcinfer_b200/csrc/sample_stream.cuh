// stream_kernel: the single pass over the logits.
//
// One persistent CTA per SM walks a list of work items (a row, or a segment of a row when
// there are few rows). Its warps have fixed roles and never meet at a CTA-wide barrier after
// start-up:
//   producer   keeps a ring of 8 KB tiles filled with 1-D bulk copies (TMA);
//   scanners   16 warps, two to a tile: a 16-byte chunk whose maximum is below the item's
//              current threshold costs a handful of instructions; the few other chunks are set
//              aside, then tested element by element, and the survivors appended to the item's
//              lists in the workspace;
//   threshold  one warp keeps raising the thresholds of the items that are streaming from the
//              coarse histograms the scanners update;
//   closing    one warp hands an item over to the finish kernel when all scanners are through
//              with it: list lengths and last thresholds to the item's header, then the release;
//   preparing  four warps build the filters and headers of the items ahead of the stream
//              (sample_prep.cuh), and find each item's first threshold: ahead of the stream they
//              fetch the item's first tiles into a side buffer (the ring's own copy of those
//              tiles then comes out of the L2 cache) and read the threshold off the maxima of
//              their 16-byte chunks.
// Items rotate over three sets of per-item state, so the ring never pauses between items.
// A list that overflows (ascending data, masses of ties) is only counted: the finish kernel
// sees the count and reads that item again itself.
#pragma once
#include "sample_prep.cuh"

namespace arcs {


constexpr int kProdWarp = kScanW;                          // producer warp (its first lanes work)
constexpr int kTauWarp = kScanW + 1;                       // threshold warp
constexpr int kCloseWarp = kScanW + 2;                     // the warp that hands items over
constexpr int kPrepWarp0 = kScanW + 3;                     // first preparing warp
constexpr int kThreadsS = (kScanW + 3 + kPrepW) * 32;      // 736 threads
// The register file is shared with one CTA of the finish kernel, which runs beside this kernel
// (128 threads x 64 registers): the bound below keeps this kernel at 72 registers a thread.
constexpr int kRegBoundThreads = 896;
constexpr int kProdLanes = 2;                              // lanes of the producer warp that issue copies (one thread cannot issue 8 KB copies fast enough)
constexpr int kTauSleepNs = 200;                           // pause between two threshold updates
constexpr int kRing = 16;                                  // tiles in the ring (a multiple of kTeams)
constexpr int kPend = 2;                                   // chunks each lane of a scanner can set aside
constexpr int kStash = kPend * 32;                         // ... per warp
constexpr int kFlushEvery = 2;                             // visits after which a warp examines what it has set aside even if its next tile is there
constexpr int kU = 2;                                      // chunks per lane per step of the scan (a step that meets a hot chunk takes the slow way as a whole: short steps)
constexpr int kBootLead = 72;                              // tiles the producer is short of an item when that item's first tiles are fetched for its first threshold
static_assert(kRing % kTeams == 0, "a team always meets its tiles in the same slots");
static_assert(kMine % (32 * kU) == 0 && kMine / 32 <= 8, "a warp's share of a tile: whole steps, at most 8 chunks per lane");

// indices into the shared scalar arrays
enum {
  S_ABORT = 0, S_PREPARED, S_STREAMED,
  S_DONE = 4 /* [3] */, S_CNT = 8 /* [3 sets][B, A, flagged, -] */,
  S_PROG = 20 /* the producer's place: item << 16 | tile */,
  S_BOOTOK = 23 /* [3] */, S_BASEB = 26 /* [3] */, S_BASEA = 29 /* [3] */, S_END = 32
};
enum { L_TAU_B = 0 /* [3] */, L_TAU_A = 3 /* [3] */, L_END = 6 };

__device__ __forceinline__ int s_tiles(const SegPlan& p) { return (p.body_bytes + kSTile - 1) / kSTile; }
__device__ __forceinline__ uint32_t s_tile_bytes(const SegPlan& p, int t) {
  const int32_t rem = p.body_bytes - t * kSTile;
  return (uint32_t)(rem < kSTile ? rem : kSTile);
}
__device__ __forceinline__ void st_release_gpu(int32_t* p, int32_t v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// element `el` of the 16-byte chunk held as four words
template <typename T>
__device__ __forceinline__ float elem_of_words(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, int el);
template <>
__device__ __forceinline__ float elem_of_words<float>(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, int el) {
  return __uint_as_float(el == 0 ? w0 : el == 1 ? w1 : el == 2 ? w2 : w3);
}
template <>
__device__ __forceinline__ float elem_of_words<__nv_bfloat16>(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, int el) {
  const uint32_t w = (el >> 1) == 0 ? w0 : (el >> 1) == 1 ? w1 : (el >> 1) == 2 ? w2 : w3;
  return __uint_as_float((el & 1) ? (w & 0xFFFF0000u) : (w << 16));
}

// ---- the scanners' rare path
struct ScanCtx {
  const uint32_t* bloom;   // the item's filter over the columns a penalty or a bias touches
  int32_t bw;              // its size in words
  int32_t touched, bans;
  const uint32_t* mrow;
  uint32_t* histB;         // coarse histograms of the item
  uint32_t* histA;
  uint32_t baseB, baseA;
  int* cnt;                // the item's list lengths so far: [B, A, flagged]
  unsigned long long* listB;  // the item's lists in the workspace (key | word y << 32)
  unsigned long long* listA;
  unsigned long long* listT;
  int32_t roomT;           // entries the flagged list still takes
  int32_t id_base;         // global id of column 0
  uint64_t tcB, tcA;       // thresholds the chunk was listed against
};

// The chunks a scanner warp has set aside are examined one per lane (q: the lane's chunk, g0: global
// id of its first element, have: the lane has one): a float compare finds the (usually single)
// element that reaches the threshold, then those elements go through the exact test together.
// The threshold of the constrained head ranking as the scanners apply it. The head (the 512 best
// of all tokens, tools/sampler.h:93-103) decides two things: whether the best token was refused,
// and, when fewer than k allowed tokens lie inside it, where rank 512 is (:106-116). Both are
// settled by the elements above the k-th best ALLOWED token, and the selection's own threshold
// never exceeds that token: nothing at or below it need be listed, unless the caller wants the
// head itself.
__device__ __forceinline__ uint64_t tau_a_of(uint64_t tauA, uint64_t tauB, bool full_head) {
  return full_head || tauA > tauB ? tauA : tauB;
}

template <typename T, bool MASKED>
__device__ __forceinline__ void scan_examine(const ScanCtx& c, bool have, uint4 q, int32_t g0) {
  constexpr int E = Elem<T>::kPerChunk;
  const int lane = threadIdx.x & 31;
  // threshold values (inclusive): the exact comparison on (key, id) follows per element
  const uint32_t kB32 = (uint32_t)(c.tcB >> 32), kA32 = (uint32_t)(c.tcA >> 32);
  const float tfB = value_of(kB32 < 0x007FFFFFu ? 0x007FFFFFu : kB32);
  const float tfA = MASKED ? value_of(kA32 < 0x007FFFFFu ? 0x007FFFFFu : kA32) : INFINITY;
  const float tf = fminf(tfB, tfA);
  uint32_t bits = 0;  // elements of this lane's chunk still to be examined
  if (have) {
#pragma unroll
    for (int e = 0; e < E; ++e) bits |= (Elem<T>::get(q, e) >= tf ? 1u : 0u) << e;
  }
  while (__any_sync(0xFFFFFFFFu, bits != 0u)) {
    const bool valid = bits != 0u;
    const int el = valid ? __ffs(bits) - 1 : 0;
    bits &= bits - 1u;
    const float v = elem_of_words<T>(q.x, q.y, q.z, q.w, el);
    const int32_t gid = g0 + el;
    const uint32_t ky = key_of(v);
    const uint64_t cm = comp_of(ky, gid);
    // eligible for the selection proper (B) / for the constrained head ranking (A)
    bool okB = valid && ky != 0u && cm > c.tcB;
    bool okA = MASKED && valid && ky != 0u && cm > c.tcA;
    if (MASKED && okB)
      okB = ((__ldg(&c.mrow[gid >> 5]) >> (gid & 31)) & 1u) && !(c.bans && v + 0.0f <= ARCS_BANNED);  // tools/sampler.h:118-119
    // a hot element the filter knows may be a penalised or biased token: it is flagged for the
    // finish kernel to settle, and counts for no threshold
    bool tch = false;
    if ((okB || okA) && c.touched) {
      tch = bloom_has([&](uint32_t wi) { return sm_ld(&c.bloom[wi]); }, c.bw, gid - c.id_base);
    }
    // count the survivors by the upper 16 bits of their keys: the threshold warp reads thresholds off these counts
    if (okB && !tch) sm_red_add(&c.histB[coarse_bin(ky, c.baseB)], 1u);
    if (okA && !tch) sm_red_add(&c.histA[coarse_bin(ky, c.baseA)], 1u);
    // survivors go straight to the item's lists; a list that is full is only counted
    const uint32_t y = (uint32_t)gid | (okB ? kOkB : 0u);
    const unsigned long long ent = (unsigned long long)ky | ((unsigned long long)y << 32);
    auto append = [&](bool p, int which, unsigned long long* list, int cap, unsigned long long e) {
      const unsigned pb = __ballot_sync(0xFFFFFFFFu, p);
      if (pb == 0u) return;
      const int leader = __ffs(pb) - 1;
      uint32_t base = 0;
      if (lane == leader) base = sm_atomic_add(&c.cnt[which], (unsigned)__popc(pb));
      base = __shfl_sync(0xFFFFFFFFu, base, leader);
      const uint32_t pos = base + __popc(pb & ((1u << lane) - 1u));
      if (p && pos < (uint32_t)cap) list[pos] = e;
    };
    append(okB && !tch, 0, c.listB, kListB, ent);
    if (MASKED) append(okA && !tch, 1, c.listA, kListA, (unsigned long long)ky | ((unsigned long long)(uint32_t)gid << 32));
    if (c.touched) append(tch && (okB || okA), 2, c.listT, c.roomT, ent | ((unsigned long long)kTch << 32));
  }
}

// bits [0, E) : the allowed-token bits of the chunk whose first element has global id gid
template <int E>
__device__ __forceinline__ uint32_t mask_bits_of(const uint32_t* mrow, int32_t gid) {
  uint32_t bits = __ldg(&mrow[gid >> 5]) >> (gid & 31);
  if ((gid & 31) + E > 32) bits |= __ldg(&mrow[(gid >> 5) + 1]) << (32 - (gid & 31));
  return bits & ((1u << E) - 1u);
}

// An item's first thresholds, read by the preparing warps off the item's first tiles (buf: nbytes of
// them in the side buffer): the maxima of the 16-byte chunks are distinct elements, so the k-th
// largest of them bounds the k-th largest element from below. Chunks that hold a listed column
// (skip: a word of chunk bits per thread) are left out: their maximum may be a token whose logit
// a penalty changes. One pass: every thread keeps the RT largest maxima of its own chunks; the
// k-th largest of all threads' kept values (a subset of the maxima, so still a lower bound) is
// then found by one warp. Two kept values a thread serve k <= 256, four the 512 of the
// constrained head ranking. tm: [2][kPrepG * RT] words of scratch.
template <typename T, bool MASKED>
__device__ __forceinline__ void boot_item(const SampleDev& a, const Item<T>& it, const ItemHdr* hd, const char* buf, int nbytes,
                                          const uint32_t* skip, uint32_t* tm, unsigned long long* tauB, unsigned long long* tauA,
                                          int* baseB, int* baseA, int gt) {
  constexpr int G = kPrepG;
  constexpr int E = Elem<T>::kPerChunk;
  constexpr int RT = MASKED ? 4 : 2;
  constexpr int R = 4;  // chunks a thread takes together: their loads and maxima overlap
  static_assert(RT * G >= (MASKED ? ARCS_HEAD : ARCS_KCAP), "enough kept values for the largest k");
  const int lane = gt & 31;
  const int nchunk = nbytes / 16;
  const uint32_t* mrow = MASKED ? a.mask + (size_t)(a.mask_row ? a.mask_row[it.b] : it.b) * a.mask_stride : nullptr;
  const int32_t gid0 = it.p.body_first + a.id_base;
  const uint32_t myskip = skip[gt];
  float topB[RT], topA[RT];
#pragma unroll
  for (int i = 0; i < RT; ++i) topB[i] = topA[i] = -INFINITY;
  // keep the RT largest, best first (a NaN is never kept: fmaxf / fminf return the other operand)
  auto keep = [&](float (&top)[RT], float v) {
#pragma unroll
    for (int i = 0; i < RT; ++i) {
      const float hi = fmaxf(top[i], v);
      v = fminf(top[i], v);
      top[i] = hi;
    }
  };
  for (int i0 = 0; i0 * G + gt < nchunk; i0 += R) {
    uint4 q[R];
#pragma unroll
    for (int x = 0; x < R; ++x) q[x] = (i0 + x) * G + gt < nchunk ? lds128(buf + ((i0 + x) * G + gt) * 16) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int x = 0; x < R; ++x) {
      const int ci = (i0 + x) * G + gt;
      if (ci >= nchunk || ((myskip >> (i0 + x)) & 1u)) continue;
      const float mA = Elem<T>::chunk_max(q[x]);
      if (!MASKED) {
        keep(topB, mA);
      } else {  // the selection proper counts allowed elements only; the head ranking all
        keep(topA, mA);
        const uint32_t bits = mask_bits_of<E>(mrow, gid0 + ci * E);
        float mB = -INFINITY;
#pragma unroll
        for (int e = 0; e < E; ++e)
          if ((bits >> e) & 1u) mB = fmaxf(mB, Elem<T>::get(q[x], e));
        keep(topB, mB);
      }
    }
  }
  // (nothing kept, or -inf itself: key zero, no number's)
#pragma unroll
  for (int i = 0; i < RT; ++i) {
    tm[i * G + gt] = topB[i] > -INFINITY ? key_of(topB[i]) : 0u;
    if (MASKED) tm[RT * G + i * G + gt] = topA[i] > -INFINITY ? key_of(topA[i]) : 0u;
  }
  group_sync<3, G>();
  if (gt < 32) {
    constexpr int PER = RT * G / 32;
    uint32_t k[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) k[i] = tm[i * 32 + lane];
    const uint32_t fB = warp_kth16_regs<PER>(k, hd->K);  // keeps ties with it
    uint32_t fA = 0u;
    if (MASKED) {
#pragma unroll
      for (int i = 0; i < PER; ++i) k[i] = tm[RT * G + i * 32 + lane];
      fA = warp_kth16_regs<PER>(k, ARCS_HEAD);
    }
    if (lane == 0) {
      // (zero: fewer than k chunks were there, no threshold)
      const unsigned long long tB = (unsigned long long)fB << 32, tA = (unsigned long long)fA << 32;
      if (tB) sm_red_max_u64(tauB, tB);
      if (MASKED && tA) sm_red_max_u64(tauA, tA);
      *baseB = (int)(tB >> 48);
      *baseA = (int)(tA >> 48);
    }
  }
  group_sync<3, G>();
}

static size_t stream_smem_bytes(bool masked, int hash_slots) {
  const size_t boot_tm_words = masked ? 8 * kPrepG : 2 * kPrepG;
  return (size_t)kRing * kSTile + kBootBytes + 3 * ((size_t)item_tab_bytes(hash_slots) + kBootSkipWords * 4) + (size_t)kScanW * kStash * 20 + (2 * kRing + 8) * 8 +
         L_END * 8 + 6 * 256 * 4 + boot_tm_words * 4 + (size_t)hash_slots * 8 + S_END * 4 + P_END * 4 + 128;
}

template <typename T, bool MASKED>
__global__ void __launch_bounds__(kRegBoundThreads, 1) stream_kernel(const SampleDev a) {
  extern __shared__ __align__(128) char smem[];
  // ---- carve shared memory (ordered by alignment)
  const int tab_bytes = item_tab_bytes(a.hash_slots) + kBootSkipWords * 4;
  char* ring = smem;                                                          // kRing * kSTile
  char* bootbuf = ring + (size_t)kRing * kSTile;                              // kBootBytes: an item's first tiles, fetched ahead of the stream
  char* tabs = bootbuf + kBootBytes;                                          // [3] header + filter of the items in flight
  uint4* stash_q = reinterpret_cast<uint4*>(tabs + 3 * (size_t)tab_bytes);     // [kScanW][kStash] chunks set aside by the scanners
  uint64_t* full = reinterpret_cast<uint64_t*>(stash_q + kScanW * kStash);     // [kRing] tile has landed
  uint64_t* empty = full + kRing;                                             // [kRing] tile has been scanned
  uint64_t* boot_full = empty + kRing;                                        // the side buffer has landed (a phase per item)
  uint64_t* prep_bar = boot_full + 2;                                         // [3] the set's item is prepared (a phase per use of the set)
  uint64_t* bootok_bar = prep_bar + 3;                                        // [3] the set's item has its first thresholds
  unsigned long long* s64 = reinterpret_cast<unsigned long long*>(bootok_bar + 3);  // [L_END]
  int32_t* stash_c = reinterpret_cast<int32_t*>(s64 + L_END);                 // [kScanW][kStash]
  uint32_t* xh = reinterpret_cast<uint32_t*>(stash_c + kScanW * kStash);      // [3 sets][B, A][256] coarse histograms
  uint32_t* boot_tm = xh + 6 * 256;                                           // [1 or 2][2 or 4][kPrepG] the preparing threads' largest chunk maxima
  uint32_t* hk = boot_tm + (MASKED ? 8 : 2) * kPrepG;                                       // [hash_slots] the preparing warps' table: columns
  uint32_t* hi_ = hk + a.hash_slots;                                          // [hash_slots] ... what applies to them
  int* sh = reinterpret_cast<int*>(hi_ + a.hash_slots);                       // [S_END]
  int* pmisc = sh + S_END;                                                    // [P_END]
  volatile int* vsh = sh;
  volatile unsigned long long* v64 = s64;
  auto tab_hdr = [&](int st) { return reinterpret_cast<ItemHdr*>(tabs + (size_t)st * tab_bytes); };
  auto tab_bloom = [&](int st) { return reinterpret_cast<uint32_t*>(tabs + (size_t)st * tab_bytes + sizeof(ItemHdr)); };
  auto tab_skip = [&](int st) { return tab_bloom(st) + bloom_words_of(a.hash_slots); };

  constexpr int E = Elem<T>::kPerChunk;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool full_head = MASKED && a.head_id != nullptr;  // (the caller wants the ranked head itself: every one of its 512 entries is listed)
  const int n_items = a.B * a.nseg;
  const int my_n = (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

  if (tid == 0) {
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kShare);
    }
    for (int i = 0; i < S_END; ++i) sh[i] = 0;
    for (int i = 0; i < L_END; ++i) s64[i] = 0ull;
    mbar_init(boot_full, 1);
    for (int i = 0; i < 3; ++i) {
      mbar_init(&prep_bar[i], 1);
      mbar_init(&bootok_bar[i], 1);
    }
    mbar_init_fence();
  }
  for (int i = tid; i < 6 * 256; i += kThreadsS) xh[i] = 0u;
  // This call's items are not released yet: the flags the finish kernel waits on are cleared
  // before that kernel is allowed to start.
  for (int j = tid; j < my_n; j += kThreadsS) item_ws(a, (int)blockIdx.x + j * (int)gridDim.x).hdr->streamed = 0;
  __threadfence();
  __syncthreads();  // the only CTA-wide barrier
  if (tid == 0) pdl_trigger();  // the finish kernel's CTAs may take their places beside this kernel: each waits for its row's items

  auto abort_now = [&]() {
    vsh[S_ABORT] = 1;
    raise_status(a.status, ARCS_ERR_TIMEOUT);
  };
  if (warp == kProdWarp) {
    // =================================================================== producer
    // Lane l issues the tiles with running number l modulo kProdLanes.
    if (lane < kProdLanes) {
      int j = 0, T_ = 0;
      uint32_t G0 = 0, g = (uint32_t)lane;
      Item<T> it{};
      if (my_n > 0) {
        it = item_of<T>(a, (int)blockIdx.x);
        T_ = s_tiles(it.p);
      }
      for (;; g += kProdLanes) {
        while (j < my_n && g >= G0 + (uint32_t)T_) {  // on to the item that holds tile g
          G0 += (uint32_t)T_;
          if (++j < my_n) {
            it = item_of<T>(a, (int)blockIdx.x + j * (int)gridDim.x);
            T_ = s_tiles(it.p);
          }
        }
        if (j >= my_n || vsh[S_ABORT]) break;
        const int slot = (int)(g % kRing);
        const int t = (int)(g - G0);
        bool ok = false;  // (no sleeping: the other producer lane of the warp would sleep too)
        for (uint32_t tries = 0; tries < kWaitLimit && !ok; ++tries) {
          ok = mbar_try_wait(&empty[slot], ((g / kRing) & 1u) ^ 1u);
          if (!ok && (tries & 1023u) == 1023u && vsh[S_ABORT]) break;
        }
        if (!ok) {
          abort_now();
          break;
        }
        if (lane == 0) vsh[S_PROG] = (j << 16) | min(t, 0xFFFF);
        const uint32_t n = s_tile_bytes(it.p, t);
        mbar_expect_tx(&full[slot], n);
        bulk_load(ring + (size_t)slot * kSTile, it.p.body + (size_t)t * kSTile, n, &full[slot]);
      }
      if (lane == 0) vsh[S_PROG] = my_n << 16;
      if (vsh[S_ABORT]) {  // give this lane's copies in flight a bounded chance to land before the CTA ends
        for (uint32_t x = g % kProdLanes; x < g; x += kProdLanes)
          if (x + kRing >= g) mbar_wait(&full[x % kRing], (x / kRing) & 1u);
      }
    }
  } else if (warp < kScanW) {
    // =================================================================== scanners
    // Team w / kShare takes the tiles whose running number is its own modulo kTeams; each of
    // its warps scans its share of the tile, so a slot is held only briefly.
    uint32_t G0 = 0;  // running number of the item's first tile
    for (int j = 0; j < my_n; ++j) {
      const int st = j % 3;  // filters / thresholds / counts rotate over three sets
      const Item<T> it = item_of<T>(a, (int)blockIdx.x + j * (int)gridDim.x);
      const int T_ = s_tiles(it.p);
      {  // the item's filter, header and first thresholds must be there
        if (!mbar_wait_warp(&prep_bar[st], (uint32_t)(j / 3) & 1u) || !mbar_wait_warp(&bootok_bar[st], (uint32_t)(j / 3) & 1u)) abort_now();
        __threadfence_block();
      }
      if (vsh[S_ABORT]) break;
      const ItemHdr* hd = tab_hdr(st);
      uint4* stq = stash_q + warp * kStash + lane;      // chunks this lane has set aside: stq[s * 32], s < have
      int32_t* stc = stash_c + warp * kStash + lane;
      int have = 0, since = 0;
      ScanCtx ctx;
      ctx.bloom = tab_bloom(st);
      ctx.bw = bloom_words_of(a.hash_slots);
      ctx.touched = hd->touched;
      ctx.bans = MASKED && hd->bans != 0;
      ctx.mrow = MASKED ? a.mask + (size_t)(a.mask_row ? a.mask_row[it.b] : it.b) * a.mask_stride : nullptr;
      ctx.histB = xh + (2 * st) * 256;
      ctx.histA = xh + (2 * st + 1) * 256;
      ctx.baseB = (uint32_t)vsh[S_BASEB + st];
      ctx.baseA = (uint32_t)vsh[S_BASEA + st];
      ctx.cnt = &sh[S_CNT + 4 * st];
      const ItemWs w = item_ws(a, (int)blockIdx.x + j * (int)gridDim.x);
      ctx.listB = w.candB;
      ctx.listA = w.candA;
      ctx.listT = w.pre + hd->n_pre;  // (right behind the preparing warps' entries)
      ctx.roomT = item_pre_cap(a.hash_slots) - hd->n_pre;
      ctx.id_base = a.id_base;
      // examine everything the warp has set aside, against the thresholds of this moment
      auto flush = [&]() {
        ctx.tcB = v64[L_TAU_B + st];
        ctx.tcA = MASKED ? tau_a_of(v64[L_TAU_A + st], ctx.tcB, full_head) : 0xFFFFFFFFFFFFFFFFull;
#pragma unroll 1
        for (int sl = 0; sl < kPend; ++sl) {
          const bool mine = have > sl;
          if (!__any_sync(0xFFFFFFFFu, mine)) break;
          scan_examine<T, MASKED>(ctx, mine, mine ? stq[sl * 32] : make_uint4(0, 0, 0, 0), mine ? stc[sl * 32] : 0);
        }
        have = 0;
        __syncwarp();
      };
      const int t_first = (int)(((uint32_t)(warp / kShare) - G0) % kTeams);
      const int c_lo = (warp % kShare) * kMine;
      for (int t = t_first; t < T_; t += kTeams) {
        const uint32_t g = G0 + (uint32_t)t;
        const int slot = (int)(g % kRing);
        const char* tile = ring + (size_t)slot * kSTile;
        // What is set aside is examined while the warp would only wait for its next tile (the time
        // the examination takes then holds nothing up), and in any case every few visits: the
        // thresholds rise only from what has been examined.
        if (__any_sync(0xFFFFFFFFu, have > 0)) {
          bool now = ++since >= kFlushEvery;
          if (!now) {
            int landed = 0;
            if (lane == 0) landed = mbar_test_wait(&full[slot], (g / kRing) & 1u);
            now = __shfl_sync(0xFFFFFFFFu, landed, 0) == 0;
          }
          if (now) {
            flush();
            since = 0;
          }
        }
        {
          if (!mbar_wait_warp(&full[slot], (g / kRing) & 1u)) {
            abort_now();
            break;
          }
        }
        const int nchunk = (int)(s_tile_bytes(it.p, t) / 16u);
        const int32_t col0 = it.p.body_first + t * (kSTile / (int)sizeof(T)) + a.id_base;  // global id of the tile's first element
        uint64_t tcB = 0, tcA = 0;
        typename Elem<T>::Thr thB, thA;
        auto refresh = [&]() {
          tcB = v64[L_TAU_B + st];
          tcA = MASKED ? tau_a_of(v64[L_TAU_A + st], tcB, full_head) : 0xFFFFFFFFFFFFFFFFull;
          // chunk-level test on values: inclusive on the threshold's value (ids are settled per element)
          const uint32_t kB32 = (uint32_t)(tcB >> 32), kA32 = (uint32_t)(tcA >> 32);
          thB = Elem<T>::make_thr(value_of(kB32 < 0x007FFFFFu ? 0x007FFFFFu : kB32));
          thA = Elem<T>::make_thr(MASKED ? value_of(kA32 < 0x007FFFFFu ? 0x007FFFFFu : kA32) : INFINITY);
        };
        const bool whole = nchunk == kSTile / 16;  // only an item's last tile can be short
        refresh();  // (once per visit: the thresholds move slowly against the few hundred cycles a visit takes)
        for (int c0 = c_lo; c0 < min(nchunk, c_lo + kMine); c0 += kU * 32) {
          uint4 q[kU];
#pragma unroll
          for (int u = 0; u < kU; ++u) q[u] = lds128(tile + (c0 + u * 32 + lane) * 16);  // (inside the slot even past a short tile's end)
          uint32_t m = 0;  // this lane's chunks that reach a threshold
#pragma unroll
          for (int u = 0; u < kU; ++u) {
            const int ci = c0 + u * 32 + lane;
            // (with a mask, whether the chunk's hot element is an allowed one is asked when the
            //  chunk is examined, for all the chunks a warp has set aside at once: a look at the
            //  mask here would stall the scan for a trip to memory at every hot chunk)
            bool h = Elem<T>::chunk_reaches(q[u], thB);
            if (MASKED) h = h || Elem<T>::chunk_reaches(q[u], thA);
            if (!whole) h = h && ci < nchunk;
            m |= (h ? 1u : 0u) << u;
          }
          if (!__any_sync(0xFFFFFFFFu, m != 0u)) continue;  // (nearly always)
          // Set the listed chunks aside, every lane its own: no lane needs to know of another's,
          // unless one has no room left (then everything pending is examined first).
          int need = __popc(m);
          while (__any_sync(0xFFFFFFFFu, have + need > kPend)) {
            flush();
            if (need > kPend) {  // (more than the lane can hold at once: the first now, the rest in the next turn)
#pragma unroll
              for (int u = 0; u < kU; ++u)
                if (((m >> u) & 1u) && have < kPend) {
                  stq[have * 32] = q[u];
                  stc[have * 32] = col0 + (c0 + u * 32 + lane) * E;
                  ++have;
                  m &= ~(1u << u);
                }
              need = __popc(m);
            }
          }
#pragma unroll
          for (int u = 0; u < kU; ++u)
            if ((m >> u) & 1u) {
              stq[have * 32] = q[u];
              stc[have * 32] = col0 + (c0 + u * 32 + lane) * E;  // global id of the chunk's first element
              ++have;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[slot]);  // the slot can be refilled while the chunks set aside are examined
      }
      if (vsh[S_ABORT]) break;
      if (__any_sync(0xFFFFFFFFu, have > 0)) flush();  // what is still set aside
      __syncwarp();
      // this warp has listed everything it found in the item; the threshold warp hands the item
      // over when all scanners have said so
      if (lane == 0) {
        __threadfence_block();
        sm_red_add(&sh[S_DONE + st], 1u);
      }
      G0 += (uint32_t)T_;
    }
  } else if (warp == kTauWarp) {
    // =================================================================== threshold warp
    // Keeps reading new thresholds off the coarse histograms of the items that are streaming: the
    // lower edge of the bin holding the k-th best survivor counted so far.
    uint32_t idle = 0;
    int seen = 0;
    for (;;) {
      if (vsh[S_ABORT]) break;
      const int done = vsh[S_STREAMED];
      if (done >= my_n) break;
      if (done != seen) {
        seen = done;
        idle = 0;
      }
      const int prepped = vsh[S_PREPARED];
      __threadfence_block();
      for (int j = done; j < min(prepped, done + 2); ++j) {
        const int st = j % 3;
        if (vsh[S_BOOTOK + st] != j + 1) continue;  // (the bins' base is known once the item has its first threshold)
        __threadfence_block();
        const ItemHdr* hd = tab_hdr(st);
        int d, kr;
        bool ex;
        find_bin(xh + (2 * st) * 256, hd->K, d, kr, ex);
        if (d > 0 && lane == 0)
          sm_red_max_u64(&s64[L_TAU_B + st], (unsigned long long)(((uint32_t)vsh[S_BASEB + st] + (uint32_t)d) << 16) << 32);
        if (MASKED) {
          find_bin(xh + (2 * st + 1) * 256, ARCS_HEAD, d, kr, ex);
          if (d > 0 && lane == 0)
            sm_red_max_u64(&s64[L_TAU_A + st], (unsigned long long)(((uint32_t)vsh[S_BASEA + st] + (uint32_t)d) << 16) << 32);
        }
      }
      __syncwarp();
      if (++idle > kWaitLimit) {  // (nothing was handed over for seconds)
        abort_now();
        break;
      }
      __nanosleep(kTauSleepNs);
    }
  } else if (warp == kCloseWarp) {
    // =================================================================== closing warp
    // Hands an item over when every scanner has listed what it found in it: list lengths and last
    // thresholds to the item's header in the workspace, the item released to the finish kernel
    // (a release at gpu scope, which takes microseconds while the memory pipes are full: the reason
    // this is a warp of its own), the set of state cleared for the item three on.
    for (int j = 0; j < my_n; ++j) {
      const int st = j % 3;
      uint32_t spins = 0;
      while ((vsh[S_PREPARED] <= j || vsh[S_DONE + st] != kScanW) && !vsh[S_ABORT]) {
        if (++spins > kWaitLimit) abort_now();
        __nanosleep(100);
      }
      if (vsh[S_ABORT]) break;
      __threadfence_block();
      const ItemHdr* hd = tab_hdr(st);
      const ItemWs w = item_ws(a, (int)blockIdx.x + j * (int)gridDim.x);
      const bool booted = vsh[S_BOOTOK + st] == j + 1;
      const uint32_t baseB = (uint32_t)vsh[S_BASEB + st], baseA = (uint32_t)vsh[S_BASEA + st];
      int d, kr;
      bool ex;
      find_bin(xh + (2 * st) * 256, hd->K, d, kr, ex);
      if (booted && d > 0 && lane == 0) sm_red_max_u64(&s64[L_TAU_B + st], (unsigned long long)((baseB + (uint32_t)d) << 16) << 32);
      if (MASKED) {
        find_bin(xh + (2 * st + 1) * 256, ARCS_HEAD, d, kr, ex);
        if (booted && d > 0 && lane == 0) sm_red_max_u64(&s64[L_TAU_A + st], (unsigned long long)((baseA + (uint32_t)d) << 16) << 32);
      }
      __syncwarp();
      int nB = vsh[S_CNT + 4 * st + 0];
      const int nA = vsh[S_CNT + 4 * st + 1], nT = vsh[S_CNT + 4 * st + 2];
      const int n_pre = hd->n_pre;
      if (!MASKED && a.nseg > 1 && nB <= kListB) {
        // A row cut into segments: the finish kernel has to merge every segment's list, most of
        // which was written under the item's first, loose thresholds. The list is cut here to
        // the entries above the item's last threshold (in place: a round's entries are all read
        // before any is written, to places at or before the round's first).
        const unsigned long long tau = v64[L_TAU_B + st];
        int kept = 0;
        for (int i0 = 0; i0 < nB; i0 += 8 * 32) {
          unsigned long long e[8];
#pragma unroll
          for (int x = 0; x < 8; ++x) e[x] = i0 + x * 32 + lane < nB ? __ldcg(&w.candB[i0 + x * 32 + lane]) : 0ull;
#pragma unroll
          for (int x = 0; x < 8; ++x) {
            const uint32_t ky = (uint32_t)e[x], y = (uint32_t)(e[x] >> 32);
            const bool keep = i0 + x * 32 + lane < nB && comp_of(ky, (int32_t)(y & kIdMask)) > tau;
            const unsigned bk = __ballot_sync(0xFFFFFFFFu, keep);
            if (keep) w.candB[kept + __popc(bk & ((1u << lane) - 1u))] = e[x];
            kept += __popc(bk);
          }
        }
        nB = kept;
        __syncwarp();
      }
      if (nB > kListB || nA > kListA || nT > item_pre_cap(a.hash_slots) - n_pre) {
        // a list overflowed: the finish kernel will read the item again and needs its filter
        const uint32_t* bl = tab_bloom(st);
        for (int i = lane; i < bloom_words_of(a.hash_slots); i += 32) w.bloom[i] = bl[i];
      }
      __syncwarp();
      if (lane == 0) {
        w.hdr->tauB = v64[L_TAU_B + st];
        w.hdr->tauA = v64[L_TAU_A + st];
        w.hdr->K = hd->K;
        w.hdr->touched = hd->touched;
        w.hdr->bans = hd->bans;
        w.hdr->n_pre = n_pre;
        w.hdr->n_tch = nT;
        w.hdr->n_candB = nB;
        w.hdr->n_candA = nA;
      }
      __syncwarp();
      // The set is free for the item three on before the release is through: nothing of the set is
      // read below.
#pragma unroll
      for (int i = 0; i < 16; ++i) xh[(2 * st) * 256 + i * 32 + lane] = 0;  // both histograms of the item's set
      if (lane < 4) sh[S_CNT + 4 * st + lane] = 0;
      if (lane == 0) sh[S_DONE + st] = 0;
      __syncwarp();
      __threadfence_block();
      if (lane == 0) vsh[S_STREAMED] = j + 1;
      if (lane == 0) {
        // (gpu scope: the scanners' list entries, ordered before their arrival at CTA scope, and
        //  the header are read by another kernel once the item is released)
        st_release_gpu(&w.hdr->streamed, 1);
      }
      __syncwarp();
    }
  } else {
    // =================================================================== preparing warps
    // Three kinds of work, decided by the group's first thread and done by all of it:
    //  - an item is prepared when the set of state it takes is free (the item three back has
    //    been handed over);
    //  - an item's first tiles are fetched into the side buffer when the producer is kBootLead
    //    tiles short of the item: late enough for the ring's own copy of these tiles to come out
    //    of the L2 cache, early enough for the threshold to be there when the scanners want it;
    //  - the item's first threshold is read off that buffer once it has landed.
    const int gt = tid - kPrepWarp0 * 32;
    int next_prep = 0, boot_issued = 0, boot_done = 0;
    int need_prog = 0;   // the producer's place from which item boot_issued may be fetched
    uint32_t idle = 0;
    while (boot_done < my_n) {
      if (gt == 0) {
        int cmd = 0;
        if (vsh[S_ABORT]) cmd = 9;
        else if (boot_issued == boot_done && vsh[S_PROG] >= need_prog) cmd = 1;
        else if (boot_issued > boot_done && next_prep > boot_done && mbar_test_wait(boot_full, (uint32_t)boot_done & 1u)) cmd = 2;
        else if (next_prep < my_n && vsh[S_STREAMED] >= next_prep - 2) cmd = 3;
        pmisc[P_CMD] = cmd;
      }
      group_sync<3, kPrepG>();
      const int cmd = pmisc[P_CMD];
      group_sync<3, kPrepG>();
      if (cmd == 9) break;
      if (cmd == 0) {  // (nothing to do yet: none of this is urgent, so the group sleeps between looks)
        if (++idle > kWaitLimit) {
          abort_now();
          break;
        }
        __nanosleep(200);
        continue;
      }
      idle = 0;
      if (cmd == 1) {
        // ---- fetch the first tiles of item boot_issued
        const Item<T> it = item_of<T>(a, (int)blockIdx.x + boot_issued * (int)gridDim.x);
        const int boot_bytes = min(it.p.body_bytes, kBootBytes);
        if (gt == 0) {
          if (boot_bytes > 0) {
            fence_proxy_async();  // (the group's reads of the buffer for the item before are done)
            mbar_expect_tx(boot_full, (uint32_t)boot_bytes);
            bulk_load(bootbuf, it.p.body, (uint32_t)boot_bytes, boot_full);
          } else {
            mbar_arrive(boot_full);
          }
        }
        // the place of the producer from which the next item may be fetched
        need_prog = (boot_issued << 16) | min(0xFFFF, max(0, s_tiles(it.p) - kBootLead));
        ++boot_issued;
      } else if (cmd == 2) {
        // ---- the first thresholds of item boot_done
        const int jb = boot_done, st = jb % 3;
        const Item<T> it = item_of<T>(a, (int)blockIdx.x + jb * (int)gridDim.x);
        const int nb = min(it.p.body_bytes, kBootBytes);
        const ItemHdr* hb = tab_hdr(st);
        unsigned long long* tB = &s64[L_TAU_B + st];
        unsigned long long* tA = &s64[L_TAU_A + st];
        boot_item<T, MASKED>(a, it, hb, bootbuf, nb, tab_skip(st), boot_tm, tB, tA, &sh[S_BASEB + st], &sh[S_BASEA + st], gt);
        if (gt == 0) {
          __threadfence_block();
          vsh[S_BOOTOK + st] = jb + 1;
          mbar_arrive(&bootok_bar[st]);
        }
        ++boot_done;
      } else {
        // ---- prepare item next_prep
        const int j = next_prep, st = j % 3;
        __threadfence_block();
        if (gt == 0) {  // (the set is free: nobody reads its thresholds now)
          s64[L_TAU_B + st] = 0ull;
          s64[L_TAU_A + st] = 0ull;
        }
        prep_item<T, MASKED>(a, (int)blockIdx.x + j * (int)gridDim.x, tab_hdr(st), tab_bloom(st), tab_skip(st), hk, hi_, pmisc, gt);
        if (gt == 0) {
          __threadfence();  // (gpu scope as well: the entries written to the workspace are read by the finish kernel)
          vsh[S_PREPARED] = j + 1;
          mbar_arrive(&prep_bar[st]);
        }
        ++next_prep;
      }
    }
  }
}

}  // namespace arcs
