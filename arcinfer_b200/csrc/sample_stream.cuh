// stream_kernel: the single pass over the logits.
//
// One persistent CTA per SM walks a list of work items (a row, or a segment of a row when
// there are few rows). Its warps have fixed roles and never meet at a CTA-wide barrier after
// start-up:
//   producer   keeps a ring of 8 KB tiles filled with 1-D bulk copies (TMA);
//   scanners   16 warps, two to a tile: a 16-byte chunk whose maximum is below the item's
//              current threshold costs a handful of instructions; the few other chunks are set
//              aside, then tested element by element, and the survivors appended to the item's
//              lists in the workspace. On their first tiles of an item the scanners find the
//              item's first threshold together (boot). The warp that closes an item last
//              releases it to the finish kernel;
//   threshold  one warp keeps raising the thresholds of the items that are streaming from the
//              coarse histograms the scanners update;
//   preparing  two warps build the filters and headers of the items ahead of the stream
//              (sample_prep.cuh).
// Items rotate over three sets of per-item state, so the ring never pauses between items.
// A list that overflows (ascending data, masses of ties) is only counted: the finish kernel
// sees the count and reads that item again itself.
#pragma once
#include "sample_prep.cuh"

namespace arcs {

constexpr int kProdWarp = kScanW;                          // producer warp (its first lanes work)
constexpr int kTauWarp = kScanW + 1;                       // threshold warp
constexpr int kPrepWarp0 = kScanW + 2;                     // first preparing warp
constexpr int kThreadsS = (kScanW + 2 + kPrepW) * 32;      // 640 threads
constexpr int kProdLanes = 2;                              // lanes of the producer warp that issue copies (one thread cannot issue 8 KB copies fast enough)
constexpr int kTauSleepNs = 200;                           // pause between two threshold updates
constexpr int kRing = 16;                                  // tiles in the ring (a multiple of kTeams)
constexpr int kPend = 2;                                   // chunks each lane of a scanner can set aside
constexpr int kStash = kPend * 32;                         // ... per warp
constexpr int kFlushEvery = 2;                             // visits after which a warp examines what it has set aside even if its next tile is there
constexpr int kU = 4;                                      // chunks per lane per step of the scan
static_assert(kRing % kTeams == 0, "a team always meets its tiles in the same slots");
static_assert(kMine % (32 * kU) == 0 && kMine / 32 <= 8, "a warp's share of a tile: whole steps, at most 8 chunks per lane");

// indices into the shared scalar arrays
enum {
  S_ABORT = 0, S_PREPARED, S_STREAMED,
  S_DONE = 4 /* [3] */, S_CNT = 8 /* [3 sets][B, A, flagged, -] */,
  S_BOOTCNT = 20 /* [3] */, S_BOOTOK = 23 /* [3] */, S_BASEB = 26 /* [3] */, S_BASEA = 29 /* [3] */, S_END = 32
};
enum { L_TAU_B = 0 /* [3] */, L_TAU_A = 3 /* [3] */, L_BOOT_B = 6 /* [3] */, L_BOOT_A = 9 /* [3] */, L_END = 12 };

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
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

static size_t stream_smem_bytes(int hash_slots) {
  return (size_t)kRing * kSTile + 3 * (size_t)item_tab_bytes(hash_slots) + (size_t)kScanW * kStash * 20 + 2 * kRing * 8 + L_END * 8 +
         6 * 256 * 4 + (size_t)hash_slots * 8 + S_END * 4 + P_END * 4 + 128;
}

template <typename T, bool MASKED>
__global__ void __launch_bounds__(kThreadsS, 1) stream_kernel(const SampleDev a) {
  extern __shared__ __align__(128) char smem[];
  // ---- carve shared memory (ordered by alignment)
  const int tab_bytes = item_tab_bytes(a.hash_slots);
  char* ring = smem;                                                          // kRing * kSTile
  char* tabs = ring + (size_t)kRing * kSTile;                                 // [3] header + filter of the items in flight
  uint4* stash_q = reinterpret_cast<uint4*>(tabs + 3 * (size_t)tab_bytes);     // [kScanW][kStash] chunks set aside by the scanners
  uint64_t* full = reinterpret_cast<uint64_t*>(stash_q + kScanW * kStash);     // [kRing] tile has landed
  uint64_t* empty = full + kRing;                                             // [kRing] tile has been scanned
  unsigned long long* s64 = reinterpret_cast<unsigned long long*>(empty + kRing);  // [L_END]
  int32_t* stash_c = reinterpret_cast<int32_t*>(s64 + L_END);                 // [kScanW][kStash]
  uint32_t* xh = reinterpret_cast<uint32_t*>(stash_c + kScanW * kStash);      // [3 sets][B, A][256] coarse histograms
  uint32_t* hk = xh + 6 * 256;                                                // [hash_slots] the preparing warps' table: columns
  uint32_t* hi_ = hk + a.hash_slots;                                          // [hash_slots] ... what applies to them
  int* sh = reinterpret_cast<int*>(hi_ + a.hash_slots);                       // [S_END]
  int* pmisc = sh + S_END;                                                    // [P_END]
  volatile int* vsh = sh;
  volatile unsigned long long* v64 = s64;
  auto tab_hdr = [&](int st) { return reinterpret_cast<ItemHdr*>(tabs + (size_t)st * tab_bytes); };
  auto tab_bloom = [&](int st) { return reinterpret_cast<uint32_t*>(tabs + (size_t)st * tab_bytes + sizeof(ItemHdr)); };

  constexpr int E = Elem<T>::kPerChunk;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_items = a.B * a.nseg;
  const int my_n = (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

  if (tid == 0) {
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kShare);
    }
    mbar_init_fence();
    for (int i = 0; i < S_END; ++i) sh[i] = 0;
    for (int i = 0; i < L_END; ++i) s64[i] = i >= L_BOOT_B ? 0xFFFFFFFFFFFFFFFFull : 0ull;
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
        const uint32_t n = s_tile_bytes(it.p, t);
        mbar_expect_tx(&full[slot], n);
        bulk_load(ring + (size_t)slot * kSTile, it.p.body + (size_t)t * kSTile, n, &full[slot]);
      }
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
      {  // the item's filter and header must be there (one lane polls)
        if (lane == 0) {
          uint32_t spins = 0;
          while (vsh[S_PREPARED] <= j && !vsh[S_ABORT]) {
            if (++spins > kWaitLimit) abort_now();
            __nanosleep(64);
          }
        }
        __syncwarp();
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
      ctx.baseB = 0;
      ctx.baseA = 0;
      ctx.cnt = &sh[S_CNT + 4 * st];
      const ItemWs w = item_ws(a, (int)blockIdx.x + j * (int)gridDim.x);
      ctx.listB = w.candB;
      ctx.listA = w.candA;
      ctx.listT = w.pre + hd->n_pre;  // (right behind the preparing warps' entries)
      ctx.roomT = item_pre_cap(a.hash_slots) - hd->n_pre;
      ctx.id_base = a.id_base;
      const uint32_t* mrow = ctx.mrow;
      // examine everything the warp has set aside, against the thresholds of this moment
      auto flush = [&]() {
        ctx.tcB = v64[L_TAU_B + st];
        ctx.tcA = MASKED ? v64[L_TAU_A + st] : 0xFFFFFFFFFFFFFFFFull;
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
        if (!mbar_wait_warp(&full[slot], (g / kRing) & 1u)) {
          abort_now();
          break;
        }
        const int nchunk = (int)(s_tile_bytes(it.p, t) / 16u);
        const int32_t col0 = it.p.body_first + t * (kSTile / (int)sizeof(T)) + a.id_base;  // global id of the tile's first element
#ifdef ARCS_DEV_FAKEBOOT
        if (t == t_first) {
          if (lane == 0) {
            const unsigned long long tB = (unsigned long long)(key_of(ARCS_DEV_FAKEBOOT) & 0xFFFF0000u) << 32;
            sm_red_max_u64(&s64[L_TAU_B + st], tB);
            sh[S_BASEB + st] = (int)(tB >> 48);
            sh[S_BASEA + st] = 0;
            __threadfence_block();
            vsh[S_BOOTOK + st] = j + 1;
          }
          __syncwarp();
        }
        if (false) {
#else
        if (t == t_first && t < kBootTiles && c_lo < nchunk) {
#endif
          // ---- boot: the item's first threshold, found together by the scanner warps that meet the
          // item's first kBootTiles tiles. A warp's kth-largest chunk maximum bounds kth elements of
          // its share from below; with kth = ceil(K / warps taking part) in every share, the smallest
          // of the warps' bounds has at least K elements of the item at or above it. Listed columns
          // inside a share (the header counts them) may own a maximum there without counting, so
          // that many more are skipped.
          int n_part = 0;
          for (int tt = 0; tt < min(T_, kBootTiles); ++tt) {
            const int nc = (int)(s_tile_bytes(it.p, tt) / 16u);
            n_part += min(kShare, (nc + kMine - 1) / kMine);
          }
          constexpr int PER = kMine / 32;
          uint32_t kA[PER], kBm[PER];  // (kBm: maxima over the allowed elements, constrained rows only)
#pragma unroll
          for (int u = 0; u < PER; ++u) {
            const int ci = c_lo + u * 32 + lane;
            kA[u] = 0u;
            if (MASKED) kBm[u] = 0u;
            if (ci < nchunk) {
              const uint4 q = lds128(tile + ci * 16);
              kA[u] = key_of(Elem<T>::chunk_max(q));
              if (MASKED) {  // the selection proper counts allowed elements only
                const uint32_t bits = mask_bits_of<E>(mrow, col0 + ci * E);
                float mB = -INFINITY;
                bool anyB = false;
#pragma unroll
                for (int e = 0; e < E; ++e)
                  if ((bits >> e) & 1u) {
                    const float v = Elem<T>::get(q, e);
                    if (!(v != v)) {  // (a NaN is never selected)
                      mB = fmaxf(mB, v);
                      anyB = true;
                    }
                  }
                if (anyB) kBm[u] = key_of(mB);
              }
            }
          }
          const int my_chunks = min(kMine, nchunk - c_lo);
          const int extra = hd->boot_extra[t * kShare + warp % kShare];
          // A small kth is read off the lanes' own maxima (disjoint sets of chunks: as good a bound,
          // a fraction of the work); a large one off all chunk maxima, upper 16 key bits.
          auto kth_of = [&](const uint32_t (&k)[PER], int kth) -> uint32_t {
            if (extra >= 255 || kth > my_chunks) return 0u;
            if (kth <= 8) {
              uint32_t m = k[0];
#pragma unroll
              for (int u = 1; u < PER; ++u) m = max(m, k[u]);
              return warp_kth_lane(m, kth) & 0xFFFF0000u;
            }
            return warp_kth16_regs<PER>(k, kth);
          };
          const int kthB = (hd->K + n_part - 1) / n_part + extra;
          const uint64_t bB = (uint64_t)(MASKED ? kth_of(kBm, kthB) : kth_of(kA, kthB)) << 32;  // keeps ties with it
          uint64_t bA = 0ull;
          if (MASKED) bA = (uint64_t)kth_of(kA, (ARCS_HEAD + n_part - 1) / n_part + extra) << 32;
          if (lane == 0) {
            sm_red_min_u64(&s64[L_BOOT_B + st], (unsigned long long)bB);
            if (MASKED) sm_red_min_u64(&s64[L_BOOT_A + st], (unsigned long long)bA);
            __threadfence_block();
            if ((int)sm_atomic_add(&sh[S_BOOTCNT + st], 1u) == n_part - 1) {
              // the warp that comes last publishes the item's first thresholds
              __threadfence_block();
              const unsigned long long tB = v64[L_BOOT_B + st], tA = MASKED ? v64[L_BOOT_A + st] : 0ull;
              if (tB) sm_red_max_u64(&s64[L_TAU_B + st], tB);
              if (MASKED && tA) sm_red_max_u64(&s64[L_TAU_A + st], tA);
              sh[S_BASEB + st] = (int)(tB >> 48);
              sh[S_BASEA + st] = (int)(tA >> 48);
              __threadfence_block();
              vsh[S_BOOTOK + st] = j + 1;
            }
          }
          __syncwarp();
        }
        if (t == t_first) {
          // nothing of the item is scanned before its first thresholds are there
          if (lane == 0) {
            uint32_t spins = 0;
            while (vsh[S_BOOTOK + st] != j + 1 && !vsh[S_ABORT]) {
              if (++spins > kWaitLimit) abort_now();
              __nanosleep(32);  // (a waiting lane must not take issue slots from the warps still at work)
            }
          }
          __syncwarp();
          __threadfence_block();
          if (vsh[S_ABORT]) break;
          ctx.baseB = (uint32_t)vsh[S_BASEB + st];
          ctx.baseA = (uint32_t)vsh[S_BASEA + st];
        }
        uint64_t tcB = 0, tcA = 0;
        typename Elem<T>::Thr thB, thA;
        auto refresh = [&]() {
          tcB = v64[L_TAU_B + st];
          tcA = MASKED ? v64[L_TAU_A + st] : 0xFFFFFFFFFFFFFFFFull;
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
            bool h = Elem<T>::chunk_reaches(q[u], thB);
            if (MASKED) {
              bool hb = h && ci < nchunk;
              if (hb) hb = mask_bits_of<E>(mrow, col0 + ci * E) != 0u;
              h = hb || Elem<T>::chunk_reaches(q[u], thA);
            }
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
    // Keeps reading new thresholds off the coarse histograms of the items that are streaming (the
    // lower edge of the bin holding the k-th best survivor counted so far), and hands an item over
    // when every scanner has listed what it found in it: list lengths and last thresholds to the
    // item's header in the workspace, the item released to the finish kernel, the set of state
    // cleared for the item three on.
    uint32_t idle = 0;
    for (;;) {
      if (vsh[S_ABORT]) break;
      const int done = vsh[S_STREAMED];
      if (done >= my_n) break;
      const int prepped = vsh[S_PREPARED];
      __threadfence_block();
      if (done < prepped && vsh[S_DONE + done % 3] == kScanW) {
        const int j = done, st = j % 3;
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
        const int nB = vsh[S_CNT + 4 * st + 0], nA = vsh[S_CNT + 4 * st + 1], nT = vsh[S_CNT + 4 * st + 2];
        const int n_pre = hd->n_pre;
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
        if (lane == 0) {
          // (gpu scope: the scanners' list entries, ordered before their arrival at CTA scope, and
          //  the header are read by another kernel once the item is released)
          __threadfence();
          st_release_gpu(&w.hdr->streamed, 1);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) xh[(2 * st) * 256 + i * 32 + lane] = 0;  // both histograms of the item's set
        if (lane < 4) sh[S_CNT + 4 * st + lane] = 0;
        if (lane == 0) {
          sh[S_DONE + st] = 0;
          sh[S_BOOTCNT + st] = 0;
          s64[L_BOOT_B + st] = 0xFFFFFFFFFFFFFFFFull;
          s64[L_BOOT_A + st] = 0xFFFFFFFFFFFFFFFFull;
        }
        __syncwarp();
        __threadfence_block();
        if (lane == 0) vsh[S_STREAMED] = j + 1;
        idle = 0;
        continue;
      }
      for (int j = done; j < min(prepped, done + 2); ++j) {
        const int st = j % 3;
        if (vsh[S_BOOTOK + st] != j + 1) continue;  // (the bins' base is known once the scanners have found the first threshold)
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
  } else {
    // =================================================================== preparing warps
    // An item may take a set of state once the item three back has been handed over.
    const int gt = tid - kPrepWarp0 * 32;
    for (int j = 0; j < my_n; ++j) {
      const int st = j % 3;
      uint32_t spins = 0;
      while (vsh[S_STREAMED] < j - 2 && !vsh[S_ABORT]) {
        if (++spins > kWaitLimit) abort_now();
        __nanosleep(100);
      }
      if (group_sync_or<3, kPrepG>(vsh[S_ABORT] != 0)) break;
      __threadfence_block();
      prep_item<T, MASKED>(a, (int)blockIdx.x + j * (int)gridDim.x, tab_hdr(st), tab_bloom(st), hk, hi_, pmisc, gt);
      if (gt == 0) {
        s64[L_TAU_B + st] = 0ull;
        s64[L_TAU_A + st] = 0ull;
        __threadfence();  // (gpu scope as well: the entries written to the workspace are read by the finish kernel)
        vsh[S_PREPARED] = j + 1;
      }
    }
  }
}

}  // namespace arcs
