// stream_kernel: the single pass over the logits.
//
// One persistent CTA per SM walks a list of work items (a row, or a segment of a row when
// there are few rows). Its warps have fixed roles and never meet at a CTA-wide barrier:
//   producer   keeps a ring of 8 KB tiles filled with 1-D bulk copies (TMA);
//   scanners   16 warps, four to a tile: a 16-byte chunk whose maximum is below the item's
//              current threshold costs a handful of instructions; the few other chunks are set
//              aside, then tested element by element, and the survivors queued;
//   examiner   one warp owns the candidate buffers: it moves the queued survivors into them,
//              drops what the threshold has overtaken, and writes what is left to the item's
//              block of the workspace when every scanner has closed the item;
//   threshold  one warp fetches the items' tables and first thresholds (written by the prepare
//              kernel) ahead of the stream, and keeps raising the thresholds of the items that
//              are streaming from the coarse histograms the scanners update.
// Items rotate over three sets of per-item state and two candidate buffers, so the ring never
// pauses between items.
#pragma once
#include "sample_common.cuh"

namespace arcs {

constexpr int kScanW = 16;                                 // scanner warps
#ifndef ARCS_SHARE
#define ARCS_SHARE 2
#endif
constexpr int kShare = ARCS_SHARE;                         // scanner warps that split one tile between them
constexpr int kTeams = kScanW / kShare;
constexpr int kExamWarp = kScanW;                          // examiner warp
constexpr int kProdWarp = kScanW + 1;                      // producer warp (its first lanes work)
constexpr int kTauWarp = kScanW + 2;                       // threshold warp
constexpr int kThreadsS = (kScanW + 3) * 32;               // 608 threads
#ifndef ARCS_PROD_LANES
#define ARCS_PROD_LANES 2
#endif
constexpr int kProdLanes = ARCS_PROD_LANES;                // lanes of the producer warp that issue copies
#ifndef ARCS_TAU_SLEEP
#define ARCS_TAU_SLEEP 200
#endif
#ifndef ARCS_EXAM_SLEEP
#define ARCS_EXAM_SLEEP 200
#endif
constexpr int kExamSleepNs = ARCS_EXAM_SLEEP;              // examiner's pause while the queue is short
constexpr int kTauSleepNs = ARCS_TAU_SLEEP;                // pause between two threshold updates
#ifndef ARCS_RING
#define ARCS_RING 16
#endif
constexpr int kRing = ARCS_RING;                           // tiles in the ring (a multiple of kTeams)
constexpr int kSTile = 8192;                               // bytes per tile (512 chunks)
constexpr int kStash = 16;                                 // chunks a scanner sets aside per flush
constexpr int kQueue = 512;                                // queued elements between scanners and examiner
constexpr uint32_t kMarker = kIdMask;                      // id field of a scanner's end-of-item entry
static_assert(kRing % kTeams == 0, "a team always meets its tiles in the same slots");

// indices into the shared scalar arrays
enum { S_ABORT = 0, S_QTAIL, S_QHEAD, S_PREPARED, S_STREAMED, S_END = 8 };
enum { L_TAU_B = 0 /* [3] */, L_TAU_A = 3 /* [3] */, L_END = 6 };

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ int s_tiles(const SegPlan& p) { return (p.body_bytes + kSTile - 1) / kSTile; }
__device__ __forceinline__ uint32_t s_tile_bytes(const SegPlan& p, int t) {
  const int32_t rem = p.body_bytes - t * kSTile;
  return (uint32_t)(rem < kSTile ? rem : kSTile);
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

// ---- the scanners' rare path, kept out of line so that the streaming loop stays small
struct ScanCtx {
  const uint32_t* bloom;   // the item's filter over the columns a penalty or a bias touches
  int32_t bw;              // its size in words
  int32_t touched, bans, par;
  const uint32_t* mrow;
  uint32_t* histB;         // coarse histograms of the item
  uint32_t* histA;
  uint32_t baseB, baseA;
  int* sh;                 // shared scalars (queue head / tail, abort flag)
  unsigned long long* q_ent;  // queue slots: 0 = empty, else key | (id, flags) << 32
  int32_t* status;
  int32_t id_base;         // global id of column 0
  uint64_t tcB, tcA;       // thresholds the chunk was listed against
};

// append one entry to the scanner -> examiner queue (the caller holds reservation e)
__device__ __forceinline__ void queue_write(int* sh, unsigned long long* q_ent, int32_t* status, uint32_t e,
                                            uint32_t key, uint32_t idp) {
  uint32_t spins = 0;  // bounded wait for room
  while ((int32_t)(e - sm_ld_volatile(&sh[S_QHEAD])) >= kQueue && !sm_ld_volatile(&sh[S_ABORT])) {
    if (++spins > kWaitLimit) {
      *reinterpret_cast<volatile int*>(&sh[S_ABORT]) = 1;
      raise_status(status, ARCS_ERR_TIMEOUT);
    }
    __nanosleep(32);
  }
  // one 64-bit store publishes the entry: a slot is zero until written and zeroed again by the
  // examiner before it frees it (an entry is never zero: data has a non-zero key, a marker a non-zero id)
  sm_st_volatile64(&q_ent[e % kQueue], (unsigned long long)key | ((unsigned long long)idp << 32));
}

// The chunks a scanner warp has set aside (data in sq[], global id of each chunk's first element
// in sc[]) are examined one chunk per lane: a float compare finds the (usually single) element
// that reaches the threshold, then those elements go through the exact test together. Runs
// after the warp has released the tile's ring slot, so the time spent here never holds up the
// copy engine.
template <typename T, bool MASKED>
__device__ __noinline__ void scan_examine(const ScanCtx& c, const uint4* sq, const int32_t* sc, int n) {
  constexpr int E = Elem<T>::kPerChunk;
  const int lane = threadIdx.x & 31;
  // threshold values (inclusive): the exact comparison on (key, id) follows per element
  const uint32_t kB32 = (uint32_t)(c.tcB >> 32), kA32 = (uint32_t)(c.tcA >> 32);
  const float tfB = value_of(kB32 < 0x007FFFFFu ? 0x007FFFFFu : kB32);
  const float tfA = MASKED ? value_of(kA32 < 0x007FFFFFu ? 0x007FFFFFu : kA32) : INFINITY;
  const float tf = fminf(tfB, tfA);
  uint4 q = make_uint4(0, 0, 0, 0);
  int32_t g0 = 0;
  uint32_t bits = 0;  // elements of this lane's chunk still to be examined
  if (lane < n) {
    q = lds128(&sq[lane]);
    g0 = (int32_t)sm_ld(&sc[lane]);
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
      const uint32_t bit = bloom_bit(gid - c.id_base, c.bw);
      tch = (sm_ld(&c.bloom[bit >> 5]) >> (bit & 31)) & 1u;
    }
    // count the survivors by the upper 16 bits of their keys: the threshold warp reads thresholds off these counts
    if (okB && !tch) sm_red_add(&c.histB[coarse_bin(ky, c.baseB)], 1u);
    if (okA && !tch) sm_red_add(&c.histA[coarse_bin(ky, c.baseA)], 1u);
    const bool pass = okB || okA;
    const unsigned pb = __ballot_sync(0xFFFFFFFFu, pass);
    if (pb) {
      const int leader = __ffs(pb) - 1;
      uint32_t base = 0;
      if (lane == leader) base = sm_atomic_add(&c.sh[S_QTAIL], (unsigned)__popc(pb));
      base = __shfl_sync(0xFFFFFFFFu, base, leader);
      if (pass)
        queue_write(c.sh, c.q_ent, c.status, base + __popc(pb & ((1u << lane) - 1u)), ky,
                    (uint32_t)gid | (tch ? kTch : 0u) | ((uint32_t)okB << 30) | ((uint32_t)c.par << 31));
    }
  }
}

static size_t stream_smem_bytes(bool masked, int hash_slots) {
  size_t n = (size_t)kRing * kSTile + 3 * (size_t)item_tab_bytes(hash_slots) + (size_t)kQueue * 8 + (size_t)kScanW * kStash * 20 +
             (2 * kRing + 4) * 8 + L_END * 8 + (256 + 6 * 256) * 4 + (size_t)kTmpCap * 8 + S_END * 4;
  n += (size_t)2 * kCapB * 8;
  if (masked) n += (size_t)2 * kCapA * 8;
  return n + 128;
}

template <typename T, bool MASKED>
__global__ void __launch_bounds__(kThreadsS, 1) stream_kernel(const SampleDev a) {
  extern __shared__ __align__(128) char smem[];
  // ---- carve shared memory (ordered by alignment)
  const int tab_bytes = item_tab_bytes(a.hash_slots);
  char* ring = smem;                                                          // kRing * kSTile
  char* tabs = ring + (size_t)kRing * kSTile;                                 // [3] item tables as the prepare kernel wrote them
  unsigned long long* q_ent = reinterpret_cast<unsigned long long*>(tabs + 3 * (size_t)tab_bytes);  // [kQueue]
  uint4* stash_q = reinterpret_cast<uint4*>(q_ent + kQueue);                   // [kScanW][kStash] chunks set aside by the scanners
  uint64_t* full = reinterpret_cast<uint64_t*>(stash_q + kScanW * kStash);     // [kRing] tile has landed
  uint64_t* empty = full + kRing;                                             // [kRing] tile has been scanned
  uint64_t* tab_full = empty + kRing;                                         // [3] (+1 pad) table has landed
  unsigned long long* s64 = reinterpret_cast<unsigned long long*>(tab_full + 4);  // [L_END]
  int32_t* stash_c = reinterpret_cast<int32_t*>(s64 + L_END);                 // [kScanW][kStash]
  uint32_t* xhist = reinterpret_cast<uint32_t*>(stash_c + kScanW * kStash);   // [256] examiner's radix histogram
  uint32_t* xh = xhist + 256;                                                 // [3 sets][B, A][256] coarse histograms
  uint32_t* xtk = xh + 6 * 256;                                               // [kTmpCap] examiner's scratch
  int32_t* xti = reinterpret_cast<int32_t*>(xtk + kTmpCap);
  int* sh = reinterpret_cast<int*>(xti + kTmpCap);                            // [S_END]
  uint32_t* bkey = reinterpret_cast<uint32_t*>(sh + S_END);                   // [2][kCapB]
  int32_t* bid = reinterpret_cast<int32_t*>(bkey + 2 * kCapB);
  uint32_t* akey = reinterpret_cast<uint32_t*>(bid + 2 * kCapB);              // [2][kCapA] when MASKED
  int32_t* aid = reinterpret_cast<int32_t*>(akey + (MASKED ? 2 * kCapA : 0));
  volatile int* vsh = sh;
  volatile unsigned long long* v64 = s64;
  auto tab_hdr = [&](int st) { return reinterpret_cast<const ItemHdr*>(tabs + (size_t)st * tab_bytes); };
  auto tab_bloom = [&](int st) { return reinterpret_cast<const uint32_t*>(tabs + (size_t)st * tab_bytes + sizeof(ItemHdr)); };

  constexpr int E = Elem<T>::kPerChunk;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_items = a.B * a.nseg;
  const int my_n = (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

  if (tid == 0) {
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kShare);
    }
    for (int i = 0; i < 3; ++i) mbar_init(&tab_full[i], 1);
    mbar_init_fence();
    for (int i = 0; i < S_END; ++i) sh[i] = 0;
    for (int i = 0; i < L_END; ++i) s64[i] = 0ull;
  }
  for (int i = tid; i < kQueue; i += kThreadsS) q_ent[i] = 0ull;
  for (int i = tid; i < 6 * 256; i += kThreadsS) xh[i] = 0u;
  __syncthreads();  // the only CTA-wide barrier
  if (tid == 0) TS(0, 0);

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
        bool ok;
        if (kProdLanes == 1) {
          ok = mbar_wait(&empty[slot], ((g / kRing) & 1u) ^ 1u);
        } else {  // (no sleeping: the other producer lanes of the warp would sleep too)
          ok = false;
          for (uint32_t tries = 0; tries < kWaitLimit && !ok; ++tries) ok = mbar_try_wait(&empty[slot], ((g / kRing) & 1u) ^ 1u);
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
    // its warps scans a quarter of the tile, so a slot is held only briefly.
    uint32_t G0 = 0;  // running number of the item's first tile
    for (int j = 0; j < my_n; ++j) {
      const int par = j & 1, st = j % 3;  // candidate buffers alternate; tables / thresholds / counts rotate over three sets
      const Item<T> it = item_of<T>(a, (int)blockIdx.x + j * (int)gridDim.x);
      const int T_ = s_tiles(it.p);
      {  // the item's table and first threshold must be there, and the item two back, which
         // used the same candidate buffers, handed over (one lane polls)
        if (lane == 0) {
          uint32_t spins = 0;
          while ((vsh[S_PREPARED] <= j || vsh[S_STREAMED] < j - 1) && !vsh[S_ABORT]) {
            if (++spins > kWaitLimit) abort_now();
            __nanosleep(64);
          }
        }
        __syncwarp();
        __threadfence_block();
      }
      if (vsh[S_ABORT]) break;
      if (tid == 0) TS(2, j);
      mbar_try_wait(&tab_full[st], (uint32_t)(j / 3) & 1u);  // (complete: every lane observes the copied table through it)
      const ItemHdr* hd = tab_hdr(st);
      uint4* stq = stash_q + warp * kStash;      // chunks this warp has set aside
      int32_t* stc = stash_c + warp * kStash;
      int nst = 0;
      ScanCtx ctx;
      ctx.bloom = tab_bloom(st);
      ctx.bw = bloom_words_of(a.hash_slots);
      ctx.touched = hd->touched;
      ctx.bans = MASKED && hd->bans != 0;
      ctx.par = par;
      ctx.mrow = MASKED ? a.mask + (size_t)(a.mask_row ? a.mask_row[it.b] : it.b) * a.mask_stride : nullptr;
      ctx.histB = xh + (2 * st) * 256;
      ctx.histA = xh + (2 * st + 1) * 256;
      ctx.baseB = (uint32_t)hd->baseB;
      ctx.baseA = (uint32_t)hd->baseA;
      ctx.sh = sh;
      ctx.q_ent = q_ent;
      ctx.status = a.status;
      ctx.id_base = a.id_base;
      const uint32_t* mrow = ctx.mrow;
      for (int t = (int)(((uint32_t)(warp / kShare) - G0) % kTeams); t < T_; t += kTeams) {
        const uint32_t g = G0 + (uint32_t)t;
        const int slot = (int)(g % kRing);
        const char* tile = ring + (size_t)slot * kSTile;
        if (!mbar_wait_warp(&full[slot], (g / kRing) & 1u)) {
          abort_now();
          break;
        }
        const int nchunk = (int)(s_tile_bytes(it.p, t) / 16u);
        const int32_t col0 = it.p.body_first + t * (kSTile / (int)sizeof(T)) + a.id_base;  // global id of the tile's first element
        // thresholds are re-read for every group of chunks: they are raised all the time
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
        constexpr int kMine = kSTile / 16 / kShare;          // chunks of a tile per warp
        constexpr int kU = kMine / 32 < 4 ? kMine / 32 : 4;   // chunks per lane per step
        const int c_lo = (warp % kShare) * kMine;
        for (int c0 = c_lo; c0 < min(nchunk, c_lo + kMine); c0 += kU * 32) {
          uint4 q[kU];
          bool h[kU];
          refresh();
#pragma unroll
          for (int u = 0; u < kU; ++u) q[u] = lds128(tile + (c0 + u * 32 + lane) * 16);  // (inside the slot even past a short tile's end)
          bool any = false;
#pragma unroll
          for (int u = 0; u < kU; ++u) {
            const int ci = c0 + u * 32 + lane;
            h[u] = Elem<T>::chunk_reaches(q[u], thB);
            if (MASKED) {
              bool hb = h[u] && ci < nchunk;
              if (hb) {
                const int32_t gid = col0 + ci * E;
                uint32_t bits = __ldg(&mrow[gid >> 5]) >> (gid & 31);
                if ((gid & 31) + E > 32) bits |= __ldg(&mrow[(gid >> 5) + 1]) << (32 - (gid & 31));
                hb = (bits & ((1u << E) - 1u)) != 0u;
              }
              h[u] = hb || Elem<T>::chunk_reaches(q[u], thA);
            }
            if (!whole) h[u] = h[u] && ci < nchunk;
            any = any || h[u];
          }
          if (__any_sync(0xFFFFFFFFu, any)) {  // set the listed chunks aside
#pragma unroll
            for (int u = 0; u < kU; ++u) {
              const unsigned all = __ballot_sync(0xFFFFFFFFu, h[u]);
              if (all == 0u) continue;
#pragma unroll
              for (int half = 0; half < 2; ++half) {  // (half a warp at a time: never more than the stash holds)
                const unsigned bal = all & (half ? 0xFFFF0000u : 0x0000FFFFu);
                if (bal == 0u) continue;
                if (nst + __popc(bal) > kStash) {  // rare: make room first
                  ctx.tcB = tcB;
                  ctx.tcA = tcA;
                  __syncwarp();
                  scan_examine<T, MASKED>(ctx, stq, stc, nst);
                  nst = 0;
                  __syncwarp();
                }
                if (h[u] && ((bal >> lane) & 1u)) {
                  const int pos = nst + __popc(bal & ((1u << lane) - 1u));
                  stq[pos] = q[u];
                  stc[pos] = col0 + (c0 + u * 32 + lane) * E;  // global id of the chunk's first element
                }
                nst += __popc(bal);
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[slot]);  // the slot can be refilled while the chunks set aside are examined
        if (nst >= kStash / 2) {  // examine in batches: full passes, and against a fresher threshold
          refresh();
          ctx.tcB = tcB;
          ctx.tcA = tcA;
          scan_examine<T, MASKED>(ctx, stq, stc, nst);
          nst = 0;
          __syncwarp();
        }
      }
      if (vsh[S_ABORT]) break;
      if (nst > 0) {  // what is still set aside
        ctx.tcB = v64[L_TAU_B + st];
        ctx.tcA = MASKED ? v64[L_TAU_A + st] : 0xFFFFFFFFFFFFFFFFull;
        __syncwarp();
        scan_examine<T, MASKED>(ctx, stq, stc, nst);
        nst = 0;
      }
      __syncwarp();
      if (tid == 0) TS(3, j);
#ifdef ARCS_TRACE
      if (lane == 0 && blockIdx.x == 0 && j < 16) atomicMax((unsigned long long*)&g_trace2[6 * 16 + j], (unsigned long long)clock64());
#endif
      if (lane == 0) {  // this warp has queued everything it found in the item
        const uint32_t e = atomicAdd(reinterpret_cast<unsigned int*>(&sh[S_QTAIL]), 1u);
        queue_write(sh, q_ent, a.status, e, 0u, kMarker | ((uint32_t)par << 31));
      }
      G0 += (uint32_t)T_;
    }
  } else if (warp == kTauWarp) {
    // =================================================================== threshold warp
    // Fetches the tables of the items ahead (an item may take a set of state once the item
    // three back has been handed over), publishes an item when its table has landed, and keeps
    // reading new thresholds off the coarse histograms of the items that are streaming: the
    // lower edge of the bin holding the k-th best survivor counted so far.
    int issued = 0, prepped = 0;
    uint32_t idle = 0;
    for (;;) {
      if (vsh[S_ABORT]) break;
      const int done = vsh[S_STREAMED];
      if (done >= my_n) break;
      __threadfence_block();
      while (issued < my_n && issued < done + 3) {
        if (lane == 0) {
          const int st = issued % 3;
          fence_proxy_async();  // the set's last readers are done (their item was handed over); order them before the copy
          mbar_expect_tx(&tab_full[st], (uint32_t)tab_bytes);
          bulk_load(tabs + (size_t)st * tab_bytes, a.ws_items + (size_t)((int)blockIdx.x + issued * (int)gridDim.x) * a.item_block,
                    (uint32_t)tab_bytes, &tab_full[st]);
        }
        ++issued;
      }
      if (prepped < issued) {
        const int st = prepped % 3;
        if (mbar_try_wait(&tab_full[st], (uint32_t)(prepped / 3) & 1u)) {
          if (lane == 0) {
            const ItemHdr* hd = tab_hdr(st);
            s64[L_TAU_B + st] = hd->tau0B;
            s64[L_TAU_A + st] = hd->tau0A;
            __threadfence_block();
            vsh[S_PREPARED] = prepped + 1;
            TS(1, prepped);
          }
          ++prepped;
          idle = 0;
          __syncwarp();
          continue;
        }
        if (prepped == done && ++idle > kWaitLimit) {  // the stream waits for this table
          abort_now();
          break;
        }
      }
      for (int j = done; j < min(prepped, done + 2); ++j) {
        const int st = j % 3;
        const ItemHdr* hd = tab_hdr(st);
        int d, kr;
        bool ex;
        find_bin(xh + (2 * st) * 256, hd->K, d, kr, ex);
        if (d > 0 && lane == 0)
          atomicMax(&s64[L_TAU_B + st], (unsigned long long)(((uint32_t)hd->baseB + (uint32_t)d) << 16) << 32);
        if (MASKED) {
          find_bin(xh + (2 * st + 1) * 256, ARCS_HEAD, d, kr, ex);
          if (d > 0 && lane == 0)
            atomicMax(&s64[L_TAU_A + st], (unsigned long long)(((uint32_t)hd->baseA + (uint32_t)d) << 16) << 32);
        }
      }
      __syncwarp();
      __nanosleep(kTauSleepNs);
    }
    // (abandoned: a table copy may still be in flight; give it a bounded chance to land)
    if (vsh[S_ABORT] && lane == 0)
      for (int x = prepped; x < issued; ++x) mbar_wait(&tab_full[x % 3], (uint32_t)(x / 3) & 1u);
  } else if (warp == kExamWarp) {
    // =================================================================== examiner
    // Owns the candidate buffers while an item streams: moves the queued survivors into them and
    // drops buffer entries the threshold has overtaken. The exact radix select runs only when a
    // buffer still overflows, i.e. when one bin holds very many equal or close keys. When every
    // scanner has closed an item, what is left goes to the item's block of the workspace.
    uint32_t head = 0, idle = 0, polls = 0;
    int streamed = 0;
    // the two items that can have entries in the queue: the older one is always served first, so
    // that items are handed over in order
    struct XItem {
      int cB, cA, marks, itm, K;
      uint32_t baseB, baseA;
      bool loaded;
      int nT, roomT;                // flagged entries written to the item's block, and the room left there
      unsigned long long* listT;
    };
    auto fresh = [](int itm) { return XItem{0, 0, 0, itm, 1, 0u, 0u, false, 0, 0, nullptr}; };
    XItem older = fresh(0), newer = fresh(1);
    constexpr int kStep = 128;     // queue entries taken per step, four per lane
    constexpr int kFullB = 512, kFullA = 1024;  // buffer fill at which stale entries are dropped
    // drop what the threshold has overtaken; if the buffer is still too full, select exactly
    auto shrink = [&](const Sel& sel, int& cnt, int full) {
      const uint64_t tc = *reinterpret_cast<volatile unsigned long long*>(sel.tau);
      int out = 0;
      for (int i0 = 0; i0 < cnt; i0 += 32) {
        const int i = i0 + lane;
        uint32_t ky = 0;
        int32_t id = 0;
        bool keep = false;
        if (i < cnt) {
          ky = sel.key[i];
          id = sel.id[i];
          keep = comp_of(ky, id) > tc;
        }
        const unsigned b = __ballot_sync(0xFFFFFFFFu, keep);  // (every lane has read its entry before any write below)
        if (keep) {
          const int pos = out + __popc(b & ((1u << lane) - 1u));
          sel.key[pos] = ky;
          sel.id[pos] = id;
        }
        out += __popc(b);
        __syncwarp();
      }
      cnt = out;
      if (full > 0 && cnt > full - kStep) cnt = sel_prune_warp(sel, cnt, sel.k, xhist, xtk, xti);
    };
    // threshold from the scanners' counts
    auto raise = [&](const Sel& sel, const uint32_t* hst, uint32_t base) {
      int d, kr;
      bool ex;
      find_bin(hst, sel.k, d, kr, ex);
      if (d <= 0) return;
      const unsigned long long tc = (unsigned long long)((base + (uint32_t)d) << 16) << 32;  // comp > tc <=> key >= edge of bin d
      if (lane == 0) atomicMax(sel.tau, tc);
      __syncwarp();
    };
    while (streamed < my_n) {
      if (vsh[S_ABORT]) break;
      const uint32_t tail = (uint32_t)vsh[S_QTAIL];
      const int avail = (int)(tail - head);
      if (avail == 0) {
        if (++idle > kWaitLimit) {
          abort_now();
          break;
        }
        __nanosleep(kExamSleepNs);
        continue;
      }
      if (avail < kStep && polls < 4) {  // let a fuller batch build up
        ++polls;
        __nanosleep(kExamSleepNs);
        continue;
      }
      idle = 0;
      polls = 0;
      const int nb = min(avail, kStep);
      uint2 ent[kStep / 32];
#pragma unroll
      for (int u = 0; u < kStep / 32; ++u) {
        const uint32_t e = head + (uint32_t)(u * 32 + lane);
        unsigned long long w = 0ull;
        if (u * 32 + lane < nb) {
          volatile unsigned long long* slot = &q_ent[e % kQueue];
          uint32_t spins = 0;  // the entry is reserved; its writer stores it right after
          while ((w = *slot) == 0ull && !vsh[S_ABORT])
            if (++spins > kWaitLimit) abort_now();
          *slot = 0ull;  // empty again before the slot is freed below
        }
        ent[u] = make_uint2((uint32_t)w, (uint32_t)(w >> 32));
      }
      __syncwarp();
      __threadfence_block();
      head += (uint32_t)nb;
      if (lane == 0) vsh[S_QHEAD] = (int)head;
      // serve one item's entries of this step; true when the item has been handed over
      auto serve = [&](XItem& x) -> bool {
        const int par = x.itm & 1, st = x.itm % 3;
        const Sel sB{bkey + par * kCapB, bid + par * kCapB, nullptr, &s64[L_TAU_B + st], x.K, 0, kCapB};
        const Sel sA{akey + par * kCapA, aid + par * kCapA, nullptr, &s64[L_TAU_A + st], ARCS_HEAD, 0, kCapA};
        bool seen = false;
        int nmark = 0;
#pragma unroll
        for (int u = 0; u < kStep / 32; ++u) {
          const bool valid = u * 32 + lane < nb && (int)(ent[u].y >> 31) == par;
          const uint32_t gid = ent[u].y & kIdMask;
          const bool marker = valid && gid == kMarker;
          nmark += __popc(__ballot_sync(0xFFFFFFFFu, marker));
          seen = seen || __any_sync(0xFFFFFFFFu, valid);
        }
        if (!seen) return false;
        if (!x.loaded) {  // first entry of a new item: its table was published before anything could be queued
          mbar_try_wait(&tab_full[st], (uint32_t)(x.itm / 3) & 1u);  // (complete: the copied table is observed through it)
          const ItemHdr* hd = tab_hdr(st);
          x.K = hd->K;
          x.baseB = (uint32_t)hd->baseB;
          x.baseA = (uint32_t)hd->baseA;
          x.listT = item_ws(a, (int)blockIdx.x + x.itm * (int)gridDim.x).pre + hd->n_pre;
          x.roomT = item_pre_cap(a.hash_slots) - hd->n_pre;
          x.loaded = true;
        }
        const Sel sBk{sB.key, sB.id, nullptr, sB.tau, x.K, 0, kCapB};
#pragma unroll
        for (int u = 0; u < kStep / 32; ++u) {
          const bool valid = u * 32 + lane < nb && (int)(ent[u].y >> 31) == par;
          const uint32_t gid = ent[u].y & kIdMask;
          const bool mine = valid && gid != kMarker;
          if (!__any_sync(0xFFFFFFFFu, mine)) continue;
          const uint64_t cm = comp_of(ent[u].x, (int32_t)gid);
          const bool tch = mine && (ent[u].y & kTch);
          if (__any_sync(0xFFFFFFFFu, tch)) {
            // flagged by the filter: straight to the item's block, raw, unless no threshold lets it matter any more.
            // (Room: the listed tokens themselves plus the filter's few false alarms among the hot elements.)
            const bool keep = tch && (cm > v64[L_TAU_B + st] || (MASKED && cm > v64[L_TAU_A + st]));
            const unsigned bt = __ballot_sync(0xFFFFFFFFu, keep);
            const int pos = x.nT + __popc(bt & ((1u << lane) - 1u));
            if (keep) {
              if (pos < x.roomT) x.listT[pos] = (unsigned long long)ent[u].x | ((unsigned long long)(ent[u].y & ~(1u << 31)) << 32);
              else raise_status(a.status, ARCS_ERR_LIST);
            }
            x.nT = min(x.nT + __popc(bt), x.roomT);
          }
          const bool okB = mine && !tch && ((ent[u].y >> 30) & 1u) && cm > v64[L_TAU_B + st];
          const unsigned bb = __ballot_sync(0xFFFFFFFFu, okB);
          if (okB) {
            const int pos = x.cB + __popc(bb & ((1u << lane) - 1u));
            sB.key[pos] = ent[u].x;
            sB.id[pos] = (int32_t)gid;
          }
          x.cB += __popc(bb);
          if (MASKED) {
            const bool okA = mine && !tch && cm > v64[L_TAU_A + st];
            const unsigned ba = __ballot_sync(0xFFFFFFFFu, okA);
            if (okA) {
              const int pos = x.cA + __popc(ba & ((1u << lane) - 1u));
              sA.key[pos] = ent[u].x;
              sA.id[pos] = (int32_t)gid;
            }
            x.cA += __popc(ba);
          }
        }
        // (the threshold warp raises the thresholds meanwhile)
        if (x.cB > kFullB - kStep) shrink(sBk, x.cB, kFullB);
        if (MASKED && x.cA > kFullA - kStep) shrink(sA, x.cA, kFullA);
        x.marks += nmark;
        if (x.marks < kScanW) return false;
        if (lane == 0) TS(5, x.itm);
        // every scanner has closed the item: write out what the last threshold has not overtaken
        raise(sBk, xh + (2 * st) * 256, x.baseB);
        shrink(sBk, x.cB, 0);
        if (a.nseg > 1 && x.cB > x.K) x.cB = sel_prune_warp(sBk, x.cB, x.K, xhist, xtk, xti);  // (a row's segments are merged later: keep their lists short)
        if (MASKED) {
          raise(sA, xh + (2 * st + 1) * 256, x.baseA);
          shrink(sA, x.cA, 0);
          if (x.cA > ARCS_HEAD) x.cA = sel_prune_warp(sA, x.cA, ARCS_HEAD, xhist, xtk, xti);
        }
        __syncwarp();
        const ItemWs w = item_ws(a, (int)blockIdx.x + x.itm * (int)gridDim.x);
        for (int i = lane; i < x.cB; i += 32)
          w.candB[i] = (unsigned long long)sB.key[i] | ((unsigned long long)((uint32_t)sB.id[i] | kOkB) << 32);
        if (MASKED)
          for (int i = lane; i < x.cA; i += 32) w.candA[i] = (unsigned long long)sA.key[i] | ((unsigned long long)(uint32_t)sA.id[i] << 32);
        if (lane == 0) {
          w.hdr->n_candB = x.cB;
          w.hdr->n_candA = MASKED ? x.cA : 0;
          w.hdr->n_tch = x.nT;
          w.hdr->tauB = *sBk.tau;
          w.hdr->tauA = *sA.tau;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) xh[(2 * st) * 256 + i * 32 + lane] = 0;  // both histograms of the item's set
        __syncwarp();
        __threadfence_block();
        ++streamed;
        if (lane == 0) vsh[S_STREAMED] = streamed;
        if (lane == 0) TS(4, x.itm);
        return true;
      };
      const bool done_o = serve(older);
      const bool done_n = serve(newer) && done_o;  // (the newer item cannot be complete before the older one)
      if (done_o) {
        const int next = newer.itm + 1;
        if (done_n) {
          older = fresh(next);
          newer = fresh(next + 1);
        } else {
          older = newer;
          newer = fresh(next);
        }
      }
    }
  }
}

}  // namespace arcs
