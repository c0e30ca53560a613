// sample_batch: penalties + temperature / top-k / top-p / min-p (+ allowed-token mask) in one
// pass over the logits.
//
// One persistent CTA per SM walks a list of work items (a row, or a segment of a row when
// there are few rows). Its warps have fixed roles and never meet at a CTA-wide barrier:
//   producer   one thread keeps a ring of 16 KB tiles filled with 1-D bulk copies (TMA);
//   scanners   16 warps take every tile from the ring; a 16-byte chunk whose maximum is
//              below the item's current threshold costs a handful of instructions, the few
//              other chunks are tested element by element and the survivors queued;
//   examiner   one warp owns the candidate buffers: it applies the exact rules to the queued
//              elements (penalised tokens are skipped here), keeps the k best under (value
//              desc, id asc) by radix select and raises the threshold the scanners read;
//   finishers  256 threads prepare the next item (table of penalised / biased tokens, first
//              threshold) and finish the previous one (exact fp32 penalty arithmetic for the
//              few touched tokens, final order, fp64 softmax, cuts, draw) while the ring keeps
//              streaming the current one.
// Items alternate between two sets of per-item state (parity), so HBM is read without pause.
#include "plan.h"
#include "select.cuh"
#include "stream.cuh"

namespace arcs {

constexpr int kScanW = 16;                                 // scanner warps
constexpr int kExamWarp = kScanW;                          // examiner warp
constexpr int kProdWarp = kScanW + 1;                      // producer warp (lane 0 works)
constexpr int kTauWarp = kScanW + 2;                       // threshold warp
constexpr int kFinWarp0 = kScanW + 3;                      // first helper warp (preparing group, then finishing group)
constexpr int kThreadsP = (kFinWarp0 + 2 * kGroup / 32) * 32;  // 864 threads
#ifndef ARCS_TAU_SLEEP
#define ARCS_TAU_SLEEP 200
#endif
constexpr int kTauSleepNs = ARCS_TAU_SLEEP;                // pause between two threshold updates
constexpr int kSortCap = 512;                              // most buffer entries ranked by counting
constexpr int kRing = kScanW;                              // tiles in the ring (a multiple of kScanW: scanner w owns slots w, w + kScanW, ...)
constexpr int kSTile = 8192;                               // bytes per tile (512 chunks: 16 per lane)
constexpr int kStash = 16;                                 // chunks a scanner sets aside per flush
constexpr int kQueue = 512;                                // queued elements between scanners and examiner
constexpr uint32_t kIdMask = 0x3FFFFFFFu;                  // queue entry word y: id | eligible-for-B << 30 | parity << 31
constexpr uint32_t kMarker = kIdMask;                      // id field of a scanner's end-of-item entry
constexpr int kCapB = 1024;   // candidate buffer: prune trigger (<= 512) + one round of pushes (<= 256)
constexpr int kCapA = 1152;   // constrained head select (k = 512): fill limit 1024 + one step / round of 128
constexpr int kBootBytes = 8192;  // prefix of an item read ahead to seed its threshold
constexpr uint32_t kEmpty = 0xFFFFFFFFu;
// per touched token: occurrences in the history (low 20 bits) and what applies to it
constexpr uint32_t kInfoCount = 0xFFFFFu, kInfoWindow = 1u << 31, kInfoBias = 1u << 30, kInfoBan = 1u << 29;

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
  unsigned int* ws_arrive;  // [B]
  char* ws_seg;             // [B][nseg] blocks of seg_block bytes
  int32_t seg_block;
  int32_t* status;
};

// layout of one (row, segment) block in the workspace
__host__ __device__ inline int32_t seg_block_bytes(bool masked) {
  return 16 + ARCS_KCAP * 8 + (masked ? ARCS_HEAD * 8 : 0);
}

// Optional role timing (build with -DARCS_ROLE_TIMING): cycles each role of CTA 0 spends in its
// phases, accumulated in registers and added to g_role[] once at the end.
#ifdef ARCS_ROLE_TIMING
__device__ unsigned long long g_role[32];
#define RT_DECL long long rt_last = clock64(); unsigned long long rt0 = 0, rt1 = 0, rt2 = 0, rt3 = 0
#define RT(i) do { const long long n_ = clock64(); const unsigned long long d_ = (unsigned long long)(n_ - rt_last); rt_last = n_; if (i == 0) rt0 += d_; else if (i == 1) rt1 += d_; else if (i == 2) rt2 += d_; else rt3 += d_; } while (0)
#define RT_COUNT(i, n) do { if (blockIdx.x == 0 && tid == 0) atomicAdd(&g_role[i], (unsigned long long)(n)); } while (0)
#define XE_T(v) const long long v = clock64()
#define XE_ADD(i, d) do { if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&g_role[i], (unsigned long long)(d)); } while (0)
#define RT_FLUSH(base, cond) do { if (blockIdx.x == 0 && (cond)) { atomicAdd(&g_role[base], rt0); atomicAdd(&g_role[base + 1], rt1); atomicAdd(&g_role[base + 2], rt2); atomicAdd(&g_role[base + 3], rt3); } } while (0)
#else
#define RT_DECL
#define RT(i)
#define RT_COUNT(i, n)
#define XE_T(v)
#define XE_ADD(i, d)
#define RT_FLUSH(base, cond)
#endif

__device__ __forceinline__ uint32_t hash_of(int32_t id, int shift) { return ((uint32_t)id * 2654435761u) >> shift; }

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// what every role derives from an item number
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

// indices into the shared scalar arrays
enum { S_ABORT = 0, S_QTAIL, S_QHEAD, S_PREPARED, S_STREAMED, S_LAST, S_FLAGS, S_NCAND, S_PICK, S_FINISHED, S_TAUACK,
       S_CNT_B /* [2] */ = 12, S_CNT_A /* [2] */ = 14,
       S_K /* [3] */ = 16, S_TOUCHED = 19, S_BANS = 22, S_BASE_B = 25, S_BASE_A = 28, S_END = 32 };
enum { L_TAU_B = 0 /* [3] */, L_TAU_A = 3, L_PRUNE_MIN = 6, L_TOP, L_LOW, L_PMIN_P, L_MROW /* [3] */ = 10, L_END = 14 };

// ---- the scanners' rare path, kept out of line so that the streaming loop stays small
struct ScanCtx {
  const uint32_t* hk;      // the item's table of replaced tokens (columns)
  const uint32_t* bloom;   // 8192-bit filter over the same columns: most lookups end here
  int32_t hash_slots, hash_shift;
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

__device__ __forceinline__ uint32_t bloom_bit(int32_t c) { return ((uint32_t)c * 0x9E3779B1u) >> 19; }  // 13 bits

__device__ __forceinline__ bool table_has(const uint32_t* hk, int32_t slots, int32_t shift, int32_t c) {
  uint32_t h = hash_of(c, shift);
  for (int probe = 0; probe < slots; ++probe) {
    const uint32_t kx = sm_ld(&hk[h]);
    if (kx == kEmpty) return false;
    if (kx == (uint32_t)c) return true;
    h = (h + 1) & (uint32_t)(slots - 1);
  }
  return false;
}

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
#ifdef ARCS_X_EMPTY
  return;
#endif
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
    // tokens the table replaces are taken from it when the item is finished, not from the stream
#ifndef ARCS_X_NOTABLE
    if ((okB || okA) && c.touched) {
      const int32_t col = gid - c.id_base;
      const uint32_t bb = bloom_bit(col);
      if (((sm_ld(&c.bloom[bb >> 5]) >> (bb & 31)) & 1u) && table_has(c.hk, c.hash_slots, c.hash_shift, col)) okB = okA = false;
    }
#endif
#ifdef ARCS_X_NOPUSH
    okB = okA = false;
#endif
    // count the survivors by the upper 16 bits of their keys: the threshold warp reads thresholds off these counts
    if (okB) sm_red_add(&c.histB[coarse_bin(ky, c.baseB)], 1u);
    if (okA) sm_red_add(&c.histA[coarse_bin(ky, c.baseA)], 1u);
    const bool pass = okB || okA;
    const unsigned pb = __ballot_sync(0xFFFFFFFFu, pass);
    if (pb) {
      const int leader = __ffs(pb) - 1;
      uint32_t base = 0;
      if (lane == leader) base = sm_atomic_add(&c.sh[S_QTAIL], (unsigned)__popc(pb));
      base = __shfl_sync(0xFFFFFFFFu, base, leader);
      if (pass)
        queue_write(c.sh, c.q_ent, c.status, base + __popc(pb & ((1u << lane) - 1u)), ky,
                    (uint32_t)gid | ((uint32_t)okB << 30) | ((uint32_t)c.par << 31));
    }
  }
}

template <typename T, bool MASKED>
__global__ void __launch_bounds__(kThreadsP, 1) sample_kernel(const SampleDev a) {
  extern __shared__ __align__(128) char smem[];
  // ---- carve shared memory (ordered by alignment)
  char* ring = smem;                                                          // kRing * kSTile
  unsigned long long* q_ent = reinterpret_cast<unsigned long long*>(ring + (size_t)kRing * kSTile);  // [kQueue]
  uint4* stash_q = reinterpret_cast<uint4*>(q_ent + kQueue);                   // [kScanW][kStash] chunks set aside by the scanners
  uint64_t* full = reinterpret_cast<uint64_t*>(stash_q + kScanW * kStash);     // [kRing] tile has landed
  uint64_t* empty = full + kRing;                                             // [kRing] tile has been scanned
  unsigned long long* s64 = reinterpret_cast<unsigned long long*>(empty + kRing);  // [L_END]
  double* spr = reinterpret_cast<double*>(s64 + L_END);                       // [ARCS_KCAP + 1]
  int32_t* stash_c = reinterpret_cast<int32_t*>(spr + ARCS_KCAP + 1);         // [kScanW][kStash]
  uint32_t* hist = reinterpret_cast<uint32_t*>(stash_c + kScanW * kStash);                                               // [512] finishers' radix histograms
  uint32_t* xhist = hist + 512;                                               // [256] examiner's radix histogram
  uint32_t* xh = xhist + 256;                                                 // [3 sets][B, A][256] coarse histograms
  uint32_t* tk = xh + 6 * 256;                                                 // [kTmpCap] finishers' scratch
  int32_t* ti = reinterpret_cast<int32_t*>(tk + kTmpCap);
  uint32_t* xtk = reinterpret_cast<uint32_t*>(ti + kTmpCap);                  // [kTmpCap] examiner's scratch
  int32_t* xti = reinterpret_cast<int32_t*>(xtk + kTmpCap);
  int* misc = reinterpret_cast<int*>(xti + kTmpCap);                          // [8]
  uint32_t* phist = reinterpret_cast<uint32_t*>(misc + 8);                    // preparing group's scratch: [512]
  uint32_t* ptk = phist + 512;                                                // [kTmpCap]
  int32_t* pti = reinterpret_cast<int32_t*>(ptk + kTmpCap);                   // [kTmpCap]
  int* pmisc = reinterpret_cast<int*>(pti + kTmpCap);                         // [8]
  int* sh = pmisc + 8;                                                        // [S_END]
  float* sv = reinterpret_cast<float*>(sh + S_END);                           // [ARCS_KCAP] sorted candidates
  int32_t* sid = reinterpret_cast<int32_t*>(sv + ARCS_KCAP);
  uint32_t* bkey = reinterpret_cast<uint32_t*>(sid + ARCS_KCAP);              // [2][kCapB]
  int32_t* bid = reinterpret_cast<int32_t*>(bkey + 2 * kCapB);
  uint32_t* akey = reinterpret_cast<uint32_t*>(bid + 2 * kCapB);              // [2][kCapA] when MASKED
  int32_t* aid = reinterpret_cast<int32_t*>(akey + (MASKED ? 2 * kCapA : 0));
  uint32_t* hkey = reinterpret_cast<uint32_t*>(aid + (MASKED ? 2 * kCapA : 0));  // [3][hash_slots] token columns
  uint32_t* hinfo = hkey + 3 * a.hash_slots;                                  // [3][hash_slots]
  uint32_t* bloom = hinfo + 3 * a.hash_slots;                                 // [3][256] filter bits over the table's columns
  volatile int* vsh = sh;
  volatile unsigned long long* v64 = s64;

  constexpr int E = Elem<T>::kPerChunk;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_items = a.B * a.nseg;
  const int my_n = (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int32_t Vg = a.v_global > 0 ? a.v_global : a.V;

  if (tid == 0) {
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init_fence();
    for (int i = 0; i < S_END; ++i) sh[i] = 0;
    for (int i = 0; i < L_END; ++i) s64[i] = 0ull;
  }
  for (int i = tid; i < kQueue; i += kThreadsP) q_ent[i] = 0ull;
  for (int i = tid; i < 6 * 256; i += kThreadsP) xh[i] = 0u;
  __syncthreads();  // the only CTA-wide barrier

  auto abort_now = [&]() {
    vsh[S_ABORT] = 1;
    raise_status(a.status, ARCS_ERR_TIMEOUT);
  };
  auto is_touched = [&](int st, int32_t c) -> bool {
    const uint32_t* hk = hkey + st * a.hash_slots;
    uint32_t h = hash_of(c, a.hash_shift);
    for (int probe = 0; probe < a.hash_slots; ++probe) {
      const uint32_t kx = hk[h];
      if (kx == kEmpty) return false;
      if (kx == (uint32_t)c) return true;
      h = (h + 1) & (uint32_t)(a.hash_slots - 1);
    }
    return false;
  };
  if (warp == kProdWarp) {
    // =================================================================== producer
    if (lane == 0) {
      RT_DECL;
      uint32_t g = 0;
      for (int j = 0; j < my_n && !vsh[S_ABORT]; ++j) {
        const Item<T> it = item_of<T>(a, (int)blockIdx.x + j * (int)gridDim.x);
        const int T_ = s_tiles(it.p);
        for (int t = 0; t < T_; ++t, ++g) {
          const int slot = (int)(g % kRing);
          if (vsh[S_ABORT]) break;
          RT(0);
          if (!mbar_wait(&empty[slot], ((g / kRing) & 1u) ^ 1u)) {
            abort_now();
            break;
          }
          RT(1);
          const uint32_t n = s_tile_bytes(it.p, t);
          mbar_expect_tx(&full[slot], n);
          bulk_load(ring + (size_t)slot * kSTile, it.p.body + (size_t)t * kSTile, n, &full[slot]);
        }
      }
      RT_FLUSH(0, true);
      if (vsh[S_ABORT]) {  // give the copies in flight a bounded chance to land before the CTA ends
        const uint32_t first = g > (uint32_t)kRing ? g - kRing : 0u;
        for (uint32_t x = first; x < g; ++x) mbar_wait(&full[x % kRing], (x / kRing) & 1u);
      }
    }
  } else if (warp < kScanW) {
    // =================================================================== scanners
    // Scanner w consumes the tiles whose running number is w modulo kScanW (its own ring slot),
    // so sixteen tiles are in work at once and no warp waits for another.
    uint32_t G0 = 0;  // running number of the item's first tile
    RT_DECL;
    for (int j = 0; j < my_n; ++j) {
      const int par = j & 1, st = j % 3;  // candidate buffers alternate; tables / thresholds / counts rotate over three sets
      const Item<T> it = item_of<T>(a, (int)blockIdx.x + j * (int)gridDim.x);
      const int T_ = s_tiles(it.p);
      RT(0);
      {  // the item's table and first threshold must be ready (one lane polls)
        if (lane == 0) {
          uint32_t spins = 0;
          // ... and the item two back, which used the same candidate buffers, must be finished
          while ((vsh[S_PREPARED] <= j || vsh[S_FINISHED] < j - 1) && !vsh[S_ABORT]) {
            if (++spins > kWaitLimit) abort_now();
            __nanosleep(64);
          }
        }
        __syncwarp();
        __threadfence_block();
      }
      RT(1);
      if (vsh[S_ABORT]) break;
      const uint32_t* mrow = MASKED ? reinterpret_cast<const uint32_t*>(s64[L_MROW + st]) : nullptr;
      const bool touched = sh[S_TOUCHED + st] != 0, bans = MASKED && sh[S_BANS + st] != 0;
      uint4* stq = stash_q + warp * kStash;      // chunks this warp has set aside
      int32_t* stc = stash_c + warp * kStash;
      int nst = 0;
      ScanCtx ctx;
      ctx.hk = hkey + st * a.hash_slots;
      ctx.bloom = bloom + st * 256;
      ctx.hash_slots = a.hash_slots;
      ctx.hash_shift = a.hash_shift;
      ctx.touched = touched;
      ctx.bans = bans;
      ctx.par = par;
      ctx.mrow = mrow;
      ctx.histB = xh + (2 * st) * 256;
      ctx.histA = xh + (2 * st + 1) * 256;
      ctx.baseB = (uint32_t)sh[S_BASE_B + st];
      ctx.baseA = (uint32_t)sh[S_BASE_A + st];
      ctx.sh = sh;
      ctx.q_ent = q_ent;
      ctx.status = a.status;
      ctx.id_base = a.id_base;
      for (int t = (int)(((uint32_t)warp - G0) % kScanW); t < T_; t += kScanW) {
        const uint32_t g = G0 + (uint32_t)t;
        const int slot = (int)(g % kRing);
        const char* tile = ring + (size_t)slot * kSTile;
        if (vsh[S_ABORT]) break;
        RT(0);
        if (!mbar_wait_warp(&full[slot], (g / kRing) & 1u)) {
          abort_now();
          break;
        }
        RT(2);
        const int nchunk = (int)(s_tile_bytes(it.p, t) / 16u);
        const int32_t col0 = it.p.body_first + t * (kSTile / (int)sizeof(T)) + a.id_base;  // global id of the tile's first element
        // thresholds are re-read for every group of chunks: the examiner raises them all the time
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
#ifndef ARCS_X_NOSCAN
        for (int c0 = 0; c0 < nchunk; c0 += 4 * 32) {
          uint4 q[4];
          bool h[4];
          refresh();
#pragma unroll
          for (int u = 0; u < 4; ++u) q[u] = lds128(tile + (c0 + u * 32 + lane) * 16);  // (inside the slot even past a short tile's end)
#pragma unroll
          for (int u = 0; u < 4; ++u) {
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
#ifdef ARCS_X_NOHOT
            h[u] = h[u] && a.V < 0;  // never true, but the test above is still evaluated
#endif
          }
          if (__any_sync(0xFFFFFFFFu, h[0] || h[1] || h[2] || h[3])) {  // set the listed chunks aside
#pragma unroll
            for (int u = 0; u < 4; ++u) {
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
#endif
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
      if (lane == 0) {  // this warp has queued everything it found in the item
        const uint32_t e = atomicAdd(reinterpret_cast<unsigned int*>(&sh[S_QTAIL]), 1u);
        queue_write(sh, q_ent, a.status, e, 0u, kMarker | ((uint32_t)par << 31));
      }
      G0 += (uint32_t)T_;
    }
    RT(0);
    RT_FLUSH(4, tid == 0);
  } else if (warp == kTauWarp) {
    // =================================================================== threshold warp
    // Keeps reading new thresholds off the coarse histograms of the items that are streaming:
    // the lower edge of the bin holding the k-th best survivor counted so far. It acknowledges
    // every hand-over, so that an item's state is recycled only after this warp is done with it.
    for (;;) {
      if (vsh[S_ABORT]) break;
      const int done = vsh[S_STREAMED];
      if (done >= my_n) break;
      const int pz = min(vsh[S_PREPARED], done + 2);
      __threadfence_block();
      for (int j = done; j < pz; ++j) {
        const int st = j % 3;
        int d, kr;
        bool ex;
        find_bin(xh + (2 * st) * 256, sh[S_K + st], d, kr, ex);
        if (d > 0 && lane == 0)
          atomicMax(&s64[L_TAU_B + st], (unsigned long long)(((uint32_t)sh[S_BASE_B + st] + (uint32_t)d) << 16) << 32);
        if (MASKED) {
          find_bin(xh + (2 * st + 1) * 256, ARCS_HEAD, d, kr, ex);
          if (d > 0 && lane == 0)
            atomicMax(&s64[L_TAU_A + st], (unsigned long long)(((uint32_t)sh[S_BASE_A + st] + (uint32_t)d) << 16) << 32);
        }
      }
      __syncwarp();
      if (lane == 0) vsh[S_TAUACK] = done;  // no threshold of an item before `done` will be written from here on
      __nanosleep(kTauSleepNs);
    }
    if (lane == 0) vsh[S_TAUACK] = my_n;
  } else if (warp == kExamWarp) {
    // =================================================================== examiner
    // Owns the candidate buffers while an item streams: moves the queued survivors into them,
    // reads a new threshold off the coarse histograms the scanners keep (the lower edge of the
    // bin that holds the k-th best survivor so far: at least k survivors are at or above it),
    // and drops buffer entries the threshold has overtaken. The exact radix select runs only
    // when a buffer still overflows, i.e. when one bin holds very many equal or close keys.
    uint32_t head = 0, idle = 0, polls = 0;
    int cB[2] = {0, 0}, cA[2] = {0, 0}, marks[2] = {0, 0}, streamed = 0;
    int kk[2] = {0, 0}, itm[2] = {0, 1};  // itm: the item each parity is on
    uint32_t baseB[2] = {0, 0}, baseA[2] = {0, 0};
    bool loaded[2] = {false, false};
    constexpr int kStep = 128;     // queue entries taken per step, four per lane
    constexpr int kFullB = 512, kFullA = 1024;  // buffer fill at which stale entries are dropped
    RT_DECL;
    unsigned long long xsteps = 0, xents = 0;
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
        __nanosleep(200);
        continue;
      }
      if (avail < kStep && polls < 4) {  // let a fuller batch build up
        ++polls;
        __nanosleep(200);
        continue;
      }
      idle = 0;
      polls = 0;
      RT(0);
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
#pragma unroll
      for (int par = 0; par < 2; ++par) {
        const int st = itm[par] % 3;
        const Sel sB{bkey + par * kCapB, bid + par * kCapB, &sh[S_CNT_B + par], &s64[L_TAU_B + st], kk[par], 0, kCapB};
        const Sel sA{akey + par * kCapA, aid + par * kCapA, &sh[S_CNT_A + par], &s64[L_TAU_A + st], ARCS_HEAD, 0, kCapA};
        bool seen = false;
        int nmark = 0;
#pragma unroll
        for (int u = 0; u < kStep / 32; ++u) {
          const bool valid = u * 32 + lane < nb && (int)(ent[u].y >> 31) == par;
          const uint32_t gid = ent[u].y & kIdMask;
          const bool marker = valid && gid == kMarker;
          const bool mine = valid && !marker;
          nmark += __popc(__ballot_sync(0xFFFFFFFFu, marker));
          if (!__any_sync(0xFFFFFFFFu, mine)) continue;
          if (!loaded[par]) {  // first entry of a new item: its settings were published before it could be queued
            loaded[par] = true;
            kk[par] = sh[S_K + st];
            baseB[par] = (uint32_t)sh[S_BASE_B + st];
            baseA[par] = (uint32_t)sh[S_BASE_A + st];
          }
          seen = true;
          const uint64_t cm = comp_of(ent[u].x, (int32_t)gid);
          const bool okB = mine && ((ent[u].y >> 30) & 1u) && cm > v64[L_TAU_B + st];
          const unsigned bb = __ballot_sync(0xFFFFFFFFu, okB);
          if (okB) {
            const int pos = cB[par] + __popc(bb & ((1u << lane) - 1u));
            sB.key[pos] = ent[u].x;
            sB.id[pos] = (int32_t)gid;
          }
          cB[par] += __popc(bb);
          if (MASKED) {
            const bool okA = mine && cm > v64[L_TAU_A + st];
            const unsigned ba = __ballot_sync(0xFFFFFFFFu, okA);
            if (okA) {
              const int pos = cA[par] + __popc(ba & ((1u << lane) - 1u));
              sA.key[pos] = ent[u].x;
              sA.id[pos] = (int32_t)gid;
            }
            cA[par] += __popc(ba);
          }
        }
        if (seen) {  // (the threshold warp raises the thresholds meanwhile)
          const Sel sBk{sB.key, sB.id, sB.cnt, sB.tau, kk[par], 0, kCapB};
          if (cB[par] > kFullB - kStep) shrink(sBk, cB[par], kFullB);
          if (MASKED && cA[par] > kFullA - kStep) shrink(sA, cA[par], kFullA);
        }
        marks[par] += nmark;
        if (marks[par] == kScanW) {  // every scanner has closed the item: hand its buffers to the finishers
          marks[par] = 0;
          if (loaded[par]) {  // leave the finishers only what the last threshold has not overtaken
            const Sel sBk{sB.key, sB.id, sB.cnt, sB.tau, kk[par], 0, kCapB};
            raise(sBk, xh + (2 * st) * 256, baseB[par]);
            shrink(sBk, cB[par], 0);
            if (MASKED) {
              raise(sA, xh + (2 * st + 1) * 256, baseA[par]);
              shrink(sA, cA[par], 0);
            }
          }
          __syncwarp();
          if (lane == 0) {
            sh[S_CNT_B + par] = cB[par];
            if (MASKED) sh[S_CNT_A + par] = cA[par];
            __threadfence_block();
            vsh[S_STREAMED] = streamed + 1;
          }
          cB[par] = cA[par] = 0;
          loaded[par] = false;
          itm[par] += 2;
#pragma unroll
          for (int x = 0; x < 16; ++x) xh[(2 * st) * 256 + x * 32 + lane] = 0;  // both histograms of the item's set
          ++streamed;
        }
      }
      RT(1);
      xsteps += 1;
      xents += nb;
    }
#ifdef ARCS_ROLE_TIMING
    rt2 = xsteps;
    rt3 = xents;
#endif
    RT_FLUSH(8, lane == 0);
  } else {
    // =================================================================== finishers
    const int gt = (tid - kFinWarp0 * 32) % kGroup;  // index inside the preparing (first) or finishing (second) group
    RT_DECL;
    const PruneScratch psF{hist, tk, ti, misc, &s64[L_PRUNE_MIN]};
    const PruneScratch psP{phist, ptk, pti, pmisc, &s64[L_PMIN_P]};

    struct RowCfg {
      arcs_row_params prm;
      int kB;
      bool greedy, k_bad, fp_on, rp_on, pp_on, pen_on, lists_ok, touched_on;
      int32_t h0, H, q0, NB;
    };
    auto row_cfg = [&](int b) {
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
    };

    // ---- prepare item j: table of the tokens the stream must not supply (every id of the
    // history a penalty applies to, every id of the bias list: tools/sampler.h:154-174) and a
    // first threshold from a short prefix of the item, read ahead of the ring.
    auto prepare = [&](int j) -> bool {
      const int st = j % 3;
      RT(0);
      {  // the item three back used the same set of state: it must be finished and acknowledged
        bool bad = false;
        if (gt == 0) {
          uint32_t spins = 0;
          while ((vsh[S_FINISHED] < j - 2 || vsh[S_TAUACK] < j - 2) && !vsh[S_ABORT]) {
            if (++spins > kWaitLimit) abort_now();
            __nanosleep(256);
          }
          bad = vsh[S_ABORT] != 0;
          __threadfence_block();
        }
        if (group_sync_or<1>(bad)) return false;
      }
      RT(1);
      const Item<T> it = item_of<T>(a, (int)blockIdx.x + j * (int)gridDim.x);
      const RowCfg r = row_cfg(it.b);
      uint32_t* hk = hkey + st * a.hash_slots;
      uint32_t* hi_ = hinfo + st * a.hash_slots;
      bool bans = false;  // Sampler::bans_: any bias entry <= -100, in range or not (tools/sampler.h:34)
      if (gt == 0) {
        if (r.k_bad) raise_status(a.status, ARCS_ERR_TOPK);
        if (!r.lists_ok) raise_status(a.status, ARCS_ERR_LIST);
        sh[S_PICK] = 0;
      }
      if (r.touched_on) {
        for (int i = gt; i < a.hash_slots; i += kGroup) {
          hk[i] = kEmpty;
          hi_[i] = 0;
        }
        for (int i = gt; i < 256; i += kGroup) bloom[st * 256 + i] = 0u;
        group_sync<1>();
        auto insert = [&](int32_t t) -> int {  // global id -> slot, -1 when it is not this segment's
          if (t < 0 || t >= Vg) return -1;
          const int32_t c = t - a.id_base;
          if (c < it.lo || c >= it.hi) return -1;
          uint32_t h = hash_of(c, a.hash_shift);
          for (int probe = 0; probe < a.hash_slots; ++probe) {
            const uint32_t old = atomicCAS(&hk[h], kEmpty, (uint32_t)c);
            if (old == kEmpty) atomicOr(&bloom[st * 256 + (bloom_bit(c) >> 5)], 1u << (bloom_bit(c) & 31));
            if (old == kEmpty || old == (uint32_t)c) return (int)h;
            h = (h + 1) & (uint32_t)(a.hash_slots - 1);
          }
          return -1;
        };
#ifndef ARCS_X_NOBUILD
        if (r.pen_on) {
          const int32_t nwin = r.prm.repeat_last_n < 0 ? r.H : min(r.H, r.prm.repeat_last_n);  // tools/sampler.h:163
          for (int i = gt; i < r.H; i += kGroup) {
            const int s = insert(a.hist_ids[r.h0 + i]);
            if (s >= 0) atomicAdd(&hi_[s], 1u);
            if (s >= 0 && i >= r.H - nwin) atomicOr(&hi_[s], kInfoWindow);
          }
        }
#endif
        for (int i = gt; i < r.NB; i += kGroup) {
          const float bv = a.bias_vals[r.q0 + i];
          bans = bans || bv <= -100.0f;
          const int s = insert(a.bias_ids[r.q0 + i]);
          if (s >= 0) atomicOr(&hi_[s], bv > -100.0f ? kInfoBias : kInfoBan);
        }
      }
      bans = group_sync_or<1>(bans);
      // first threshold: the k-th largest of 256 (or, constrained, 1024) maxima over disjoint
      // pieces of the prefix is a lower bound of the k-th best element. Tokens of the prefix that
      // the table replaces may own a maximum without counting, so that many more are skipped.
      const int nchunk = min(it.p.body_bytes, MASKED ? 2 * kBootBytes : kBootBytes) / 16;
      if (r.touched_on) {
        int extra = 0;
        const int32_t c_lo = it.p.body_first, c_hi = it.p.body_first + nchunk * E;
        for (int i = gt; i < a.hash_slots; i += kGroup) {
          const uint32_t ck = hk[i];
          extra += ck != kEmpty && (int32_t)ck >= c_lo && (int32_t)ck < c_hi;
        }
        if (extra) atomicAdd(&sh[S_PICK], extra);
        group_sync<1>();
      }
      const int kth = (MASKED ? ARCS_HEAD : r.kB) + sh[S_PICK];
      unsigned long long tau0B = 0ull, tau0A = 0ull;
      if (!MASKED) {
        // two maxima per thread, each over every other one of the thread's chunks of the prefix
        float m0 = -INFINITY, m1 = -INFINITY;
        bool any0 = false, any1 = false;
        for (int ci = gt; ci < nchunk; ci += 2 * kGroup) {
          m0 = fmaxf(m0, Elem<T>::chunk_max(ldg128_stream(it.p.body + (size_t)ci * 16)));
          any0 = true;
          if (ci + kGroup < nchunk) {
            m1 = fmaxf(m1, Elem<T>::chunk_max(ldg128_stream(it.p.body + (size_t)(ci + kGroup) * 16)));
            any1 = true;
          }
        }
        ptk[gt] = any0 ? key_of(m0) : 0u;
        ptk[kGroup + gt] = any1 ? key_of(m1) : 0u;
        group_sync<1>();
        if (kth <= min(nchunk, 2 * kGroup)) {
          const uint32_t kk0 = group_kth_key<1>(ptk, 2 * kGroup, kth, psP, gt);
          tau0B = (unsigned long long)kk0 << 32;  // keeps ties with it
        }
      }
      if (MASKED) {
        // constrained rows rank the whole vocabulary's best 512: k-th largest of up to 1024 chunk
        // maxima of the prefix (kept in this group's own scratch: the candidate buffers may still
        // belong to the item two back)
        constexpr int kKeys = 2 * kTmpCap;  // ptk and pti lie back to back
        if (kth <= nchunk && nchunk <= kKeys) {
          for (int ci = gt; ci < kKeys; ci += kGroup)
            ptk[ci] = ci < nchunk ? key_of(Elem<T>::chunk_max(ldg128_stream(it.p.body + (size_t)ci * 16))) : 0u;
          group_sync<1>();
          tau0A = (unsigned long long)group_kth_key<1>(ptk, kKeys, kth, psP, gt) << 32;  // keeps ties with it
        }
      }
      if (gt == 0) {
        s64[L_TAU_B + st] = tau0B;
        s64[L_TAU_A + st] = tau0A;
        sh[S_K + st] = r.kB;
        sh[S_TOUCHED + st] = r.touched_on;
        sh[S_BANS + st] = bans;
        sh[S_BASE_B + st] = (int)(tau0B >> 48);
        sh[S_BASE_A + st] = (int)(tau0A >> 48);
        if (MASKED)
          s64[L_MROW + st] = reinterpret_cast<unsigned long long>(a.mask + (size_t)(a.mask_row ? a.mask_row[it.b] : it.b) * a.mask_stride);
        __threadfence_block();
        vsh[S_PREPARED] = j + 1;
      }
      group_sync<1>();
      RT(2);
      return true;
    };

    // ---- finish item j once the examiner has handed its buffers over. Returns false when the
    // kernel is being abandoned (uniform over the group).
    auto finish = [&](int j) -> bool {
      const int par = j & 1, st = j % 3;
      RT(0);
      bool bad = false;
      if (gt == 0) {
        uint32_t spins = 0;
        while (vsh[S_STREAMED] <= j && !vsh[S_ABORT]) {
          if (++spins > kWaitLimit) abort_now();
          __nanosleep(256);
        }
        bad = vsh[S_ABORT] != 0;
        __threadfence_block();
      }
      if (group_sync_or<2>(bad)) return false;
      RT(3);
      const Item<T> it = item_of<T>(a, (int)blockIdx.x + j * (int)gridDim.x);
      const RowCfg r = row_cfg(it.b);
      const int b = it.b;
      const T* row = it.row;
      const SegPlan& p = it.p;
      const uint32_t* hk = hkey + st * a.hash_slots;
      const uint32_t* hi_ = hinfo + st * a.hash_slots;
      bool bans = sh[S_BANS + st] != 0;
      const uint32_t* mrow = MASKED ? reinterpret_cast<const uint32_t*>(s64[L_MROW + st]) : nullptr;
      const Sel selB{bkey + par * kCapB, bid + par * kCapB, &sh[S_CNT_B + par], &s64[L_TAU_B + st], r.kB,
                     min(512, max(2 * r.kB, r.kB + 128)), kCapB};
      const Sel selA{akey + par * kCapA, aid + par * kCapA, &sh[S_CNT_A + par], &s64[L_TAU_A + st], ARCS_HEAD, 1024, kCapA};

      bool hot = false;
      // one more element for the selections (all lanes of every finisher warp call it together);
      // v is the final (adjusted) logit, c the column; from_table: the element comes from the table
      auto consider = [&](bool valid, float v, int32_t c, bool from_table) {
        const uint32_t ky = key_of(v);
        const uint64_t cm = comp_of(ky, c + a.id_base);
        bool okB = valid && ky != 0u && cm > *selB.tau;
        bool okA = MASKED && valid && ky != 0u && cm > *selA.tau;
        if ((okB || okA) && r.touched_on && !from_table && is_touched(st, c)) okB = okA = false;
        if (MASKED && okB) {
          const int32_t g = c + a.id_base;
          okB = ((__ldg(&mrow[g >> 5]) >> (g & 31)) & 1u) && !(bans && v + 0.0f <= ARCS_BANNED);  // tools/sampler.h:118-119
        }
        sel_push(selB, okB, ky, c + a.id_base, hot, a.status);
        if (MASKED) sel_push(selA, okA, ky, c + a.id_base, hot, a.status);
      };
      // called by the whole group after a barrier behind which nobody pushes
      auto maybe_prune = [&]() {
        const bool pb = *selB.cnt > selB.trig, pa = MASKED && *selA.cnt > selA.trig;
        group_sync<2>();
        if (pb) sel_prune<2>(selB, selB.k, psF, gt);
        if (pa) sel_prune<2>(selA, selA.k, psF, gt);
      };

      // the scalar elements before the first and after the last 16-byte boundary
      {
        const bool hv = gt < p.head_n;
        consider(hv, hv ? Elem<T>::load(row + it.lo + gt) : 0.0f, it.lo + gt, false);
        const bool tv = gt < p.tail_n;
        consider(tv, tv ? Elem<T>::load(row + p.tail_first + gt) : 0.0f, p.tail_first + gt, false);
      }
      // touched tokens: exact fp32 arithmetic of Sampler::adjusted, one token per thread
#ifdef ARCS_X_NOTOUCH
      if (false) {
#else
      if (r.touched_on) {
#endif
        constexpr int R = MASKED ? 1 : 4;  // table slots per thread per batch: their logits are fetched together
        for (int s0 = 0; s0 < a.hash_slots; s0 += R * kGroup) {
          uint32_t ck[R], info[R];
          float raw[R];
#pragma unroll
          for (int x = 0; x < R; ++x) {
            const int s = s0 + x * kGroup + gt;
            ck[x] = s < a.hash_slots ? hk[s] : kEmpty;
            info[x] = ck[x] != kEmpty ? hi_[s] : 0u;
            raw[x] = ck[x] != kEmpty ? Elem<T>::load(row + (int32_t)ck[x]) : 0.0f;
          }
#pragma unroll
          for (int x = 0; x < R; ++x) {
            const bool valid = ck[x] != kEmpty;
            float v = raw[x];
            if (valid) {
              const uint32_t cnt = info[x] & kInfoCount;
              if (info[x] & kInfoBias) {  // :154-155 in list order, duplicates add again
                const int32_t g = (int32_t)ck[x] + a.id_base;
                for (int i = 0; i < r.NB; ++i)
                  if (a.bias_ids[r.q0 + i] == g && a.bias_vals[r.q0 + i] > -100.0f) v = __fadd_rn(v, a.bias_vals[r.q0 + i]);
              }
              if (r.pen_on && cnt > 0) {
                if (r.fp_on) v = __fsub_rn(v, __fmul_rn(r.prm.frequency_penalty, (float)cnt));             // :160
                if (r.rp_on && (info[x] & kInfoWindow))
                  v = v > 0.0f ? __fdiv_rn(v, r.prm.repeat_penalty) : __fmul_rn(v, r.prm.repeat_penalty);   // :166
                if (r.pp_on) v = __fsub_rn(v, r.prm.presence_penalty);                                      // :171
              }
              if (info[x] & kInfoBan) v = ARCS_BANNED;                                                      // :174
            }
            consider(valid, v, (int32_t)ck[x], true);
          }
          // at most R * kGroup pushes on top of a buffer at or below its trigger: inside its capacity
          if (group_sync_or<2>(hot)) {
            maybe_prune();
            hot = false;
          }
        }
      }
      group_sync<2>();
      if (MASKED) sel_prune<2>(selA, selA.k, psF, gt);

      // rows cut into segments: publish this segment's survivors; the CTA that arrives last merges
      if (a.nseg > 1) {
        sel_prune<2>(selB, selB.k, psF, gt);
        char* blk = a.ws_seg + ((size_t)b * a.nseg + it.seg) * a.seg_block;
        int32_t* hdr = reinterpret_cast<int32_t*>(blk);
        uint32_t* wk = reinterpret_cast<uint32_t*>(blk + 16);
        int32_t* wi = reinterpret_cast<int32_t*>(wk + ARCS_KCAP);
        const int nb = min(*selB.cnt, ARCS_KCAP), na = MASKED ? min(*selA.cnt, ARCS_HEAD) : 0;
        for (int i = gt; i < nb; i += kGroup) {
          wk[i] = selB.key[i];
          wi[i] = selB.id[i];
        }
        if (MASKED) {
          uint32_t* xk = reinterpret_cast<uint32_t*>(wi + ARCS_KCAP);
          int32_t* xi = reinterpret_cast<int32_t*>(xk + ARCS_HEAD);
          for (int i = gt; i < na; i += kGroup) {
            xk[i] = selA.key[i];
            xi[i] = selA.id[i];
          }
        }
        if (gt == 0) {
          hdr[0] = nb;
          hdr[1] = na;
          hdr[2] = bans;
        }
        __threadfence();
        group_sync<2>();
        if (gt == 0) {
          const unsigned int old = atomicAdd(&a.ws_arrive[b], 1u);
          sh[S_LAST] = old == (unsigned int)a.nseg - 1u;
          if (sh[S_LAST]) a.ws_arrive[b] = 0u;  // ready for the next launch
        }
        group_sync<2>();
        if (!sh[S_LAST]) {
          group_sync<2>();
          if (gt == 0) {
            sh[S_CNT_B + par] = 0;
            sh[S_CNT_A + par] = 0;
            __threadfence_block();
            vsh[S_FINISHED] = j + 1;
          }
          return true;
        }
        __threadfence();
        if (gt == 0) {
          *selB.cnt = 0;
          *selA.cnt = 0;
          *selB.tau = 0ull;
          *selA.tau = 0ull;
        }
        hot = false;
        for (int g = 0; g < a.nseg; ++g) {
          const char* gb = a.ws_seg + ((size_t)b * a.nseg + g) * a.seg_block;
          const int32_t* gh = reinterpret_cast<const int32_t*>(gb);
          const uint32_t* gk = reinterpret_cast<const uint32_t*>(gb + 16);
          const int32_t* gi = reinterpret_cast<const int32_t*>(gk + ARCS_KCAP);
          const int gnb = __ldcg(&gh[0]), gna = __ldcg(&gh[1]);
          bans = bans || __ldcg(&gh[2]) != 0;
          const int rounds = ((MASKED ? ARCS_HEAD : ARCS_KCAP) + kGroup - 1) / kGroup;
          for (int rr = 0; rr < rounds; ++rr) {
            group_sync<2>();
            maybe_prune();
            hot = false;
            const int i = rr * kGroup + gt;
            const bool pb = i < gnb;
            uint32_t ky = pb ? __ldcg(&gk[i]) : 0u;
            int32_t id = pb ? __ldcg(&gi[i]) : 0;
            sel_push(selB, pb && comp_of(ky, id) > *selB.tau, ky, id, hot, a.status);
            if (MASKED) {
              const uint32_t* xk = reinterpret_cast<const uint32_t*>(gi + ARCS_KCAP);
              const int32_t* xi = reinterpret_cast<const int32_t*>(xk + ARCS_HEAD);
              const bool pa = i < gna;
              ky = pa ? __ldcg(&xk[i]) : 0u;
              id = pa ? __ldcg(&xi[i]) : 0;
              sel_push(selA, pa && comp_of(ky, id) > *selA.tau, ky, id, hot, a.status);
            }
          }
        }
        group_sync<2>();
        if (MASKED) sel_prune<2>(selA, selA.k, psF, gt);
      }

      // ---- candidates best first. Up to 512 entries are ranked by counting, which selects the k
      // best and sorts them in one step; a longer buffer is cut by the radix select first.
      if (*selB.cnt > kSortCap) sel_prune<2>(selB, selB.k, psF, gt);
      group_sync<2>();
      const int nbuf = min(*selB.cnt, kSortCap);
      const int nB = min(nbuf, selB.k);
      for (int i = gt; i < nbuf; i += kGroup) {
        const uint32_t ky = selB.key[i];
        const int32_t id = selB.id[i];
        const uint64_t c = comp_of(ky, id);
        int rank = 0;
        for (int x = 0; x < nbuf; ++x) rank += comp_of(selB.key[x], selB.id[x]) > c;
        if (rank < nB) {
          sv[rank] = value_of(ky);
          sid[rank] = id;
        }
      }
      if (gt == 0) {
        s64[L_TOP] = 0ull;                    // best composite among head entries that are not skipped as banned
        s64[L_LOW] = 0xFFFFFFFFFFFFFFFFull;   // smallest composite of the head
        sh[S_FLAGS] = 0;
      }
      group_sync<2>();
      // ---- tools/sampler.h:54-77 (or :105-143)
      int flags = 0, nc = nB;
      if (MASKED) {
        const int nA = min(*selA.cnt, ARCS_HEAD);
        for (int i = gt; i < nA; i += kGroup) {
          const uint64_t c = comp_of(selA.key[i], selA.id[i]);
          if (!(bans && value_of(selA.key[i]) <= ARCS_BANNED)) atomicMax(&s64[L_TOP], (unsigned long long)c);
          atomicMin(&s64[L_LOW], (unsigned long long)c);
        }
        group_sync<2>();
        if (gt == 0) {
          const uint64_t top = s64[L_TOP], low = s64[L_LOW];
          if (top != 0ull && (nB == 0 || comp_of(key_of(sv[0]), sid[0]) != top)) flags |= ARCS_FLAG_FIRST_REFUSED;
          if (Vg > ARCS_HEAD && nA == ARCS_HEAD) {  // the scan reaches rank 512 (tools/sampler.h:106-116)
            int nh = 0;
            while (nh < nB && comp_of(key_of(sv[nh]), sid[nh]) >= low) ++nh;
            if (nh < selB.k) {
              const float l512 = value_of(comp_key(low));
              if (!r.greedy && nh > 0 && __fdiv_rn(__fsub_rn(sv[0], l512), r.prm.temperature) > 20.0f) {  // :111
                nc = nh;
                flags |= ARCS_FLAG_TAIL_SKIPPED;
              } else {
                flags |= ARCS_FLAG_TAIL_USED;
              }
            }
          }
          sh[S_NCAND] = nc;
          sh[S_FLAGS] = flags;
        }
        group_sync<2>();
        nc = sh[S_NCAND];
      } else {
        if (gt == 0) {
          if (bans)  // tools/sampler.h:54-55
            while (nc > 1 && sv[nc - 1] <= ARCS_BANNED) --nc;
          sh[S_NCAND] = nc;
        }
        group_sync<2>();
        nc = sh[S_NCAND];
      }
      {  // equal logits among the candidates kept: the reference's order there is not defined
        bool tie = false;
        for (int i = gt; i + 1 < nc; i += kGroup) tie = tie || sv[i] == sv[i + 1];
        if (tie) atomicOr(&sh[S_FLAGS], ARCS_FLAG_TIE_TOPK);
      }
      const bool draw = (!r.greedy && nc > 1) || (!MASKED && !r.greedy && nc == 1);
      if (draw) {
        const float mx = sv[0];
        for (int i = gt; i < nc; i += kGroup) {
          const float x = __fdiv_rn(__fsub_rn(sv[i], mx), r.prm.temperature);  // :60 float arithmetic
          spr[i] = (double)(float)exp((double)x);                              // float exp, widened
        }
        group_sync<2>();
        if (gt == 0) {
          double z = 0.0;
          for (int i = 0; i < nc; ++i) z = __dadd_rn(z, spr[i]);  // :58-60 in candidate order
          spr[ARCS_KCAP] = z;
        }
        group_sync<2>();
        const double z = spr[ARCS_KCAP];
        for (int i = gt; i < nc; i += kGroup) spr[i] = __ddiv_rn(spr[i], z);  // :64, the same quotients in any order
      }
      group_sync<2>();
      if (gt == 0) {
        int token = nc > 0 ? sid[0] : -1, n = nc > 0 ? 1 : 0;
        if (draw) {
          n = nc;
          double cum = 0.0;
          const double mp = __dmul_rn((double)r.prm.min_p, spr[0]);
          for (int i = 0; i < nc; ++i) {
            if (r.prm.min_p > 0.0f && spr[i] < mp) { n = max(1, i); break; }        // :65
            cum = __dadd_rn(cum, spr[i]);
            if (cum >= (double)r.prm.top_p) { n = i + 1; break; }                   // :67
          }
          double tot = 0.0;
          for (int i = 0; i < n; ++i) tot = __dadd_rn(tot, spr[i]);
          double rr = __dmul_rn(a.u[b], tot);                                       // :71-72
          int pick = n - 1;
          for (int i = 0; i < n; ++i) {
            rr = __dsub_rn(rr, spr[i]);
            if (rr <= 0.0) { pick = i; break; }
          }
          token = sid[pick];
        }
        if (r.k_bad || !r.lists_ok) token = -1;
        a.token[b] = token;
        if (a.n_cand) a.n_cand[b] = nc;
        if (a.n_kept) a.n_kept[b] = n;
      }
      group_sync<2>();
      if (gt == 0 && a.flags) a.flags[b] = sh[S_FLAGS];
      for (int i = gt; i < a.cand_stride && (a.cand_id || a.cand_val || a.cand_pr); i += kGroup) {
        const size_t o = (size_t)b * a.cand_stride + i;
        const bool in = i < nc;
        if (a.cand_id) a.cand_id[o] = in ? sid[i] : -1;
        if (a.cand_val) a.cand_val[o] = in ? sv[i] : 0.0f;
        if (a.cand_pr) a.cand_pr[o] = in ? (draw ? (float)spr[i] : (i == 0 ? 1.0f : 0.0f)) : 0.0f;
      }
      group_sync<2>();
      if (gt == 0) {
        sh[S_CNT_B + par] = 0;  // the buffers are free for the item after next
        sh[S_CNT_A + par] = 0;
        __threadfence_block();
        vsh[S_FINISHED] = j + 1;
      }
      RT(2);
      return true;
    };

    if (warp < kFinWarp0 + kGroup / 32) {
      for (int j = 0; j < my_n; ++j)
        if (!prepare(j)) break;
    } else {
      for (int j = 0; j < my_n; ++j)
        if (!finish(j)) break;
    }
    RT_FLUSH(warp < kFinWarp0 + kGroup / 32 ? 12 : 20, gt == 0);
  }
}

static size_t sample_smem_bytes(bool masked, int hash_slots) {
  size_t n = (size_t)kRing * kSTile + (size_t)kQueue * 8 + (size_t)kScanW * kStash * 20 + 2 * kRing * 8 + L_END * 8 + (ARCS_KCAP + 1) * 8 +
             (512 + 256 + 1536) * 4 + (size_t)kTmpCap * 16 + 8 * 4 + S_END * 4 + ARCS_KCAP * 8 + 512 * 4 + (size_t)kTmpCap * 8 + 8 * 4;
  n += (size_t)2 * kCapB * 8;
  if (masked) n += (size_t)2 * kCapA * 8;
  n += (size_t)3 * hash_slots * 8 + 3 * 256 * 4;
  return n + 128;
}

}  // namespace arcs

using namespace arcs;

#ifdef ARCS_ROLE_TIMING
extern "C" int arcs_debug_roles(unsigned long long* out32) {
  unsigned long long z[32] = {0};
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out32, g_role, sizeof(z));
  cudaMemcpyToSymbol(g_role, z, sizeof(z));
  return 0;
}
#endif

// Workspace layout: [0, 256) reserved; then kMaxRows arrival counters (a fixed zone, so that no
// launch of another shape ever leaves list data where a later launch keeps a counter: counters are
// the only words that must be zero between launches, and every launch leaves them zero); then the
// per-segment survivor lists, which need no initialisation.
constexpr int kMaxRows = 65536;
constexpr size_t kSegZone = 256 + (size_t)kMaxRows * 4;

extern "C" size_t arcs_sample_workspace_bytes(int32_t B, int32_t V, int32_t masked) {
  if (B <= 0 || V <= 0) return 0;
  int nseg, seg_len;
  plan_segments(B, V, &nseg, &seg_len);
  return kSegZone + (nseg > 1 ? (size_t)B * nseg * seg_block_bytes(masked != 0) : 0);
}

extern "C" int arcs_sample_batch(const arcs_sample_args* g, void* stream) {
  if (int inj = fault_injected()) return inj;
  if (!g || !g->logits || !g->params || !g->u || !g->token || g->B <= 0 || g->V <= 0 || g->row_stride < g->V ||
      (g->dtype != ARCS_F32 && g->dtype != ARCS_BF16))
    return set_error(ARCS_ERR_ARG, "sample_batch: bad argument");
  if ((g->hist_off && !g->hist_ids) || (g->bias_off && (!g->bias_ids || !g->bias_vals)))
    return set_error(ARCS_ERR_ARG, "sample_batch: list offsets without the list");
  if (g->max_hist < 0 || g->max_bias < 0 || g->max_hist > (1 << 19) || g->max_bias > (1 << 16))
    return set_error(ARCS_ERR_ARG, "sample_batch: max_hist / max_bias out of range");
  if (g->B > kMaxRows) return set_error(ARCS_ERR_ARG, "sample_batch: more than 65536 rows in one call");
  const bool masked = g->mask != nullptr;
  if (masked && g->mask_stride < (g->V + 31) / 32) return set_error(ARCS_ERR_ARG, "sample_batch: mask_stride too small");
  if (masked && (g->id_base != 0 || (g->v_global != 0 && g->v_global != g->V)))
    return set_error(ARCS_ERR_ARG, "sample_batch: a mask cannot be combined with a vocabulary shard");
  if ((g->cand_id || g->cand_val || g->cand_pr) && g->cand_stride < ARCS_KCAP)
    return set_error(ARCS_ERR_ARG, "sample_batch: cand_stride must be at least ARCS_KCAP");
  if (!g->workspace || g->workspace_bytes < arcs_sample_workspace_bytes(g->B, g->V, masked))
    return set_error(ARCS_ERR_WORKSPACE, "sample_batch: workspace too small");

  SampleDev a;
  a.logits = g->logits;
  a.row_stride = g->row_stride;
  a.B = g->B;
  a.V = g->V;
  plan_segments(g->B, g->V, &a.nseg, &a.seg_len);
  a.params = g->params;
  a.hist_off = g->hist_off;
  a.hist_ids = g->hist_ids;
  a.bias_off = g->bias_off;
  a.bias_ids = g->bias_ids;
  a.bias_vals = g->bias_vals;
  a.u = g->u;
  a.mask = g->mask;
  a.mask_row = g->mask_row;
  a.mask_stride = g->mask_stride;
  a.id_base = g->id_base;
  a.v_global = g->v_global;
  a.max_hist = g->hist_off ? g->max_hist : 0;
  a.max_bias = g->bias_off ? g->max_bias : 0;
  int slots = 32;
  while (slots < 2 * (a.max_hist + a.max_bias)) slots <<= 1;
  if (slots < kGroup) slots = kGroup;
  a.hash_slots = slots;
  a.hash_shift = 32;
  for (int s = slots; s > 1; s >>= 1) --a.hash_shift;
  a.token = g->token;
  a.n_cand = g->n_cand;
  a.n_kept = g->n_kept;
  a.flags = g->flags;
  a.cand_id = g->cand_id;
  a.cand_val = g->cand_val;
  a.cand_pr = g->cand_pr;
  a.cand_stride = g->cand_stride;
  char* ws = static_cast<char*>(g->workspace);
  a.ws_arrive = reinterpret_cast<unsigned int*>(ws + 256);
  a.ws_seg = ws + kSegZone;
  a.seg_block = seg_block_bytes(masked);
  a.status = g->status;

  const size_t smem = sample_smem_bytes(masked, slots);
  if (smem > 227 * 1024) return set_error(ARCS_ERR_LIST, "sample_batch: history / bias lists too long for the on-chip table");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int items = a.nseg * a.B;
  const dim3 grid((unsigned)(items < kSmCount ? items : kSmCount));
#define ARCS_LAUNCH(T, M)                                                                                \
  do {                                                                                                   \
    cudaError_t e = cudaFuncSetAttribute(sample_kernel<T, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e != cudaSuccess) return set_error(ARCS_ERR_CUDA, cudaGetErrorString(e));                        \
    sample_kernel<T, M><<<grid, kThreadsP, smem, st>>>(a);                                                \
  } while (0)
  if (g->dtype == ARCS_F32) {
    if (masked) ARCS_LAUNCH(float, true);
    else ARCS_LAUNCH(float, false);
  } else {
    if (masked) ARCS_LAUNCH(__nv_bfloat16, true);
    else ARCS_LAUNCH(__nv_bfloat16, false);
  }
#undef ARCS_LAUNCH
  return check_launch("sample_batch");
}
