// sample_batch: penalties + temperature / top-k / top-p / min-p (+ allowed-token mask) in one
// pass over the logits. One CTA streams one segment of one row through a ring of bulk-copied
// shared-memory tiles, keeps the exact k best (value desc, id asc) in a shared-memory buffer
// with a rising threshold, handles the few tokens touched by penalties / bias separately from
// their exact fp32 arithmetic, and finishes the row (softmax over the candidates in fp64, the
// cuts and the draw) without another launch. Rows cut into several segments are merged by the
// CTA that finishes the row last.
#include "plan.h"
#include "select.cuh"
#include "stream.cuh"

namespace arcs {

constexpr int kChunks = kTileBytes / 16 / kThreads;  // 16-byte chunks per thread per tile
constexpr int kCapB = 1024;   // candidate buffer: prune trigger (<= 512) + one round of pushes (<= 256); holds a tile's chunk maxima
constexpr int kCapA = 1280;   // constrained head select (k = 512, trigger 1024)
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

__device__ __forceinline__ uint32_t hash_of(int32_t id, int shift) { return ((uint32_t)id * 2654435761u) >> shift; }

template <typename T, bool MASKED>
__global__ void __launch_bounds__(kThreads) sample_kernel(const SampleDev a) {
  extern __shared__ __align__(128) char smem[];
  // ---- carve shared memory
  char* stage = smem;                                                  // kStages * kTileBytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage + kStages * kTileBytes);
  uint32_t* hist = reinterpret_cast<uint32_t*>(bars + kStages);        // [2][256]
  uint32_t* tk = hist + 512;
  int32_t* ti = reinterpret_cast<int32_t*>(tk + kTmpCap);
  int* misc = reinterpret_cast<int*>(ti + kTmpCap);                    // [8] prune scratch
  int* sh = misc + 8;                                                  // [24] kernel scalars
  uint32_t* bkey = reinterpret_cast<uint32_t*>(sh + 24);
  int32_t* bid = reinterpret_cast<int32_t*>(bkey + kCapB);
  uint32_t* akey = reinterpret_cast<uint32_t*>(bid + kCapB);
  int32_t* aid = reinterpret_cast<int32_t*>(akey + (MASKED ? kCapA : 0));
  uint32_t* hkey = reinterpret_cast<uint32_t*>(aid + (MASKED ? kCapA : 0));  // [hash_slots] token ids
  uint32_t* hinfo = hkey + a.hash_slots;                                      // [hash_slots]
  uint16_t* hotl = reinterpret_cast<uint16_t*>(hinfo + a.hash_slots);         // [kTileBytes / 16] chunks to examine
  // after streaming, the tile ring is reused for the sorted candidates
  float* sv = reinterpret_cast<float*>(stage);
  int32_t* sid = reinterpret_cast<int32_t*>(sv + ARCS_KCAP);
  double* spr = reinterpret_cast<double*>(sid + ARCS_KCAP);
  unsigned long long* s64 = reinterpret_cast<unsigned long long*>(spr + ARCS_KCAP);  // [2]

  // sh[] indices
  enum { S_CNT_B = 0, S_TAU_B, S_CNT_A, S_TAU_A, S_LAST, S_FLAGS, S_NCAND, S_NKEPT, S_TOKEN, S_PICK, S_HOT0, S_HOT1 };

  constexpr int E = Elem<T>::kPerChunk;
  const int tid = threadIdx.x, seg = blockIdx.x % a.nseg, b = blockIdx.x / a.nseg;
  const T* row = reinterpret_cast<const T*>(a.logits) + (size_t)b * a.row_stride;
  const int32_t lo = seg * a.seg_len, hi = min(a.V, lo + a.seg_len);
  const int32_t Vg = a.v_global > 0 ? a.v_global : a.V;
  const SegPlan p = make_plan(row, lo, hi);
  const PruneScratch ps{hist, tk, ti, misc};

  // ---- row parameters
  const arcs_row_params prm = a.params[b];
  const bool greedy = prm.temperature <= 0.0f;
  int kB;
  if (MASKED) kB = greedy ? 1 : (prm.top_k > 0 ? min(prm.top_k, Vg) : 40);       // `need`, tools/sampler.h:86
  else kB = greedy ? 1 : min(prm.top_k > 0 ? min(prm.top_k, Vg) : 256, Vg);      // tools/sampler.h:38-40
  const bool k_bad = kB > ARCS_KCAP;
  if (k_bad) kB = ARCS_KCAP;
  const bool fp_on = prm.frequency_penalty != 0.0f;
  const bool rp_on = prm.repeat_penalty != 1.0f && prm.repeat_penalty > 0.0f && prm.repeat_last_n != 0;
  const bool pp_on = prm.presence_penalty != 0.0f;
  const int32_t h0 = a.hist_off ? a.hist_off[b] : 0, H = a.hist_off ? a.hist_off[b + 1] - h0 : 0;
  const int32_t q0 = a.bias_off ? a.bias_off[b] : 0, NB = a.bias_off ? a.bias_off[b + 1] - q0 : 0;
  const bool pen_on = (fp_on || rp_on || pp_on) && H > 0;
  const bool lists_ok = H <= a.max_hist && NB <= a.max_bias;
  const bool touched_on = (pen_on || NB > 0) && lists_ok;
  const uint32_t* mrow = nullptr;
  if (MASKED) mrow = a.mask + (size_t)(a.mask_row ? a.mask_row[b] : b) * a.mask_stride;

  Sel selB{bkey, bid, &sh[S_CNT_B], reinterpret_cast<uint32_t*>(&sh[S_TAU_B]), kB, min(512, max(2 * kB, kB + 128)), kCapB};
  Sel selA{akey, aid, &sh[S_CNT_A], reinterpret_cast<uint32_t*>(&sh[S_TAU_A]), ARCS_HEAD, 1024, kCapA};

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) mbar_init(&bars[i], 1);
    mbar_init_fence();
    sh[S_CNT_B] = 0;
    sh[S_TAU_B] = 0;
    sh[S_CNT_A] = 0;
    sh[S_TAU_A] = 0;
    sh[S_LAST] = 0;
    sh[S_FLAGS] = 0;
    sh[S_PICK] = 0;
    sh[S_HOT0] = 0;
    sh[S_HOT1] = 0;
    if (k_bad) raise_status(a.status, ARCS_ERR_TOPK);
    if (!lists_ok) raise_status(a.status, ARCS_ERR_LIST);
  }
  __syncthreads();
  if (tid == 0)
    for (int t = 0; t < p.tiles && t < kStages; ++t) issue_tile(p, t, stage, bars);

  // ---- table of the tokens this segment must not take from the stream: every id of the
  // history that a penalty applies to and every id of the bias list (tools/sampler.h:154-174)
  bool bans = false;  // Sampler::bans_: any bias entry <= -100, in range or not (tools/sampler.h:34)
  if (touched_on) {
    for (int i = tid; i < a.hash_slots; i += kThreads) {
      hkey[i] = kEmpty;
      hinfo[i] = 0;
    }
    __syncthreads();
    auto insert = [&](int32_t t) -> int {  // global id -> slot, -1 when it is not this segment's
      if (t < 0 || t >= Vg) return -1;
      const int32_t c = t - a.id_base;
      if (c < lo || c >= hi) return -1;
      uint32_t h = hash_of(c, a.hash_shift);
      for (int probe = 0; probe < a.hash_slots; ++probe) {
        const uint32_t old = atomicCAS(&hkey[h], kEmpty, (uint32_t)c);
        if (old == kEmpty || old == (uint32_t)c) return (int)h;
        h = (h + 1) & (uint32_t)(a.hash_slots - 1);
      }
      return -1;
    };
    if (pen_on) {
      const int32_t nwin = prm.repeat_last_n < 0 ? H : min(H, prm.repeat_last_n);  // tools/sampler.h:163
      for (int i = tid; i < H; i += kThreads) {
        const int s = insert(a.hist_ids[h0 + i]);
        if (s >= 0) atomicAdd(&hinfo[s], 1u);
        if (s >= 0 && i >= H - nwin) atomicOr(&hinfo[s], kInfoWindow);
      }
    }
    for (int i = tid; i < NB; i += kThreads) {
      const float bv = a.bias_vals[q0 + i];
      bans = bans || bv <= -100.0f;
      const int s = insert(a.bias_ids[q0 + i]);
      if (s >= 0) atomicOr(&hinfo[s], bv > -100.0f ? kInfoBias : kInfoBan);
    }
    bans = __syncthreads_or(bans);
  }
  auto is_touched = [&](int32_t c) -> bool {
    uint32_t h = hash_of(c, a.hash_shift);
    for (int probe = 0; probe < a.hash_slots; ++probe) {
      const uint32_t kx = hkey[h];
      if (kx == kEmpty) return false;
      if (kx == (uint32_t)c) return true;
      h = (h + 1) & (uint32_t)(a.hash_slots - 1);
    }
    return false;
  };

  // ---- one element of the stream (all lanes of a warp call this together)
  // v: logit as read; c: column; `in_order`: the element arrives in increasing id order, so an
  // element equal to the smallest kept key loses to it (threshold tau_key); otherwise ties with
  // the smallest kept key must still be taken (threshold tau_key - 1).
  bool hot = false;
  auto consider = [&](bool valid, float v, int32_t c, uint32_t tauB, uint32_t tauA, bool from_table) {
    v = v + 0.0f;
    const uint32_t ky = key_of(v);
    bool okB = valid && ky >= tauB && ky != 0u;
    bool okA = MASKED && valid && ky >= tauA && ky != 0u;
    if ((okB || okA) && touched_on && !from_table && is_touched(c)) okB = okA = false;
    if (MASKED && okB) {
      const int32_t g = c + a.id_base;
      okB = ((__ldg(&mrow[g >> 5]) >> (g & 31)) & 1u) && !(bans && v <= ARCS_BANNED);  // tools/sampler.h:118-119
    }
    sel_push(selB, okB, ky, c + a.id_base, hot, a.status);
    if (MASKED) sel_push(selA, okA, ky, c + a.id_base, hot, a.status);
  };
  // Called by all threads after a barrier behind which no thread is pushing. The counts are
  // read before a second barrier so that every thread takes the same branches even though
  // threads that leave early start pushing again.
  auto maybe_prune = [&]() {
    const bool pb = sh[S_CNT_B] > selB.trig, pa = MASKED && sh[S_CNT_A] > selA.trig;
    __syncthreads();
    if (pb) sel_prune(selB, selB.k, ps);
    if (pa) sel_prune(selA, selA.k, ps);
  };

  // ---- the stream. Per tile: (A) every thread looks at its 16-byte chunks and lists the few
  // whose maximum reaches the current threshold; (B) the listed chunks are examined one
  // element per thread. Nearly all chunks fail (A), which costs a handful of instructions.
  bool failed = false;
  for (int t = 0; t < p.tiles; ++t) {
    const int slot = t % kStages;
    const char* tile = stage + (size_t)slot * kTileBytes;
    if (!mbar_wait(&bars[slot], (uint32_t)((t / kStages) & 1))) failed = true;
    const int nchunk = (int)(tile_bytes(p, t) / 16u);
    if (t == 0) {
      // Bootstrap of the threshold: the k-th largest chunk maximum is a lower bound of the
      // k-th largest element. Tokens of this tile that the table replaces may own a chunk
      // maximum without counting as candidates, so that many extra maxima are skipped.
      Sel& s0 = MASKED ? selA : selB;
      if (touched_on) {
        int extra = 0;
        const int32_t c_lo = p.body_first, c_hi = p.body_first + nchunk * E;
        for (int i = tid; i < a.hash_slots; i += kThreads) {
          const uint32_t ck = hkey[i];
          extra += ck != kEmpty && (int32_t)ck >= c_lo && (int32_t)ck < c_hi;
        }
        if (extra) atomicAdd(&sh[S_PICK], extra);
      }
      const int fail0 = __syncthreads_or(failed);
      const int kth = s0.k + sh[S_PICK];
      if (!fail0 && kth <= nchunk && nchunk <= s0.cap) {
#pragma unroll
        for (int j = 0; j < kChunks; ++j) {
          const int ci = j * kThreads + tid;
          if (ci < nchunk) {
            s0.key[ci] = key_of(Elem<T>::chunk_max(lds128(tile + ci * 16)));
            s0.id[ci] = ci;
          }
        }
        if (tid == 0) *s0.cnt = nchunk;
        __syncthreads();
        sel_prune(s0, kth, ps);
        if (tid == 0) {
          const uint32_t tk0 = *s0.tau_key;  // 1 + smallest kept maximum (0: nothing was dropped)
          *s0.tau_key = tk0 > 0u && tk0 != 0xFFFFFFFFu ? tk0 - 1u : tk0;
          *s0.cnt = 0;
        }
        __syncthreads();
      }
    }
    const uint32_t tauB = *selB.tau_key, tauA = MASKED ? *selA.tau_key : 0xFFFFFFFFu;
    const uint32_t tmin = min(tauB, tauA);
    const float tf = value_of(tmin < 0x007FFFFFu ? 0x007FFFFFu : tmin);  // -inf while nothing has been dropped
    int* hot_n = &sh[S_HOT0 + (t & 1)];
    // (A)
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
      const int ci = j * kThreads + tid;
      bool h = false;
      if (ci < nchunk && !failed) h = Elem<T>::chunk_max(lds128(tile + ci * 16)) >= tf;
      const unsigned bal = __ballot_sync(0xFFFFFFFFu, h);
      if (bal) {
        const int lane = tid & 31, leader = __ffs(bal) - 1;
        int base = 0;
        if (lane == leader) base = atomicAdd(hot_n, __popc(bal));
        base = __shfl_sync(0xFFFFFFFFu, base, leader);
        if (h) hotl[base + __popc(bal & ((1u << lane) - 1u))] = (uint16_t)ci;
      }
    }
    if (__syncthreads_or(failed)) {
      if (tid == 0) {
        raise_status(a.status, ARCS_ERR_TIMEOUT);
        drain_tiles(p, t, bars);
      }
      __syncthreads();
      return;
    }
    // (B)
    const int nhot = *hot_n;
    if (tid == 0) sh[S_HOT0 + ((t + 1) & 1)] = 0;
    const int32_t col0 = p.body_first + t * (kTileBytes / (int)sizeof(T));
    uint32_t tb = tauB, ta = tauA;
    for (int r0 = 0; r0 < nhot; r0 += kThreads / E) {
      const int qi = r0 + tid / E, e = tid % E;
      const bool valid = qi < nhot;
      float v = 0.0f;
      int32_t c = 0;
      if (valid) {
        const int ci = hotl[qi];
        v = Elem<T>::from_smem(tile + ci * 16 + e * (int)sizeof(T));
        c = col0 + ci * E + e;
      }
      consider(valid, v, c, tb, ta, false);
      if (r0 + kThreads / E < nhot) {  // more rounds: keep the buffer below its capacity
        if (__syncthreads_or(hot)) {
          maybe_prune();
          hot = false;
          // the entries kept may now come from this tile, and the chunks still listed are in no
          // particular order: a tie with the smallest kept key can still win on its id
          tb = *selB.tau_key;
          tb = tb ? tb - 1u : 0u;
          ta = MASKED ? *selA.tau_key : 0xFFFFFFFFu;
          ta = MASKED && ta ? ta - 1u : ta;
        }
      }
    }
    // every thread is done with the tile: refill the slot, prune if the buffer has grown
    const int any = __syncthreads_or(hot);
    if (tid == 0 && t + kStages < p.tiles) issue_tile(p, t + kStages, stage, bars);
    if (any) {
      maybe_prune();
      hot = false;
    }
  }
  // ---- the scalar elements after the last and before the first 16-byte boundary. The tail
  // follows the stream in id order; the head has the lowest ids of the segment, so there a tie
  // with the smallest kept key must still be taken.
  {
    __syncthreads();
    maybe_prune();
    hot = false;
    const bool valid = tid < p.tail_n;
    const float v = valid ? Elem<T>::load(row + p.tail_first + tid) : 0.0f;
    consider(valid, v, p.tail_first + tid, *selB.tau_key, MASKED ? *selA.tau_key : 0u, false);
    __syncthreads();
    maybe_prune();
    hot = false;
    const bool hvalid = tid < p.head_n;
    const float hv = hvalid ? Elem<T>::load(row + lo + tid) : 0.0f;
    const uint32_t tb = *selB.tau_key, ta = MASKED ? *selA.tau_key : 0u;
    consider(hvalid, hv, lo + tid, tb ? tb - 1u : 0u, ta ? ta - 1u : 0u, false);
  }

  // ---- touched tokens: exact fp32 arithmetic of Sampler::adjusted, one token per thread
  if (touched_on) {
    for (int s0 = 0; s0 < a.hash_slots; s0 += kThreads) {
      __syncthreads();
      maybe_prune();
      hot = false;
      const int s = s0 + tid;
      const uint32_t ck = hkey[s];
      const bool valid = ck != kEmpty;
      float v = 0.0f;
      if (valid) {
        const uint32_t info = hinfo[s];
        const uint32_t cnt = info & kInfoCount;
        v = Elem<T>::load(row + (int32_t)ck);
        if (info & kInfoBias) {  // :154-155 in list order, duplicates add again
          const int32_t g = (int32_t)ck + a.id_base;
          for (int i = 0; i < NB; ++i)
            if (a.bias_ids[q0 + i] == g && a.bias_vals[q0 + i] > -100.0f) v = __fadd_rn(v, a.bias_vals[q0 + i]);
        }
        if (pen_on && cnt > 0) {
          if (fp_on) v = __fsub_rn(v, __fmul_rn(prm.frequency_penalty, (float)cnt));             // :160
          if (rp_on && (info & kInfoWindow))
            v = v > 0.0f ? __fdiv_rn(v, prm.repeat_penalty) : __fmul_rn(v, prm.repeat_penalty);   // :166
          if (pp_on) v = __fsub_rn(v, prm.presence_penalty);                                      // :171
        }
        if (info & kInfoBan) v = ARCS_BANNED;                                                     // :174
      }
      // these ids are not in stream order: a tie with the smallest kept key must still be taken
      const uint32_t tb = *selB.tau_key, ta = MASKED ? *selA.tau_key : 0u;
      consider(valid, v, (int32_t)ck, tb ? tb - 1u : 0u, ta ? ta - 1u : 0u, true);
    }
  }
  __syncthreads();
  sel_prune(selB, selB.k, ps);
  if (MASKED) sel_prune(selA, selA.k, ps);
  __syncthreads();

  // ---- rows cut into segments: publish this segment's survivors; the last CTA merges them
  if (a.nseg > 1) {
    char* blk = a.ws_seg + ((size_t)b * a.nseg + seg) * a.seg_block;
    int32_t* hdr = reinterpret_cast<int32_t*>(blk);
    uint32_t* wk = reinterpret_cast<uint32_t*>(blk + 16);
    int32_t* wi = reinterpret_cast<int32_t*>(wk + ARCS_KCAP);
    const int nb = min(sh[S_CNT_B], ARCS_KCAP), na = MASKED ? min(sh[S_CNT_A], ARCS_HEAD) : 0;
    for (int i = tid; i < nb; i += kThreads) {
      wk[i] = bkey[i];
      wi[i] = bid[i];
    }
    if (MASKED) {
      uint32_t* xk = reinterpret_cast<uint32_t*>(wi + ARCS_KCAP);
      int32_t* xi = reinterpret_cast<int32_t*>(xk + ARCS_HEAD);
      for (int i = tid; i < na; i += kThreads) {
        xk[i] = akey[i];
        xi[i] = aid[i];
      }
    }
    if (tid == 0) {
      hdr[0] = nb;
      hdr[1] = na;
      hdr[2] = bans;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const unsigned int old = atomicAdd(&a.ws_arrive[b], 1u);
      sh[S_LAST] = old == (unsigned int)a.nseg - 1u;
      if (sh[S_LAST]) a.ws_arrive[b] = 0u;  // ready for the next launch
    }
    __syncthreads();
    if (!sh[S_LAST]) return;
    __threadfence();
    if (tid == 0) {
      sh[S_CNT_B] = 0;
      sh[S_TAU_B] = 0;
      sh[S_CNT_A] = 0;
      sh[S_TAU_A] = 0;
    }
    hot = false;
    for (int g = 0; g < a.nseg; ++g) {
      const char* gb = a.ws_seg + ((size_t)b * a.nseg + g) * a.seg_block;
      const int32_t* gh = reinterpret_cast<const int32_t*>(gb);
      const uint32_t* gk = reinterpret_cast<const uint32_t*>(gb + 16);
      const int32_t* gi = reinterpret_cast<const int32_t*>(gk + ARCS_KCAP);
      const int gnb = __ldcg(&gh[0]), gna = __ldcg(&gh[1]);
      bans = bans || __ldcg(&gh[2]) != 0;
      const int rounds = MASKED ? (ARCS_HEAD + kThreads - 1) / kThreads : 1;
      for (int r = 0; r < rounds; ++r) {
        __syncthreads();
        maybe_prune();
        hot = false;
        const int i = r * kThreads + tid;
        const uint32_t tb = *selB.tau_key;
        const bool pb = i < gnb;
        uint32_t ky = pb ? __ldcg(&gk[i]) : 0u;
        sel_push(selB, pb && ky >= (tb ? tb - 1u : 0u), ky, pb ? __ldcg(&gi[i]) : 0, hot, a.status);
        if (MASKED) {
          const uint32_t* xk = reinterpret_cast<const uint32_t*>(gi + ARCS_KCAP);
          const int32_t* xi = reinterpret_cast<const int32_t*>(xk + ARCS_HEAD);
          const uint32_t ta = *selA.tau_key;
          const bool pa = i < gna;
          ky = pa ? __ldcg(&xk[i]) : 0u;
          sel_push(selA, pa && ky >= (ta ? ta - 1u : 0u), ky, pa ? __ldcg(&xi[i]) : 0, hot, a.status);
        }
      }
    }
    __syncthreads();
    sel_prune(selB, selB.k, ps);
    if (MASKED) sel_prune(selA, selA.k, ps);
    __syncthreads();
  }

  // ---- finish the row: candidates best first, then tools/sampler.h:54-77 (or :105-143)
  int nB = min(sh[S_CNT_B], selB.k);
  sel_sort(selB, nB, sv, sid);
  if (tid == 0) {
    s64[0] = 0ull;                    // best composite among head entries that are not skipped as banned
    s64[1] = 0xFFFFFFFFFFFFFFFFull;   // smallest composite of the head
  }
  __syncthreads();
  int flags = 0, nc = nB;
  if (MASKED) {
    const int nA = min(sh[S_CNT_A], ARCS_HEAD);
    for (int i = tid; i < nA; i += kThreads) {
      const uint64_t c = comp_of(akey[i], aid[i]);
      if (!(bans && value_of(akey[i]) <= ARCS_BANNED)) atomicMax(&s64[0], (unsigned long long)c);
      atomicMin(&s64[1], (unsigned long long)c);
    }
    __syncthreads();
    if (tid == 0) {
      const uint64_t top = s64[0], low = s64[1];
      if (top != 0ull && (nB == 0 || comp_of(key_of(sv[0]), sid[0]) != top)) flags |= ARCS_FLAG_FIRST_REFUSED;
      if (Vg > ARCS_HEAD && nA == ARCS_HEAD) {  // the scan reaches rank 512 (tools/sampler.h:106-116)
        int nh = 0;
        while (nh < nB && comp_of(key_of(sv[nh]), sid[nh]) >= low) ++nh;
        if (nh < selB.k) {
          const float l512 = value_of(comp_key(low));
          if (!greedy && nh > 0 && __fdiv_rn(__fsub_rn(sv[0], l512), prm.temperature) > 20.0f) {  // :111
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
    __syncthreads();
    nc = sh[S_NCAND];
  } else {
    if (tid == 0) {
      if (bans)  // tools/sampler.h:54-55
        while (nc > 1 && sv[nc - 1] <= ARCS_BANNED) --nc;
      sh[S_NCAND] = nc;
    }
    __syncthreads();
    nc = sh[S_NCAND];
  }
  // equal logits among the candidates kept: the reference's order there is not defined
  {
    bool tie = false;
    for (int i = tid; i + 1 < nc; i += kThreads) tie = tie || sv[i] == sv[i + 1];
    if (tie) atomicOr(&sh[S_FLAGS], ARCS_FLAG_TIE_TOPK);
  }
  const bool draw = !greedy && nc > 1 || (!MASKED && !greedy && nc == 1);
  if (draw) {
    const float mx = sv[0];
    for (int i = tid; i < nc; i += kThreads) {
      const float x = __fdiv_rn(__fsub_rn(sv[i], mx), prm.temperature);  // :60 float arithmetic
      spr[i] = (double)(float)exp((double)x);                            // float exp, widened
    }
  }
  __syncthreads();
  if (tid == 0) {
    int token = nc > 0 ? sid[0] : -1, n = nc > 0 ? 1 : 0;
    if (draw) {
      double z = 0.0;
      for (int i = 0; i < nc; ++i) z = __dadd_rn(z, spr[i]);
      for (int i = 0; i < nc; ++i) spr[i] = __ddiv_rn(spr[i], z);
      n = nc;
      double cum = 0.0;
      const double mp = __dmul_rn((double)prm.min_p, spr[0]);
      for (int i = 0; i < nc; ++i) {
        if (prm.min_p > 0.0f && spr[i] < mp) { n = max(1, i); break; }          // :65
        cum = __dadd_rn(cum, spr[i]);
        if (cum >= (double)prm.top_p) { n = i + 1; break; }                     // :67
      }
      double tot = 0.0;
      for (int i = 0; i < n; ++i) tot = __dadd_rn(tot, spr[i]);
      double r = __dmul_rn(a.u[b], tot);                                        // :71-72
      int pick = n - 1;
      for (int i = 0; i < n; ++i) {
        r = __dsub_rn(r, spr[i]);
        if (r <= 0.0) { pick = i; break; }
      }
      token = sid[pick];
    }
    if (k_bad || !lists_ok) token = -1;
    a.token[b] = token;
    if (a.n_cand) a.n_cand[b] = nc;
    if (a.n_kept) a.n_kept[b] = n;
    sh[S_NKEPT] = n;
  }
  __syncthreads();
  if (tid == 0 && a.flags) a.flags[b] = sh[S_FLAGS];
  for (int i = tid; i < a.cand_stride && (a.cand_id || a.cand_val || a.cand_pr); i += kThreads) {
    const size_t o = (size_t)b * a.cand_stride + i;
    const bool in = i < nc;
    if (a.cand_id) a.cand_id[o] = in ? sid[i] : -1;
    if (a.cand_val) a.cand_val[o] = in ? sv[i] : 0.0f;
    if (a.cand_pr) a.cand_pr[o] = in ? (draw ? (float)spr[i] : (i == 0 ? 1.0f : 0.0f)) : 0.0f;
  }
}

static size_t sample_smem_bytes(bool masked, int hash_slots) {
  size_t n = (size_t)kStages * kTileBytes + kStages * 8 + 512 * 4 + (size_t)kTmpCap * 8 + 8 * 4 + 24 * 4;
  n += (size_t)kCapB * 8;
  if (masked) n += (size_t)kCapA * 8;
  n += (size_t)hash_slots * 8;
  n += (size_t)(kTileBytes / 16) * 2;
  return n + 128;
}

}  // namespace arcs

using namespace arcs;

extern "C" size_t arcs_sample_workspace_bytes(int32_t B, int32_t V, int32_t masked) {
  if (B <= 0 || V <= 0) return 0;
  int nseg, seg_len;
  plan_segments(B, V, &nseg, &seg_len);
  return 256 + (size_t)B * 4 + 256 + (nseg > 1 ? (size_t)B * nseg * seg_block_bytes(masked != 0) : 0);
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
  if (slots < kThreads) slots = kThreads;
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
  a.ws_seg = ws + 256 + (((size_t)g->B * 4 + 255) / 256) * 256;
  a.seg_block = seg_block_bytes(masked);
  a.status = g->status;

  const size_t smem = sample_smem_bytes(masked, slots);
  if (smem > 227 * 1024) return set_error(ARCS_ERR_LIST, "sample_batch: history / bias lists too long for the on-chip table");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid((unsigned)a.nseg * (unsigned)a.B);
#define ARCS_LAUNCH(T, M)                                                                                \
  do {                                                                                                   \
    cudaError_t e = cudaFuncSetAttribute(sample_kernel<T, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e != cudaSuccess) return set_error(ARCS_ERR_CUDA, cudaGetErrorString(e));                        \
    sample_kernel<T, M><<<grid, kThreads, smem, st>>>(a);                                                \
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
