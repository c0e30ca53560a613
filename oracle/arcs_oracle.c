/*
 * CPU oracle for the token-selection path (see arcs_oracle.h for scope and parity status).
 * TEST INFRASTRUCTURE ONLY. Plain C, single thread, written for clarity, not speed.
 * Build: gcc -O2 -ffp-contract=off -fPIC -shared (no -ffast-math, no -march=native: every
 * float operation below must round exactly once, as in the reference's /fp:precise build).
 */
#include "arcs_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ---------------------------------------------------------------- mt19937_64 */
/* Matsumoto & Nishimura's 64-bit Mersenne Twister, the generator std::mt19937_64 names
 * (Sampler::rng_, tools/sampler.h:202). */
#define MT_N 312
#define MT_M 156
typedef struct {
  uint64_t s[MT_N];
  int i;
} mt64;

static void mt64_seed(mt64* g, uint64_t seed) {
  g->s[0] = seed;
  for (int i = 1; i < MT_N; ++i)
    g->s[i] = 6364136223846793005ull * (g->s[i - 1] ^ (g->s[i - 1] >> 62)) + (uint64_t)i;
  g->i = MT_N;
}
static uint64_t mt64_next(mt64* g) {
  if (g->i >= MT_N) {
    for (int i = 0; i < MT_N; ++i) {
      uint64_t x = (g->s[i] & 0xFFFFFFFF80000000ull) | (g->s[(i + 1) % MT_N] & 0x7FFFFFFFull);
      uint64_t xa = x >> 1;
      if (x & 1ull) xa ^= 0xB5026F5AA96619E9ull;
      g->s[i] = g->s[(i + MT_M) % MT_N] ^ xa;
    }
    g->i = 0;
  }
  uint64_t y = g->s[g->i++];
  y ^= (y >> 29) & 0x5555555555555555ull;
  y ^= (y << 17) & 0x71D67FFFEDA60000ull;
  y ^= (y << 37) & 0xFFF7EEE000000000ull;
  y ^= y >> 43;
  return y;
}

void orc_mt64_u01(uint64_t seed, int n, double* out) {
  mt64 g;
  mt64_seed(&g, seed);
  for (int i = 0; i < n; ++i) {
    /* libstdc++ generate_canonical<double,53> on a 64-bit engine: one word divided by 2^64,
     * rounded to double once, and a result of 1.0 replaced by the double just below it */
    double u = (double)mt64_next(&g) * 5.42101086242752217e-20; /* 2^-64, exact scaling */
    if (u >= 1.0) u = nextafter(1.0, 0.0);
    out[i] = u;
  }
}

/* ---------------------------------------------------------------- adjusted() */
int orc_adjusted(const float* logits, int V, const orc_params* p, const int32_t* hist, int H,
                 const int32_t* bias_id, const float* bias_val, int nb, float* out) {
  /* tools/sampler.h:148-151: which stages are on; nothing on = the input itself */
  const int fp = p->frequency_penalty != 0.0f;
  const int rp = p->repeat_penalty != 1.0f && p->repeat_penalty > 0.0f && p->repeat_last_n != 0;
  const int pp = p->presence_penalty != 0.0f;
  memcpy(out, logits, (size_t)V * sizeof(float));
  if (!fp && !rp && !pp && nb == 0) return 0;
  /* :154-155 bias entries above -100, in list order, duplicates add again */
  for (int i = 0; i < nb; ++i)
    if (bias_id[i] >= 0 && bias_id[i] < V && bias_val[i] > -100.0f) out[bias_id[i]] += bias_val[i];
  int32_t* cnt = (int32_t*)calloc((size_t)(V > 0 ? V : 1), sizeof(int32_t));
  uint8_t* done = (uint8_t*)calloc((size_t)(V > 0 ? V : 1), 1);
  if (fp) { /* :156-161 once per distinct id, count over the whole history */
    for (int i = 0; i < H; ++i)
      if (hist[i] >= 0 && hist[i] < V) ++cnt[hist[i]];
    for (int i = 0; i < H; ++i) {
      const int t = hist[i];
      if (t < 0 || t >= V || done[t]) continue;
      done[t] = 1;
      const float m = p->frequency_penalty * (float)cnt[t];
      out[t] = out[t] - m;
    }
    for (int i = 0; i < H; ++i)
      if (hist[i] >= 0 && hist[i] < V) done[hist[i]] = 0;
  }
  if (rp) { /* :162-167 distinct ids among the last n entries */
    const int n = p->repeat_last_n < 0 ? H : (H < p->repeat_last_n ? H : p->repeat_last_n);
    for (int i = H - n; i < H; ++i) {
      const int t = hist[i];
      if (t < 0 || t >= V || done[t]) continue;
      done[t] = 1;
      out[t] = out[t] > 0.0f ? out[t] / p->repeat_penalty : out[t] * p->repeat_penalty;
    }
    for (int i = H - n; i < H; ++i)
      if (hist[i] >= 0 && hist[i] < V) done[hist[i]] = 0;
  }
  if (pp) { /* :168-172 once per distinct id of the whole history */
    for (int i = 0; i < H; ++i) {
      const int t = hist[i];
      if (t < 0 || t >= V || done[t]) continue;
      done[t] = 1;
      out[t] = out[t] - p->presence_penalty;
    }
  }
  /* :173-174 bans last */
  for (int i = 0; i < nb; ++i)
    if (bias_id[i] >= 0 && bias_id[i] < V && bias_val[i] <= -100.0f) out[bias_id[i]] = ORC_BANNED;
  free(cnt);
  free(done);
  return 1;
}

static int has_ban(const float* bias_val, int nb) { /* Sampler::bans_, tools/sampler.h:34 */
  for (int i = 0; i < nb; ++i)
    if (bias_val[i] <= -100.0f) return 1;
  return 0;
}

/* ---------------------------------------------------------------- ordering */
/* The K best ids of l[0..V) under (value descending, id ascending), best first. One pass
 * that keeps a sorted list: a later id replaces nothing it merely ties with, which is the
 * stated total order (the same rule as the one-pass top-K of zero/engine_drafters.h:476-484). */
static int top_ids(const float* l, int V, int K, int32_t* idx) {
  int n = 0;
  for (int i = 0; i < V; ++i) {
    const float v = l[i];
    if (n == K && !(v > l[idx[K - 1]])) continue;
    int j = n < K ? n++ : K - 1;
    while (j > 0 && l[idx[j - 1]] < v) {
      idx[j] = idx[j - 1];
      --j;
    }
    idx[j] = i;
  }
  return n;
}

static const float* g_sort_l;
static int cmp_desc(const void* a, const void* b) {
  const int32_t x = *(const int32_t*)a, y = *(const int32_t*)b;
  if (g_sort_l[x] > g_sort_l[y]) return -1;
  if (g_sort_l[x] < g_sort_l[y]) return 1;
  return x < y ? -1 : (x > y ? 1 : 0);
}

int32_t orc_argmax(const float* row, int V) {
  int32_t b = 0;
  for (int i = 1; i < V; ++i)
    if (row[i] > row[b]) b = i;
  return V > 0 ? b : -1;
}

/* ---------------------------------------------------------------- softmax / cut / draw */
/* tools/sampler.h:57-77 (and :123-143): v[] are the candidates' logits in order */
static int draw_from(const float* v, int k, const orc_params* p, double u, int* n_kept, double* pr) {
  const float mx = v[0];
  double z = 0;
  for (int i = 0; i < k; ++i) {
    const float a = (v[i] - mx) / p->temperature;
    pr[i] = (double)expf(a);
    z += pr[i];
  }
  /* the reference divides pr[i] by z inside the cut loop and leaves the entries after the
   * cut undivided; they are never read again there, so dividing all of them first gives the
   * same kept values and lets the caller see every candidate's probability */
  for (int i = 0; i < k; ++i) pr[i] /= z;
  int n = k;
  double cum = 0;
  for (int i = 0; i < k; ++i) {
    if (p->min_p > 0 && pr[i] < (double)p->min_p * pr[0]) { /* :65 */
      n = i > 1 ? i : 1;
      break;
    }
    cum += pr[i];
    if (cum >= (double)p->top_p) { /* :67 */
      n = i + 1;
      break;
    }
  }
  double tot = 0;
  for (int i = 0; i < n; ++i) tot += pr[i];
  double r = u * tot;
  *n_kept = n;
  for (int i = 0; i < n; ++i) {
    r -= pr[i];
    if (r <= 0) return i;
  }
  return n - 1;
}

void orc_sample(const float* logits, int V, const orc_params* p, const int32_t* hist, int H,
                const int32_t* bias_id, const float* bias_val, int nb, double u,
                orc_result* res, int32_t* cand_id, double* cand_pr) {
  res->token = -1;
  res->n_cand = res->n_kept = res->flags = 0;
  if (V <= 0) return;
  float* adj = (float*)malloc((size_t)V * sizeof(float));
  orc_adjusted(logits, V, p, hist, H, bias_id, bias_val, nb, adj);
  if (p->temperature <= 0.0f) { /* :38 */
    res->token = orc_argmax(adj, V);
    res->n_cand = res->n_kept = 1;
    if (cand_id) cand_id[0] = res->token;
    if (cand_pr) cand_pr[0] = 1.0;
    free(adj);
    return;
  }
  int k = p->top_k > 0 ? (p->top_k < V ? p->top_k : V) : 256; /* :40 */
  if (k > V) k = V; /* the reference assumes V >= 256 here; the batched API defines min(k, V) */
  int32_t* idx = (int32_t*)malloc((size_t)(k + 2) * sizeof(int32_t));
  const int kk = top_ids(adj, V, k + 1 <= V ? k + 1 : k, idx); /* one extra: tie at the cut */
  for (int i = 0; i + 1 < kk; ++i)
    if (adj[idx[i]] == adj[idx[i + 1]]) res->flags |= ORC_FLAG_TIE_TOPK;
  if (has_ban(bias_val, nb)) /* :54-55 */
    while (k > 1 && adj[idx[k - 1]] <= ORC_BANNED) --k;
  float* v = (float*)malloc((size_t)k * sizeof(float));
  double* pr = (double*)malloc((size_t)k * sizeof(double));
  for (int i = 0; i < k; ++i) v[i] = adj[idx[i]];
  int n = k;
  const int pick = draw_from(v, k, p, u, &n, pr);
  res->token = idx[pick];
  res->n_cand = k;
  res->n_kept = n;
  for (int i = 0; i < k; ++i) {
    if (cand_id) cand_id[i] = idx[i];
    if (cand_pr) cand_pr[i] = pr[i];
  }
  free(adj);
  free(idx);
  free(v);
  free(pr);
}

void orc_sample_allowed(const float* logits, int V, const orc_params* p, const int32_t* hist, int H,
                        const int32_t* bias_id, const float* bias_val, int nb,
                        const uint32_t* allowed, double u, orc_result* res, int32_t* cand_id,
                        double* cand_pr) {
  res->token = -1;
  res->n_cand = res->n_kept = res->flags = 0;
  if (V <= 0) return; /* :85 */
  float* adj = (float*)malloc((size_t)V * sizeof(float));
  orc_adjusted(logits, V, p, hist, H, bias_id, bias_val, nb, adj);
  const int greedy = p->temperature <= 0.0f;
  const int need = greedy ? 1 : (p->top_k > 0 ? (p->top_k < V ? p->top_k : V) : 40); /* :86 */
  const int head = V < 512 ? V : 512;                                                /* :93 */
  int32_t* order = (int32_t*)malloc((size_t)V * sizeof(int32_t));
  top_ids(adj, V, head, order); /* :94-103 in the stated total order */
  const int bans = has_ban(bias_val, nb);
  int32_t* c = (int32_t*)malloc((size_t)(need + 1) * sizeof(int32_t));
  int nc = 0, first = 1;
  for (int r = 0; r < V && nc < need; ++r) { /* :105-120 */
    if (r == head) {
      if (nc > 0 && (adj[c[0]] - adj[order[head - 1]]) / p->temperature > 20.0f) { /* :111 */
        res->flags |= ORC_FLAG_TAIL_SKIPPED;
        break;
      }
      res->flags |= ORC_FLAG_TAIL_USED;
      for (int i = 0; i < V; ++i) order[i] = i; /* :112-115 the rest, sorted */
      g_sort_l = adj;
      qsort(order, (size_t)V, sizeof(int32_t), cmp_desc);
    }
    const int t = order[r];
    if (bans && adj[t] <= ORC_BANNED) continue; /* :118 */
    const int ok = (allowed[t >> 5] >> (t & 31)) & 1u;
    if (first && !ok) res->flags |= ORC_FLAG_FIRST_REFUSED; /* tools/server_chat.h:542 */
    first = 0;
    if (ok) c[nc++] = t;
  }
  for (int i = 0; i + 1 < nc; ++i)
    if (adj[c[i]] == adj[c[i + 1]]) res->flags |= ORC_FLAG_TIE_TOPK;
  /* Where the reference's examination order is not defined: an eligible token outside the
   * candidate set equal to the last candidate (TIE_TOPK), two equal best tokens or a tie
   * across the rank-512 boundary (TIE_HEAD). */
  {
    int top = -1, ntop = 0;
    for (int t = 0; t < V; ++t) {
      if (bans && adj[t] <= ORC_BANNED) continue;
      if (top < 0 || adj[t] > adj[top]) { top = t; ntop = 1; }
      else if (adj[t] == adj[top]) ++ntop;
      if (nc > 0 && ((allowed[t >> 5] >> (t & 31)) & 1u) && adj[t] == adj[c[nc - 1]]) {
        int in = 0;
        for (int i = 0; i < nc; ++i) in |= c[i] == t;
        if (!in) res->flags |= ORC_FLAG_TIE_TOPK;
      }
    }
    if (ntop > 1) res->flags |= ORC_FLAG_TIE_HEAD;
    if (V > head) {
      int32_t* h2 = (int32_t*)malloc((size_t)(head + 1) * sizeof(int32_t));
      top_ids(adj, V, head + 1, h2);
      if (adj[h2[head - 1]] == adj[h2[head]]) res->flags |= ORC_FLAG_TIE_HEAD;
      free(h2);
    }
  }
  res->n_cand = nc;
  if (nc == 0) { /* :121 */
    free(adj);
    free(order);
    free(c);
    return;
  }
  if (greedy || nc == 1) { /* :122 no draw */
    res->token = c[0];
    res->n_kept = 1;
    for (int i = 0; i < nc; ++i) {
      if (cand_id) cand_id[i] = c[i];
      if (cand_pr) cand_pr[i] = i == 0 ? 1.0 : 0.0;
    }
    free(adj);
    free(order);
    free(c);
    return;
  }
  float* v = (float*)malloc((size_t)nc * sizeof(float));
  double* pr = (double*)malloc((size_t)nc * sizeof(double));
  for (int i = 0; i < nc; ++i) v[i] = adj[c[i]];
  int n = nc;
  const int pick = draw_from(v, nc, p, u, &n, pr); /* :123-143 */
  res->token = c[pick];
  res->n_kept = n;
  for (int i = 0; i < nc; ++i) {
    if (cand_id) cand_id[i] = c[i];
    if (cand_pr) cand_pr[i] = pr[i];
  }
  free(adj);
  free(order);
  free(c);
  free(v);
  free(pr);
}

/* ---------------------------------------------------------------- acceptance */
void orc_verify_greedy(const int32_t* sel, const int32_t* row_off, const int32_t* draft,
                       const int32_t* draft_off, int slots, int32_t* accepted, int32_t* next) {
  for (int s = 0; s < slots; ++s) {
    const int r0 = row_off[s], nd = draft_off[s + 1] - draft_off[s];
    const int32_t* d = draft + draft_off[s];
    int acc = 0, nx = sel[r0]; /* zero/runz.cpp:699 */
    while (acc < nd && nx == d[acc]) {
      ++acc;
      nx = sel[r0 + acc];
    }
    accepted[s] = acc;
    next[s] = nx;
  }
}

/* ---------------------------------------------------------------- confidence */
double orc_softmax_den(const float* l, int64_t n, float mx) {
  double z = 0;
  for (int64_t i0 = 0; i0 < n; i0 += 4096) {
    const int64_t i1 = n < i0 + 4096 ? n : i0 + 4096;
    float zs = 0.0f;
    for (int64_t i = i0; i < i1; ++i) zs += expf(l[i] - mx);
    z += zs;
  }
  return z;
}
double orc_softmax_den_exact(const float* l, int64_t n, float mx) {
  double z = 0;
  for (int64_t i = 0; i < n; ++i) z += exp((double)l[i] - (double)mx);
  return z;
}

/* ---------------------------------------------------------------- log probabilities */
double orc_logprobs(const float* l, int V, int32_t token, int top_n, double* logprob,
                    int32_t* top_id, double* top_logprob) {
  float mx = l[0];                                   /* tools/server_chat.h:419 */
  for (int i = 1; i < V; ++i)
    if (l[i] > mx) mx = l[i];
  double z = 0;
  for (int i = 0; i < V; ++i) z += exp((double)l[i] - mx);   /* :420-421 */
  const double lse = mx + log(z);                             /* :422 */
  if (token >= 0 && token < V && logprob) *logprob = (double)l[token] - lse;  /* :427 */
  if (top_n > V) top_n = V;
  /* :433-438: the top_n largest, best first: one scan that keeps a sorted list (top_n <= 256);
   * a precedes b when l[a] > l[b], or they are equal and a < b */
  int m = 0;
  for (int i = 0; i < V && top_n > 0; ++i) {
    const float v = l[i];
    if (v != v) continue;
    if (m == top_n && !(v > l[top_id[m - 1]])) continue; /* (equal to the last: the later id loses) */
    int pos = m < top_n ? m : top_n - 1;
    while (pos > 0 && v > l[top_id[pos - 1]]) {
      top_id[pos] = top_id[pos - 1];
      --pos;
    }
    top_id[pos] = i;
    if (m < top_n) ++m;
  }
  for (int r = 0; r < top_n; ++r) {
    if (r < m) top_logprob[r] = (double)l[top_id[r]] - lse;
    else {
      top_id[r] = -1;
      top_logprob[r] = NAN;
    }
  }
  return lse;
}

/* ---------------------------------------------------------------- byte automaton */
void orc_dfa_mask(const uint16_t* table, int S, int dead, int state, const uint32_t* byte_off,
                  const uint8_t* bytes, const uint8_t* special, int special_ok, int V,
                  uint32_t* out_bits) {
  (void)S;
  const int W = (V + 31) / 32;
  memset(out_bits, 0, (size_t)W * sizeof(uint32_t));
  for (int t = 0; t < V; ++t) {
    const uint32_t b0 = byte_off[t], b1 = byte_off[t + 1];
    if (b1 == b0) continue;                                   /* empty piece: never */
    if (special && special[t] && !special_ok) continue;       /* control token */
    int s = state;
    for (uint32_t i = b0; i < b1 && s != dead; ++i) s = table[(size_t)s * 256 + bytes[i]];
    if (s != dead) out_bits[t >> 5] |= 1u << (t & 31);
  }
}

/* ---------------------------------------------------------------- DFlash2 candidate selector */
/* zero/engine_drafters.h:461-506: per draft position the K largest raw logits; every candidate's
 * score is its logit plus the inner product of (pred[prev] * h) with succ[candidate] over the
 * rank of the bf16 codebooks, each product a float, summed in index order into a double
 * (:489-493); the best score (the first among equals, :494) is the draft; the drafts are kept
 * while the drafter's own probability of the path stays at or above min_p (:497-503: the first
 * draft always goes). Returns the number of drafts. path_p (optional, [positions]): the path
 * probability after each position visited. */
static float bf16_bits_to_float(uint16_t b) {
  const uint32_t w = (uint32_t)b << 16;
  float f;
  memcpy(&f, &w, 4);
  return f;
}
int orc_dflash_select(const float* logits, const float* hproj, const uint16_t* pred, const uint16_t* succ,
                      int V, int rank, int topk, int nd, int max_drafts, int tok, double min_p,
                      int32_t* out_tokens, double* path_p_out) {
  const int K = topk < V ? topk : V; /* :465 */
  int32_t* idx = (int32_t*)malloc((size_t)(K > 0 ? K : 1) * sizeof(int32_t));
  float* ph = (float*)malloc((size_t)rank * sizeof(float));
  int prev = tok, n_out = 0;
  double path_p = 1.0;
  const int steps = nd < max_drafts ? nd : max_drafts;
  for (int t = 0; t < steps; ++t) { /* :473 */
    const float* l = logits + (size_t)t * V;
    top_ids(l, V, K, idx); /* :476-484 */
    const float* h = hproj + (size_t)t * rank;
    for (int r = 0; r < rank; ++r) ph[r] = bf16_bits_to_float(pred[(size_t)prev * rank + r]) * h[r]; /* :487 */
    double best = -1e300;
    int bt = idx[0];
    for (int k = 0; k < K; ++k) { /* :490-495 */
      const int c = idx[k];
      double sc = l[c];
      const uint16_t* sv = succ + (size_t)c * rank;
      for (int r = 0; r < rank; ++r) {
        const float prod = ph[r] * bf16_bits_to_float(sv[r]);
        sc += prod;
      }
      if (sc > best) {
        best = sc;
        bt = c;
      }
    }
    if (min_p > 0) { /* :496-503 */
      float mx = l[idx[0]];
      for (int k = 1; k < K; ++k) mx = mx > l[idx[k]] ? mx : l[idx[k]];
      const double z = orc_softmax_den(l, V, mx);
      path_p *= exp((double)l[bt] - mx) / z;
      if (path_p_out) path_p_out[t] = path_p;
      if (t > 0 && path_p < min_p) break;
    }
    out_tokens[n_out++] = bt;
    prev = bt;
  }
  free(idx);
  free(ph);
  return n_out;
}

/* ---------------------------------------------------------------- bf16 */
void orc_bf16_to_f32(const uint16_t* in, int64_t n, float* out) {
  for (int64_t i = 0; i < n; ++i) {
    const uint32_t b = (uint32_t)in[i] << 16;
    memcpy(&out[i], &b, 4);
  }
}
void orc_f32_to_bf16(const float* in, int64_t n, uint16_t* out) {
  for (int64_t i = 0; i < n; ++i) {
    uint32_t b;
    memcpy(&b, &in[i], 4);
    if ((b & 0x7FFFFFFFu) > 0x7F800000u) { /* NaN stays NaN */
      out[i] = (uint16_t)((b >> 16) | 0x40);
      continue;
    }
    b += 0x7FFFu + ((b >> 16) & 1u); /* round to nearest, ties to even */
    out[i] = (uint16_t)(b >> 16);
  }
}
