/*
 * CPU oracle for the token-selection path. TEST INFRASTRUCTURE ONLY: nothing in the
 * shipped library links, loads or calls this file; it exists so that the CUDA path can
 * be checked against an independent restatement of the reference's arithmetic.
 *
 * Every function restates, in plain C, what the reference computes (citations are to
 * files of the reference project, by their path inside it):
 *   tools/sampler.h              Sampler::adjusted / sample / sample_allowed
 *   zero/runz.cpp                greedy argmax + accepted-prefix loop
 *   zero/engine_drafters.h       softmax_den (draft confidence)
 *   tools/server_chat.h          allowed(t) predicate around a constraint checker
 *
 * Parity status: PINNED for everything the reference itself pins. The restatement is
 * checked (tests/test_oracle_pin.py) against the reference's own Sampler compiled from
 * its sources into oracle/_ref/ and against fixtures generated from it
 * (tests/golden/).  Where the reference leaves the result to the C++ standard library
 * (order among exactly equal logits inside std::partial_sort / heap code) parity is
 * UNPINNED by the reference; this oracle uses the total order (value descending, id
 * ascending) and reports rows that contain such ties so a harness can count them.
 */
#ifndef ARCS_ORACLE_H
#define ARCS_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* Same field meaning and defaults as SamplingParams (tools/sampler.h:15-26), minus the
 * seed (the uniform draw is an explicit input) and the logit_bias list (passed beside). */
typedef struct {
  float temperature, top_p, min_p, presence_penalty, frequency_penalty, repeat_penalty;
  int32_t repeat_last_n, top_k;
} orc_params;

#define ORC_BANNED (-1e30f) /* Sampler::kBanned, tools/sampler.h:32 */

enum {
  ORC_FLAG_TIE_TOPK = 1,      /* two equal values among the kept candidates or at the cut */
  ORC_FLAG_FIRST_REFUSED = 2, /* sample_allowed: most likely non-banned token not allowed */
  ORC_FLAG_TAIL_SKIPPED = 4,  /* sample_allowed: e^-20 stop at rank 512 applied */
  ORC_FLAG_TAIL_USED = 8,     /* sample_allowed: candidates beyond rank 512 examined */
  ORC_FLAG_TIE_HEAD = 16      /* sample_allowed: equal logits at the top or across rank 512 (oracle only) */
};

typedef struct {
  int32_t token;  /* chosen id, -1 if none */
  int32_t n_cand; /* candidates after top-k and banned trimming */
  int32_t n_kept; /* candidates kept after min-p / top-p */
  int32_t flags;
} orc_result;

/* std::mt19937_64 (published algorithm) and the uniform draw the reference makes with
 * std::uniform_real_distribution<double>(0, tot) under libstdc++: u = x * 2^-64 rounded
 * to double, clamped below 1; the draw is then u * tot (tools/sampler.h:71-72). */
void orc_mt64_u01(uint64_t seed, int n, double* out);

/* Sampler::adjusted (tools/sampler.h:147-176). Returns 1 if anything was applied. */
int orc_adjusted(const float* logits, int V, const orc_params* p, const int32_t* hist, int H,
                 const int32_t* bias_id, const float* bias_val, int nb, float* out);

/* Sampler::sample (tools/sampler.h:36-78) with an explicit u in [0,1).
 * cand_id / cand_pr (size >= the row's k; may be NULL) receive the candidates in order and their
 * normalised probabilities pr[i]/z as doubles. */
void orc_sample(const float* logits, int V, const orc_params* p, const int32_t* hist, int H,
                const int32_t* bias_id, const float* bias_val, int nb, double u,
                orc_result* res, int32_t* cand_id, double* cand_pr);

/* Sampler::sample_allowed (tools/sampler.h:82-144); the predicate is a packed bitmask
 * (bit t of word t/32 set = token allowed). */
void orc_sample_allowed(const float* logits, int V, const orc_params* p, const int32_t* hist, int H,
                        const int32_t* bias_id, const float* bias_val, int nb,
                        const uint32_t* allowed, double u, orc_result* res, int32_t* cand_id,
                        double* cand_pr);

/* first maximum (tools/sampler.h:38, zero/runz.cpp:283) */
int32_t orc_argmax(const float* row, int V);

/* accepted-prefix length per slot (zero/runz.cpp:699-708, :361-374): rows of slot s are
 * sel[row_off[s] .. row_off[s+1]); drafts of slot s are draft[draft_off[s] .. draft_off[s+1]);
 * acc = number of leading i with sel[r0+i] == draft[i]; next = sel[r0+acc]. */
void orc_verify_greedy(const int32_t* sel, const int32_t* row_off, const int32_t* draft,
                       const int32_t* draft_off, int slots, int32_t* accepted, int32_t* next);

/* softmax_den (zero/engine_drafters.h:380-389): float exp, blocks of 4096 summed in float,
 * blocks summed in double. orc_softmax_den_exact is the same sum in double throughout. */
double orc_softmax_den(const float* l, int64_t n, float mx);
double orc_softmax_den_exact(const float* l, int64_t n, float mx);

/* a token's log probability and the top_n most likely alternatives from the raw logits
 * (tools/server_chat.h:417-441; the same log-softmax scores perplexity, zero/runz.cpp:478-484):
 * mx = max; z = sum exp((double)l - mx) in index order; lse = mx + log(z);
 * logprob(t) = (double)l[t] - lse. The alternatives are the top_n largest logits; the reference
 * leaves the order of equal logits to std::partial_sort, here the lower id comes first.
 * token < 0: no per-token entry (*logprob untouched). Returns lse. */
double orc_logprobs(const float* l, int V, int32_t token, int top_n, double* logprob,
                    int32_t* top_id, double* top_logprob);

/* allowed(t) over a vocabulary for a byte automaton (tools/server_chat.h:539-557 with the
 * checker replaced by a transition table): token t is allowed iff its byte string is not
 * empty, it is not special (or special_ok), and walking its bytes from `state` never
 * reaches `dead`. table is [S][256] next-state ids. */
void orc_dfa_mask(const uint16_t* table, int S, int dead, int state, const uint32_t* byte_off,
                  const uint8_t* bytes, const uint8_t* special, int special_ok, int V,
                  uint32_t* out_bits);

/* The DFlash2 candidate selector (zero/engine_drafters.h:461-506) for one slot: logits [nd][V],
 * hproj [nd][rank] fp32; pred / succ [V][rank] bf16 bit patterns. Returns the number of drafts
 * written to out_tokens; path_p_out (optional, [nd]) receives the path probability after each
 * position visited (only with min_p > 0). */
int orc_dflash_select(const float* logits, const float* hproj, const uint16_t* pred, const uint16_t* succ,
                      int V, int rank, int topk, int nd, int max_drafts, int tok, double min_p,
                      int32_t* out_tokens, double* path_p_out);

/* exact widening / round-to-nearest-even narrowing between fp32 and bf16 */
void orc_bf16_to_f32(const uint16_t* in, int64_t n, float* out);
void orc_f32_to_bf16(const float* in, int64_t n, uint16_t* out);

#ifdef __cplusplus
}
#endif
#endif
