/*
 * libarcsample — per-step token selection on NVIDIA B200 (sm_100a), C ABI.
 *
 * This is the boundary a host application binds instead of running the reference's
 * single-threaded host sampler over a logits row read back from the GPU. Every entry point
 * takes plain pointers and sizes; device pointers are owned by the caller; nothing throws;
 * the return value is an arcs_status. Calls enqueue work on the caller's stream (passed as
 * void*, a cudaStream_t) and do not synchronise unless the name ends in _host. The arcs_jcon_* and
 * arcs_tcon_create functions are host code and enqueue nothing.
 *
 * Citations name files of the reference project (rizagp/arcinfer) by their path inside it.
 *
 * Ordering rule everywhere: candidates are ranked by (logit descending, token id ascending).
 * The reference leaves the order among exactly equal logits to the C++ standard library's
 * heap code; with distinct logits both orders are the same.
 */
#ifndef ARCSAMPLE_H
#define ARCSAMPLE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define ARCS_VERSION 1
#define ARCS_KCAP 256          /* most candidates a row can keep (top_k <= 0 means 256) */
#define ARCS_HEAD 512          /* sample_allowed: ranks examined before the tail rule */
#define ARCS_BANNED (-1e30f)   /* Sampler::kBanned, tools/sampler.h:32 */

typedef enum {
  ARCS_OK = 0,
  ARCS_ERR_ARG = 1,        /* null pointer, negative size, unknown dtype, V == 0 ... */
  ARCS_ERR_TOPK = 2,       /* a row asks for more than ARCS_KCAP candidates */
  ARCS_ERR_WORKSPACE = 3,  /* workspace missing or smaller than arcs_*_workspace_bytes says */
  ARCS_ERR_CUDA = 4,       /* a CUDA call failed; arcs_last_error() has the text */
  ARCS_ERR_LIST = 5,       /* a row's history / bias list is longer than max_hist / max_bias */
  ARCS_ERR_TIMEOUT = 6,    /* device side: a bounded wait ran out (status word only) */
  ARCS_ERR_INJECTED = 7,   /* host-side fault injection (ARCS_FAIL_CALL=N environment variable) */
  ARCS_ERR_UNSUPPORTED = 8 /* jcon: the schema (or this step's table) is outside what the automaton expresses */
} arcs_status;

typedef enum { ARCS_F32 = 0, ARCS_BF16 = 1 } arcs_dtype;

/* One row's sampling parameters: SamplingParams (tools/sampler.h:15-26) field for field,
 * without the seed (the uniform draw u is an explicit input) and without the logit_bias
 * list (a CSR list beside it). Defaults there: temperature 1, top_p .95, min_p 0,
 * presence 0, frequency 0, repeat_penalty 1, repeat_last_n 64, top_k 20. */
typedef struct {
  float temperature, top_p, min_p, presence_penalty, frequency_penalty, repeat_penalty;
  int32_t repeat_last_n, top_k;
} arcs_row_params;

/* per-row result flags */
enum {
  ARCS_FLAG_TIE_TOPK = 1,      /* two equal logits among the candidates kept */
  ARCS_FLAG_FIRST_REFUSED = 2, /* constrained: the most likely token was not allowed (tools/server_chat.h:542) */
  ARCS_FLAG_TAIL_SKIPPED = 4,  /* constrained: e^-20 stop at rank 512 applied (tools/sampler.h:111) */
  ARCS_FLAG_TAIL_USED = 8      /* constrained: candidates beyond rank 512 were needed */
};

const char* arcs_last_error(void); /* text of the calling thread's last failure */
int arcs_version(void);

/* ------------------------------------------------------------------------------------------
 * sample_batch: Sampler::adjusted + Sampler::sample for B rows in one call (two launches on the
 * stream: the single pass over the logits, and a small per-row finish that runs beside it)
 * (tools/sampler.h:36-78, :147-176); with a mask, Sampler::sample_allowed (:82-144) where
 * the predicate ok(t) is bit t of the row's mask.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  /* inputs (device pointers) */
  const void* logits;        /* [B][row_stride] of dtype; row b starts at b*row_stride elements */
  int32_t dtype;             /* arcs_dtype */
  int32_t B, V;              /* B <= 65536; token ids (id_base + V, v_global) below 2^29 - 1 */
  int64_t row_stride;        /* in elements, >= V */
  const arcs_row_params* params; /* [B] */
  const int32_t* hist_off;   /* [B+1] CSR offsets into hist_ids, or NULL: no history (`recent`) */
  const int32_t* hist_ids;   /* token ids generated so far, oldest first; ids outside [0,V) ignored */
  const int32_t* bias_off;   /* [B+1] CSR offsets of the logit_bias lists, or NULL */
  const int32_t* bias_ids;
  const float* bias_vals;    /* <= -100 bans the token (tools/sampler.h:24) */
  const double* u;           /* [B] uniform draws in [0,1); the reference's draw is u*tot */
  const uint32_t* mask;      /* NULL: unconstrained. Else packed allowed-token bits, rows of mask_stride words */
  const int32_t* mask_row;   /* [B] mask row used by each batch row, or NULL: row b uses mask row b */
  int64_t mask_stride;       /* words per mask row, >= ceil(V/32) */
  int32_t max_hist, max_bias;/* upper bounds on any row's list length (they size the on-chip filter and table). A row
                                whose penalties can only lower logits (repeat_penalty >= 1, presence and frequency
                                >= 0) and whose bias list has at most 64 entries takes a history of any length up to
                                max_hist; any other row's lists may hold 1024 entries together, else ARCS_ERR_LIST */
  int32_t id_base;           /* global id of column 0 (vocabulary shards); 0 otherwise */
  int32_t v_global;          /* whole vocabulary size when sharded; 0 means V */
  /* outputs (device pointers; optional ones may be NULL) */
  int32_t* token;            /* [B] chosen id, -1 when no token is allowed */
  int32_t* n_cand;           /* [B] optional: candidates after top-k / banned trimming */
  int32_t* n_kept;           /* [B] optional: candidates left after min-p / top-p */
  int32_t* flags;            /* [B] optional: ARCS_FLAG_* */
  int32_t* cand_id;          /* [B][cand_stride] optional: candidate ids in order */
  float* cand_val;           /* [B][cand_stride] optional: their adjusted logits */
  float* cand_pr;            /* [B][cand_stride] optional: their probabilities pr[i]/z */
  int32_t cand_stride;       /* >= ARCS_KCAP when any cand_* is given */
  /* scratch */
  void* workspace;           /* arcs_sample_workspace_bytes() bytes, 16-byte aligned; needs no initialisation */
  size_t workspace_bytes;
  int32_t* status;           /* optional device word: 0 or an arcs_status set by the kernels */
  /* The ranked head of a constrained row (only with a mask; all three or none): the ARCS_HEAD most
   * likely tokens by adjusted logit, banned ones included, in (logit descending, id ascending)
   * order - the order in which Sampler::sample_allowed calls its predicate (tools/sampler.h:93-120).
   * A host whose predicate cannot be written as a mask calls with an all-zero mask, reads the head,
   * and calls the predicate itself in that order. */
  int32_t* head_id;          /* [B][ARCS_HEAD] optional; entries past n_head are -1 */
  float* head_val;           /* [B][ARCS_HEAD] their adjusted logits */
  int32_t* n_head;           /* [B] min(V, ARCS_HEAD) less the NaN logits among them */
  /* Entries written per row of cand_id / cand_val / cand_pr: 0 means cand_stride (which must then be
   * >= ARCS_KCAP). A smaller width lets the lists be written straight into packed per-row records
   * (ids, values and whatever else the record carries, cand_stride apart): what a vocabulary shard
   * sends to the others. A row that keeps more candidates than cand_width raises ARCS_ERR_TOPK in
   * the status word and writes the first cand_width. */
  int32_t cand_width;
} arcs_sample_args;

/* max_list: max_hist + max_bias of the call (0 without lists) */
size_t arcs_sample_workspace_bytes(int32_t B, int32_t V, int32_t masked, int32_t max_list);
int arcs_sample_batch(const arcs_sample_args* args, void* stream);
/* Measurement aid: the same two launches, one after the other (the finish kernel does not run
 * beside the stream kernel here), with CUDA events between them on `stream`; waits for them and
 * returns the device time of the stream and finish kernels in ms2[0..1]. */
int arcs_sample_batch_timed(const arcs_sample_args* args, void* stream, float* ms2);

/* adjusted_batch: Sampler::adjusted (tools/sampler.h:147-176) for whole rows: the logits after
 * logit_bias, the frequency / repeat / presence penalties and the bans, as fp32 (bit for bit the
 * reference's values: every operation a separate fp32 rounding in its order). Device pointers. */
typedef struct {
  const void* logits;        /* [B][row_stride] of dtype */
  int32_t dtype, B, V;
  int64_t row_stride;
  const arcs_row_params* params;
  const int32_t* hist_off;   /* as in arcs_sample_args; lists of any length */
  const int32_t* hist_ids;
  const int32_t* bias_off;
  const int32_t* bias_ids;
  const float* bias_vals;
  float* out;                /* [B][out_stride] */
  int64_t out_stride;        /* >= V */
} arcs_adjusted_args;
int arcs_adjusted_batch(const arcs_adjusted_args* args, void* stream);

/* Vocabulary shards (no counterpart in the reference, which has one device): every GPU runs
 * arcs_sample_batch on its columns of all rows (`id_base`, `v_global`; lists are filtered by range)
 * with candidate outputs, the lists are all-gathered (NCCL, by the caller), and this call takes the
 * global k best of the G lists under the same order and finishes as the single-GPU path does. */
typedef struct arcs_merge_args {
  int32_t G, B, cand_stride;   /* shards, rows, stride of the gathered lists */
  const int32_t* cand_id;      /* [G][B][cand_stride] global ids, best first (device) */
  const float* cand_val;       /* [G][B][cand_stride] their adjusted logits */
  const int32_t* n_cand;       /* [G][B] entries per list (may be NULL with packed records, below) */
  const arcs_row_params* params;
  const double* u;
  const int32_t* bias_off;     /* optional: only "does the row ban anything" is read from the bias list */
  const float* bias_vals;
  int32_t v_global;            /* whole vocabulary size */
  int32_t* token;              /* outputs as in arcs_sample_args */
  int32_t* n_cand_out;
  int32_t* n_kept;
  int32_t* flags;
  int32_t* out_id;
  float* out_val;
  float* out_pr;
  int32_t out_stride;
  int32_t* status;
  /* Packed records. cand_width: entries per gathered list (0: cand_stride); n_cand may then be NULL:
   * a list ends at its first negative id. shard_mz: [G][B] pairs (max, sum of exp(l - max)) of every
   * shard's raw logits, mz_stride floats apart (optional, e.g. from arcs_argmax_batch's max_sumexp),
   * combined into mz_out [B][2]: M = max m_g, Z = sum z_g exp(m_g - M), so that
   * log-probabilities over the whole vocabulary are M + log Z away from a raw logit. With
   * cand_id = rec, cand_val = rec + k, shard_mz = rec + 2k, cand_stride = mz_stride = 2k + 2 the
   * call reads a gathered buffer of [G][B] records of k * 8 + 8 bytes in place. */
  int32_t cand_width;
  const float* shard_mz;
  int32_t mz_stride;
  float* mz_out;
} arcs_merge_args;
int arcs_merge_batch(const arcs_merge_args* args, void* stream);

/* ------------------------------------------------------------------------------------------
 * argmax_batch: first maximum of each row (tools/sampler.h:38; zero/runz.cpp:283;
 * zero/engine_drafters.h:80-81, :632-633), optionally with (max, sum exp(l - max)) per row
 * (softmax_den, zero/engine_drafters.h:380-389) and, for rows grouped by slot, the greedy
 * draft acceptance of zero/runz.cpp:699-708 / :361-374: accepted[s] = number of leading
 * drafts equal to the row argmax, next[s] = argmax of row accepted[s] of the slot.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  const void* logits;
  int32_t dtype;
  int32_t R, V;
  int64_t row_stride;
  int32_t* argmax;           /* [R] */
  float* max_sumexp;         /* [R][2] optional */
  int32_t slots;             /* 0: no verification */
  const int32_t* row_off;    /* [slots+1] first row of each slot (rows of a slot are contiguous) */
  const int32_t* draft;      /* draft tokens of all slots */
  const int32_t* draft_off;  /* [slots+1] */
  int32_t* accepted;         /* [slots] */
  int32_t* next;             /* [slots] */
  void* workspace;           /* arcs_argmax_workspace_bytes(), zeroed before its first use and again before a call of another shape (R, V) takes it over */
  size_t workspace_bytes;
  int32_t* status;
} arcs_argmax_args;

size_t arcs_argmax_workspace_bytes(int32_t R, int32_t V);
int arcs_argmax_batch(const arcs_argmax_args* args, void* stream);

/* Variant of arcs_argmax_batch for callers that cannot allocate device memory (no counterpart in
 * the reference, whose sampler runs on the host). A host that has given all of HBM to its own
 * pool, or that must not call the allocator between the kernels of a step because the call may
 * synchronise the device, cannot supply the workspace the plain entry point wants. Here the
 * scratch is a fixed array inside the library: arcs_argmax_static_scratch_bytes() bytes (1 MiB)
 * on every GPU that loads the library, held until the process exits. `workspace` and
 * `workspace_bytes` of the argument block are ignored; inputs and outputs are still the
 * caller's. Shapes whose scratch (arcs_argmax_workspace_bytes) exceeds the array are refused with
 * ARCS_ERR_WORKSPACE. The first call on a device looks the array's device address up and clears
 * it on the given stream: make that call before capturing a stream. All calls on a device share
 * the array: two calls that overlap on the GPU (different streams) race; calls on one stream are
 * safe, each leaves the array clean for the next (also a call whose bounded device wait ran out
 * and set ARCS_ERR_TIMEOUT in the status word). The set-up is guarded by a lock, so first calls
 * from several host threads enqueue the clearing once. The stream must belong to the current
 * device. No allocation is made by this call. */
/* accept_batch: the acceptance walk over tokens chosen by any means: with sampled tokens it is
 * the verification of drafts under sampling (tools/server_chat.h:578-591: the server samples from
 * the row after each accepted draft, with the accepted drafts appended to the history, and stops
 * at the first sample that differs). Because an accepted token EQUALS its draft, the history of
 * verification row i, if the walk reaches it, is known beforehand: the slot's history followed by
 * the first i drafts. So all rows of all slots are sampled in ONE arcs_sample_batch call (row i
 * of a slot with that history and its own uniform number), and this call walks the result:
 * accepted[s] = leading drafts equal to their row's token, next[s] = the token of the first row
 * that differs (or of the row after the last draft). Rows past that point were sampled in vain;
 * a host that draws its uniforms from a generator advances it by accepted[s] + 1 draws only. */
int arcs_accept_batch(const int32_t* token, const int32_t* row_off, const int32_t* draft, const int32_t* draft_off,
                      int32_t slots, int32_t* accepted, int32_t* next, void* stream);

size_t arcs_argmax_static_scratch_bytes(void);
int arcs_argmax_batch_static(const arcs_argmax_args* args, void* stream);

/* ------------------------------------------------------------------------------------------
 * dfa_mask: allowed(t) for every token of a vocabulary under a byte automaton, packed.
 * Replaces the per-candidate predicate calls of tools/server_chat.h:539-557
 * (piece(t) not empty, not special unless special_ok, check(text + piece) != FAIL) by one
 * pass over the vocabulary per distinct automaton state: token t is allowed iff its byte
 * string is not empty and walking it from the state never reaches `dead`.
 * table: [n_table_states][256] uint16 next state; states: [n_states] start states;
 * out: [n_states][out_stride] words. vocabulary: byte_off[V+1] offsets into bytes.
 * ---------------------------------------------------------------------------------------- */
int arcs_dfa_mask(const uint16_t* table, int32_t n_table_states, int32_t dead, const int32_t* states,
                  int32_t n_states, const uint32_t* byte_off, const uint8_t* bytes, const uint8_t* special,
                  int32_t special_ok, int32_t V, uint32_t* out, int64_t out_stride, void* stream);

/* ------------------------------------------------------------------------------------------
 * jcon: the constrained-JSON prefix checker (jcon::Checker, tools/json_constraint.h:30-281) as an
 * incremental byte automaton, and the bridge from it to arcs_dfa_mask. HOST code, no GPU work.
 * The reference asks check(answer + piece(t)) != FAIL per candidate token, each call parsing the
 * whole answer again (tools/server_chat.h:553-557); here the answer is walked once per step and
 * the transitions that the vocabulary's tokens can take from there are written out as a table.
 *   arcs_jcon_create: schema_json is the schema's JSON text ("{}" = any value), object_only the
 *     json_object mode (tools/server_chat.h:30-31); the vocabulary (byte_off[V+1], bytes; host
 *     memory, copied) is the one later given to arcs_dfa_mask. Returns ARCS_ERR_UNSUPPORTED, with
 *     the handle still created so that arcs_jcon_why() names the construct, for the two schema
 *     forms without a finite automaton: anyOf / oneOf whose branches can begin with the same
 *     character, and an enum with one option's text a proper prefix of another's. The caller
 *     then keeps the reference's per-candidate predicate (arcs_sample_batch's ranked head).
 *   arcs_jcon_check: jcon::Checker::check(text): 0 FAIL, 1 PARTIAL, 2 DONE (-1: bad handle).
 *   arcs_jcon_table: the table for the step after `text`: state 0 is the configuration after
 *     text; token t is allowed iff walking its bytes from state 0 never reaches *dead, i.e. iff
 *     check(text + piece(t)) != FAIL. done[s] != 0: the answer is complete in state s
 *     (tools/server_chat.h:550: the server then ends the answer). text_state receives
 *     check(text). Only transitions some token takes are filled in; the rest lead to *dead. The
 *     pointers are host memory owned by the handle and stay valid until the next call on it;
 *     tables are cached by configuration. ARCS_ERR_ARG when text itself already fails;
 *     ARCS_ERR_UNSUPPORTED when the step needs more than 8192 states.
 *   One corner differs from the reference inside a single token: a token that closes TWO keys
 *   the schema does not name, in one object that allows other keys, is refused even if the two
 *   keys differ (the table does not remember such keys' text).
 * ---------------------------------------------------------------------------------------- */
typedef struct arcs_jcon arcs_jcon;
int arcs_jcon_create(const char* schema_json, int32_t object_only, const uint32_t* byte_off, const uint8_t* bytes,
                     int32_t V, arcs_jcon** out);
const char* arcs_jcon_why(const arcs_jcon* h);
int arcs_jcon_check(const arcs_jcon* h, const char* text, int64_t len);
int arcs_jcon_table(arcs_jcon* h, const char* text, int64_t len, const uint16_t** table, int32_t* n_states,
                    int32_t* dead, const uint8_t** done, int32_t* text_state);
void arcs_jcon_cache_stats(const arcs_jcon* h, int64_t* hits, int64_t* misses);
/* The same machinery for a tool call (tools/tool_constraint.h): the handle's text is what follows
 * the call's open marker; check / table / why / destroy are the arcs_jcon_* functions above.
 * ARCS_TCON_GEMMA: tcon::GemmaCall (:66-280), call:NAME{key:value,...}<tool_call|> with bare keys,
 * strings between <|"|> delimiters, no whitespace, no exponents; tools_json is the request's
 * "tools" array (:45-51). The same two schema forms are refused as for JSON. Control tokens: the
 * reference lets the pieces <|"|> and <tool_call|> through inside a call (special_ok, :75); give
 * arcs_dfa_mask a `special` array that leaves those two out.
 * ARCS_TCON_QWEN: tcon::QwenCall (:285-371), <function=NAME> then <parameter=KEY> VALUE
 * </parameter> blocks, </function> </tool_call>, up to two blanks between the parts; a "string"
 * (or untyped) value is raw text without the two parameter markers, any other is JSON for its
 * schema (its own root, as jcon::Checker(vs, false)), optionally followed by one newline. */
enum { ARCS_TCON_GEMMA = 0, ARCS_TCON_QWEN = 1 };
int arcs_tcon_create(int32_t kind, const char* tools_json, const uint32_t* byte_off, const uint8_t* bytes, int32_t V,
                     arcs_jcon** out);
void arcs_jcon_destroy(arcs_jcon* h);

/* ------------------------------------------------------------------------------------------
 * logprobs_batch: per row, the log probability of one token and the top_n most likely
 * alternatives, from the RAW logits (no penalty, no bias): the `logprobs` entry of
 * tools/server_chat.h:417-441, and the log-softmax that scores perplexity and KL
 * (zero/runz.cpp:478-484, :639-646). One pass over the logits, one launch. When there are few
 * rows each is cut into segments, whose results meet in the workspace.
 *   mx = max; z = sum exp(l - mx) accumulated in fp64; lse = mx + log(z);
 *   logprob[b] = l[token[b]] - lse;  top_id / top_logprob: the top_n largest logits, best first
 *   (equal logits: lower id first), as log probabilities.
 * The reference sums fp64 exponentials in index order; here each term is a single-precision
 * exponential (ex2.approx of the rounded product (l - m) * log2 e), summed pairwise in fp32 per
 * 16-byte chunk and then in fp64, in another order: lse agrees with an fp64 log-sum-exp to about
 * 4e-8 absolute on the tested distributions (the tests hold it to 1e-6). NaN logits are skipped.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  const void* logits;     /* [B][row_stride] device */
  int32_t dtype;          /* arcs_dtype */
  int32_t B, V;
  int64_t row_stride;     /* elements */
  const int32_t* token;   /* [B] token whose log probability is wanted; NULL or an id < 0: none */
  int32_t top_n;          /* alternatives per row, 0 .. ARCS_KCAP (the reference serves 0 .. 20) */
  int32_t top_stride;     /* >= top_n */
  double* logprob;        /* [B] (NaN where no token was given); may be NULL when token is */
  double* lse;            /* [B] optional: log of the sum of exponentials */
  int32_t* top_id;        /* [B][top_stride]; entries past min(top_n, V) are not written */
  double* top_logprob;    /* [B][top_stride] */
  void* workspace;        /* arcs_logprobs_workspace_bytes(), zeroed before its first use and again before a call of another shape (B, V, top_n) takes it over */
  size_t workspace_bytes;
  int32_t* status;        /* device status word (first error wins), may be NULL */
} arcs_logprob_args;

size_t arcs_logprobs_workspace_bytes(int32_t B, int32_t V, int32_t top_n);
int arcs_logprobs_batch(const arcs_logprob_args* args, void* stream);

/* ------------------------------------------------------------------------------------------
 * dflash_select: the candidate selector of the DFlash2 drafter (zero/engine_drafters.h:461-506),
 * for many slots in one call. Per slot and draft position t (rows of raw logits, as the
 * drafter's head produced them): the topk largest logits (value descending, id ascending,
 * :476-484); score(c) = logit(c) + sum_r (pred[prev][r] * hproj[t][r]) * succ[c][r], every
 * product a float and the sum a double built in index order (:487-493); the candidate with the
 * best score, the first among equals, becomes the draft and the next position's `prev` (:494,
 * :505). With min_p > 0 the drafts stop when the drafter's own probability of the path,
 * prod exp(logit(draft) - max) / sum exp(l - max), falls below min_p; the first draft always
 * goes (:496-503; the reference reads min_p from ARC_DFL_P, default 0.3).
 * Drafts are bit-exact against the reference's loop; the path probability uses this library's
 * log-sum-exp (logprobs_batch), within 1e-7 relative of the exact sum where the reference's
 * float sums over blocks of 4096 are within about 1e-6: a path probability that close to min_p
 * may be cut one draft apart.
 * The first step is arcs_logprobs_batch on slots * nd rows; the second one warp per slot.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  const void* logits;      /* [slots][nd][row_stride] device, of dtype */
  int32_t dtype;           /* arcs_dtype */
  int32_t slots, nd, V;
  int64_t row_stride;      /* elements */
  const float* hproj;      /* [slots][nd][rank] the selector's projection of the hidden states */
  const uint16_t* pred;    /* [V][rank] bf16 bit patterns: codebook indexed by the previous token */
  const uint16_t* succ;    /* [V][rank] bf16 bit patterns: codebook indexed by the candidate */
  int32_t rank;            /* 1 .. 1024 */
  int32_t topk;            /* 1 .. 64 (the reference's dfl_topk_, 16) */
  int32_t max_drafts;      /* at most min(nd, max_drafts) drafts per slot */
  const int32_t* tok;      /* [slots] the token before the first draft */
  double min_p;            /* 0: no cut */
  int32_t* n_out;          /* [slots] drafts kept */
  int32_t* out_tokens;     /* [slots][out_stride] */
  int32_t out_stride;      /* >= min(nd, max_drafts) */
  double* path_p;          /* [slots][nd] optional: path probability after each position visited */
  void* workspace;         /* arcs_dflash_workspace_bytes(), 256-byte aligned, zeroed before its first use and again before a call of another shape takes it over */
  size_t workspace_bytes;
  int32_t* status;         /* device status word, may be NULL */
} arcs_dflash_args;

size_t arcs_dflash_workspace_bytes(int32_t slots, int32_t nd, int32_t V, int32_t topk);
int arcs_dflash_select(const arcs_dflash_args* args, void* stream);

/* ------------------------------------------------------------------------------------------
 * Host-buffer entry points: what a host application that keeps its logits in host memory
 * (the reference reads every row back from the GPU, zero/engine.h:255-258, and hands
 * Sampler::sample a std::vector<float>, tools/server_chat.h:561) calls instead of
 * Sampler::sample / sample_allowed. All pointers in `host_args` are HOST pointers (pinned
 * memory makes the copies asynchronous); workspace / status are ignored. The context owns
 * the device buffers, two streams and the scratch; rows are copied and processed in chunks so
 * that the host-to-device copy of one chunk overlaps the kernel of the previous one. The call
 * returns after the results are in the host output arrays. A context is not thread-safe (the
 * reference's Sampler is not either, tools/sampler.h:204-206).
 * ---------------------------------------------------------------------------------------- */
typedef struct arcs_host_ctx arcs_host_ctx;
int arcs_host_create(arcs_host_ctx** out, int32_t device, int32_t max_B, int32_t max_V, int32_t dtype,
                     int64_t max_hist_total, int64_t max_bias_total, int64_t max_mask_words);
void arcs_host_destroy(arcs_host_ctx* ctx);
int arcs_sample_batch_host(arcs_host_ctx* ctx, const arcs_sample_args* host_args);
/* Sampler::adjusted with host buffers (tools/sampler.h:147-176); all pointers of host_args are host pointers */
int arcs_adjusted_batch_host(arcs_host_ctx* ctx, const arcs_adjusted_args* host_args);
/* The last step of Sampler::sample_allowed (tools/sampler.h:121-143) for a host that has called its
 * predicate itself, in the order of the ranked head: n <= ARCS_KCAP candidates in the order they
 * were found (ids, adjusted logits: host pointers), the row's settings, the uniform draw;
 * softmax, min-p / top-p cuts and the draw on the device. *token = -1 when n == 0. */
int arcs_draw_candidates_host(arcs_host_ctx* ctx, const int32_t* ids, const float* vals, int32_t n, const arcs_row_params* params,
                              double u, int32_t v_global, int32_t* token, int32_t* n_kept);
/* greedy selection + acceptance with host buffers (zero/runz.cpp:683-715) */
int arcs_argmax_batch_host(arcs_host_ctx* ctx, const arcs_argmax_args* host_args);
/* device status word of the last host call (0 = fine) */
int arcs_host_last_status(arcs_host_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif
