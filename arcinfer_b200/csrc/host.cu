// Host-buffer entry points: a context that owns device buffers and pipelines
// host->device copies of row chunks with the kernels that consume them.
#include <algorithm>
#include <new>

#include "plan.h"

using namespace arcs;

struct arcs_host_ctx {
  int device = 0;
  int32_t max_B = 0, max_V = 0, dtype = 0;
  int64_t max_hist = 0, max_bias = 0, max_mask = 0;
  cudaStream_t st[2] = {nullptr, nullptr};
  cudaEvent_t small_ready = nullptr;
  char* logits = nullptr;
  arcs_row_params* params = nullptr;
  int32_t *hist_off = nullptr, *hist_ids = nullptr, *bias_off = nullptr, *bias_ids = nullptr;
  float* bias_vals = nullptr;
  double* u = nullptr;
  uint32_t* mask = nullptr;
  int32_t* mask_row = nullptr;
  int32_t *token = nullptr, *n_cand = nullptr, *n_kept = nullptr, *flags = nullptr, *cand_id = nullptr;
  float *cand_val = nullptr, *cand_pr = nullptr;
  int32_t *argmax = nullptr, *row_off = nullptr, *draft = nullptr, *draft_off = nullptr, *accepted = nullptr, *next = nullptr;
  float* max_sumexp = nullptr;
  void* ws[2] = {nullptr, nullptr};  // sample_batch scratch, one per stream, grown on demand
  size_t ws_sample_bytes = 0;
  void* ws_argmax = nullptr;
  size_t ws_bytes = 0;               // argmax scratch
  int32_t* status = nullptr;
  int32_t last_status = 0;
  // grown on first use
  int32_t *head_id = nullptr, *n_head = nullptr;  // [max_B][ARCS_HEAD], [max_B]
  float* head_val = nullptr;
  float* adj_out = nullptr;                       // [max_B][max_V]
  int32_t* draw_id = nullptr;                     // [ARCS_KCAP] candidates handed in by the host
  float* draw_val = nullptr;
  int32_t* draw_n = nullptr;
};

#define CU(x)                                                                  \
  do {                                                                         \
    cudaError_t e_ = (x);                                                      \
    if (e_ != cudaSuccess) return set_error(ARCS_ERR_CUDA, cudaGetErrorString(e_)); \
  } while (0)

template <typename T>
static cudaError_t dalloc(T** p, size_t n) {
  return cudaMalloc(reinterpret_cast<void**>(p), std::max<size_t>(n, 1) * sizeof(T));
}

extern "C" void arcs_host_destroy(arcs_host_ctx* c) {
  if (!c) return;
  cudaSetDevice(c->device);
  for (void* p : {(void*)c->logits, (void*)c->params, (void*)c->hist_off, (void*)c->hist_ids, (void*)c->bias_off,
                  (void*)c->bias_ids, (void*)c->bias_vals, (void*)c->u, (void*)c->mask, (void*)c->mask_row,
                  (void*)c->token, (void*)c->n_cand, (void*)c->n_kept, (void*)c->flags, (void*)c->cand_id,
                  (void*)c->cand_val, (void*)c->cand_pr, (void*)c->argmax, (void*)c->row_off, (void*)c->draft,
                  (void*)c->draft_off, (void*)c->accepted, (void*)c->next, (void*)c->max_sumexp, c->ws[0], c->ws[1], c->ws_argmax,
                  (void*)c->status, (void*)c->head_id, (void*)c->n_head, (void*)c->head_val, (void*)c->adj_out, (void*)c->draw_id,
                  (void*)c->draw_val, (void*)c->draw_n})
    if (p) cudaFree(p);
  if (c->small_ready) cudaEventDestroy(c->small_ready);
  for (auto s : c->st)
    if (s) cudaStreamDestroy(s);
  delete c;
}

extern "C" int arcs_host_create(arcs_host_ctx** out, int32_t device, int32_t max_B, int32_t max_V, int32_t dtype,
                                int64_t max_hist_total, int64_t max_bias_total, int64_t max_mask_words) {
  if (!out || max_B <= 0 || max_V <= 0 || (dtype != ARCS_F32 && dtype != ARCS_BF16) || max_hist_total < 0 ||
      max_bias_total < 0 || max_mask_words < 0)
    return set_error(ARCS_ERR_ARG, "host_create: bad argument");
  CU(cudaSetDevice(device));
  arcs_host_ctx* c = new (std::nothrow) arcs_host_ctx;
  if (!c) return set_error(ARCS_ERR_ARG, "host_create: out of host memory");
  c->device = device;
  c->max_B = max_B;
  c->max_V = max_V;
  c->dtype = dtype;
  c->max_hist = max_hist_total;
  c->max_bias = max_bias_total;
  c->max_mask = max_mask_words;
  const size_t es = dtype == ARCS_F32 ? 4 : 2;
  const size_t B = (size_t)max_B;
  // Upper bound of the scratch any chunk of <= max_B rows can ask for: rows * segments never
  // exceeds 4 CTAs per SM plus one segment per row (plan_segments), each with a masked block.
  const size_t wsb = 4096 + ((size_t)1 << 18) + (size_t)max_B * 16 + ((size_t)kSmCount * 4 + (size_t)max_B) * (16 + ARCS_KCAP * 8 + ARCS_HEAD * 8 + 8);
  c->ws_bytes = wsb;
  cudaError_t e = cudaSuccess;
  auto ok = [&](cudaError_t r) { if (e == cudaSuccess) e = r; };
  ok(cudaStreamCreateWithFlags(&c->st[0], cudaStreamNonBlocking));
  ok(cudaStreamCreateWithFlags(&c->st[1], cudaStreamNonBlocking));
  ok(cudaEventCreateWithFlags(&c->small_ready, cudaEventDisableTiming));
  ok(dalloc(&c->logits, B * (size_t)max_V * es + 64));
  ok(dalloc(&c->params, B));
  ok(dalloc(&c->hist_off, B + 1));
  ok(dalloc(&c->hist_ids, (size_t)max_hist_total));
  ok(dalloc(&c->bias_off, B + 1));
  ok(dalloc(&c->bias_ids, (size_t)max_bias_total));
  ok(dalloc(&c->bias_vals, (size_t)max_bias_total));
  ok(dalloc(&c->u, B));
  ok(dalloc(&c->mask, (size_t)max_mask_words));
  ok(dalloc(&c->mask_row, B));
  ok(dalloc(&c->token, B));
  ok(dalloc(&c->n_cand, B));
  ok(dalloc(&c->n_kept, B));
  ok(dalloc(&c->flags, B));
  ok(dalloc(&c->cand_id, B * ARCS_KCAP));
  ok(dalloc(&c->cand_val, B * ARCS_KCAP));
  ok(dalloc(&c->cand_pr, B * ARCS_KCAP));
  ok(dalloc(&c->argmax, B));
  ok(dalloc(&c->row_off, B + 1));
  ok(dalloc(&c->draft, B));
  ok(dalloc(&c->draft_off, B + 1));
  ok(dalloc(&c->accepted, B));
  ok(dalloc(&c->next, B));
  ok(dalloc(&c->max_sumexp, B * 2));
  ok(cudaMalloc(&c->ws_argmax, wsb));
  if (e == cudaSuccess) ok(cudaMemset(c->ws_argmax, 0, wsb));
  ok(dalloc(&c->status, 1));
  if (e == cudaSuccess) ok(cudaMemset(c->status, 0, sizeof(int32_t)));
  if (e == cudaSuccess) ok(cudaDeviceSynchronize());
  if (e != cudaSuccess) {
    arcs_host_destroy(c);
    return set_error(ARCS_ERR_CUDA, cudaGetErrorString(e));
  }
  *out = c;
  return ARCS_OK;
}

extern "C" int arcs_host_last_status(arcs_host_ctx* c) { return c ? c->last_status : ARCS_ERR_ARG; }

// rows per chunk: about 32 MB of logits, at least 1 row
static int32_t chunk_rows(const arcs_host_ctx* c, int32_t B, int32_t V) {
  const size_t row = (size_t)V * (c->dtype == ARCS_F32 ? 4 : 2);
  int64_t r = (int64_t)((32u << 20) / std::max<size_t>(row, 1));
  r = std::max<int64_t>(1, std::min<int64_t>(r, B));
  if (B <= 2 * r) r = B > 1 && (size_t)B * row > (8u << 20) ? (B + 1) / 2 : B;  // two chunks overlap copy and compute
  return (int32_t)r;
}

static int finish(arcs_host_ctx* c) {
  // the status word is read after the kernels of BOTH streams have ended: row chunks alternate
  // between the streams, and a chunk on the second one may be the one that raises it
  CU(cudaStreamSynchronize(c->st[1]));
  CU(cudaMemcpyAsync(&c->last_status, c->status, sizeof(int32_t), cudaMemcpyDeviceToHost, c->st[0]));
  CU(cudaStreamSynchronize(c->st[0]));
  if (c->last_status != 0) {  // leave the scratch clean for the next call
    CU(cudaMemset(c->ws_argmax, 0, c->ws_bytes));
    CU(cudaMemset(c->status, 0, sizeof(int32_t)));
    return set_error(c->last_status, "device status set by the kernels");
  }
  return ARCS_OK;
}

extern "C" int arcs_sample_batch_host(arcs_host_ctx* c, const arcs_sample_args* h) {
  if (!c || !h || !h->logits || !h->params || !h->u || !h->token || h->B <= 0 || h->V <= 0 || h->row_stride < h->V)
    return set_error(ARCS_ERR_ARG, "sample_batch_host: bad argument");
  if (h->B > c->max_B || h->V > c->max_V || h->dtype != c->dtype)
    return set_error(ARCS_ERR_ARG, "sample_batch_host: batch larger than the context was created for");
  CU(cudaSetDevice(c->device));
  const int32_t B = h->B, V = h->V;
  const size_t es = c->dtype == ARCS_F32 ? 4 : 2;
  const int64_t nh = h->hist_off ? h->hist_off[B] : 0, nb = h->bias_off ? h->bias_off[B] : 0;
  const bool masked = h->mask != nullptr;
  int64_t mask_rows = 0;
  if (masked) {
    if (h->mask_row) { for (int32_t b = 0; b < B; ++b) mask_rows = std::max<int64_t>(mask_rows, h->mask_row[b] + 1); }
    else mask_rows = B;
  }
  if (nh > c->max_hist || nb > c->max_bias || mask_rows * h->mask_stride > c->max_mask)
    return set_error(ARCS_ERR_ARG, "sample_batch_host: lists or masks larger than the context was created for");
  cudaStream_t s0 = c->st[0];
  // small inputs first, on stream 0; stream 1 waits for them
  CU(cudaMemcpyAsync(c->params, h->params, sizeof(arcs_row_params) * B, cudaMemcpyHostToDevice, s0));
  CU(cudaMemcpyAsync(c->u, h->u, sizeof(double) * B, cudaMemcpyHostToDevice, s0));
  if (h->hist_off) {
    CU(cudaMemcpyAsync(c->hist_off, h->hist_off, sizeof(int32_t) * (B + 1), cudaMemcpyHostToDevice, s0));
    if (nh) CU(cudaMemcpyAsync(c->hist_ids, h->hist_ids, sizeof(int32_t) * nh, cudaMemcpyHostToDevice, s0));
  }
  if (h->bias_off) {
    CU(cudaMemcpyAsync(c->bias_off, h->bias_off, sizeof(int32_t) * (B + 1), cudaMemcpyHostToDevice, s0));
    if (nb) {
      CU(cudaMemcpyAsync(c->bias_ids, h->bias_ids, sizeof(int32_t) * nb, cudaMemcpyHostToDevice, s0));
      CU(cudaMemcpyAsync(c->bias_vals, h->bias_vals, sizeof(float) * nb, cudaMemcpyHostToDevice, s0));
    }
  }
  if (masked) {
    CU(cudaMemcpyAsync(c->mask, h->mask, sizeof(uint32_t) * mask_rows * h->mask_stride, cudaMemcpyHostToDevice, s0));
    if (h->mask_row) CU(cudaMemcpyAsync(c->mask_row, h->mask_row, sizeof(int32_t) * B, cudaMemcpyHostToDevice, s0));
  }
  CU(cudaEventRecord(c->small_ready, s0));
  CU(cudaStreamWaitEvent(c->st[1], c->small_ready, 0));

  const int32_t R = chunk_rows(c, B, V);
  {  // the kernels' scratch depends on the chunk shape and the longest list: grow it when needed
    const size_t need = arcs_sample_workspace_bytes(R, V, masked, (h->hist_off ? h->max_hist : 0) + (h->bias_off ? h->max_bias : 0));
    if (need > c->ws_sample_bytes) {
      CU(cudaStreamSynchronize(c->st[1]));
      for (int i = 0; i < 2; ++i) {
        if (c->ws[i]) CU(cudaFree(c->ws[i]));
        c->ws[i] = nullptr;
      }
      c->ws_sample_bytes = 0;
      for (int i = 0; i < 2; ++i) CU(cudaMalloc(&c->ws[i], need));
      c->ws_sample_bytes = need;
    }
  }
  const bool cands = h->cand_id || h->cand_val || h->cand_pr;
  const bool head = h->head_id || h->head_val || h->n_head;
  if (head && !(masked && h->head_id && h->head_val && h->n_head))
    return set_error(ARCS_ERR_ARG, "sample_batch_host: the ranked head needs a mask and all three of head_id, head_val, n_head");
  if (head && !c->head_id) {
    CU(dalloc(&c->head_id, (size_t)c->max_B * ARCS_HEAD));
    CU(dalloc(&c->head_val, (size_t)c->max_B * ARCS_HEAD));
    CU(dalloc(&c->n_head, (size_t)c->max_B));
  }
  int k = 0;
  for (int32_t r0 = 0; r0 < B; r0 += R, ++k) {
    const int32_t rows = std::min(R, B - r0);
    cudaStream_t st = c->st[k & 1];
    char* dl = c->logits + (size_t)r0 * V * es;
    if (h->row_stride == V) {
      CU(cudaMemcpyAsync(dl, static_cast<const char*>(h->logits) + (size_t)r0 * V * es, (size_t)rows * V * es,
                         cudaMemcpyHostToDevice, st));
    } else {
      CU(cudaMemcpy2DAsync(dl, (size_t)V * es, static_cast<const char*>(h->logits) + (size_t)r0 * h->row_stride * es,
                           (size_t)h->row_stride * es, (size_t)V * es, rows, cudaMemcpyHostToDevice, st));
    }
    arcs_sample_args d = *h;
    d.logits = dl;
    d.B = rows;
    d.row_stride = V;
    d.params = c->params + r0;
    d.hist_off = h->hist_off ? c->hist_off + r0 : nullptr;
    d.hist_ids = c->hist_ids;
    d.bias_off = h->bias_off ? c->bias_off + r0 : nullptr;
    d.bias_ids = c->bias_ids;
    d.bias_vals = c->bias_vals;
    d.u = c->u + r0;
    d.mask = masked ? (h->mask_row ? c->mask : c->mask + (size_t)r0 * h->mask_stride) : nullptr;
    d.mask_row = masked && h->mask_row ? c->mask_row + r0 : nullptr;
    d.token = c->token + r0;
    d.n_cand = c->n_cand + r0;
    d.n_kept = c->n_kept + r0;
    d.flags = c->flags + r0;
    d.cand_id = cands ? c->cand_id + (size_t)r0 * ARCS_KCAP : nullptr;
    d.cand_val = cands ? c->cand_val + (size_t)r0 * ARCS_KCAP : nullptr;
    d.cand_pr = cands ? c->cand_pr + (size_t)r0 * ARCS_KCAP : nullptr;
    d.cand_stride = ARCS_KCAP;
    d.head_id = head ? c->head_id + (size_t)r0 * ARCS_HEAD : nullptr;
    d.head_val = head ? c->head_val + (size_t)r0 * ARCS_HEAD : nullptr;
    d.n_head = head ? c->n_head + r0 : nullptr;
    d.workspace = c->ws[k & 1];
    d.workspace_bytes = c->ws_sample_bytes;
    d.status = c->status;
    const int rc = arcs_sample_batch(&d, st);
    if (rc != ARCS_OK) {
      cudaStreamSynchronize(c->st[0]);
      cudaStreamSynchronize(c->st[1]);
      return rc;
    }
    CU(cudaMemcpyAsync(h->token + r0, d.token, sizeof(int32_t) * rows, cudaMemcpyDeviceToHost, st));
    if (h->n_cand) CU(cudaMemcpyAsync(h->n_cand + r0, d.n_cand, sizeof(int32_t) * rows, cudaMemcpyDeviceToHost, st));
    if (h->n_kept) CU(cudaMemcpyAsync(h->n_kept + r0, d.n_kept, sizeof(int32_t) * rows, cudaMemcpyDeviceToHost, st));
    if (h->flags) CU(cudaMemcpyAsync(h->flags + r0, d.flags, sizeof(int32_t) * rows, cudaMemcpyDeviceToHost, st));
    auto back2d = [&](void* dst, const void* src, size_t elt) {
      return cudaMemcpy2DAsync(static_cast<char*>(dst) + (size_t)r0 * h->cand_stride * elt, (size_t)h->cand_stride * elt,
                               src, (size_t)ARCS_KCAP * elt, (size_t)ARCS_KCAP * elt, rows, cudaMemcpyDeviceToHost, st);
    };
    if (h->cand_id) CU(back2d(h->cand_id, d.cand_id, 4));
    if (h->cand_val) CU(back2d(h->cand_val, d.cand_val, 4));
    if (h->cand_pr) CU(back2d(h->cand_pr, d.cand_pr, 4));
    if (head) {
      CU(cudaMemcpyAsync(h->head_id + (size_t)r0 * ARCS_HEAD, d.head_id, sizeof(int32_t) * ARCS_HEAD * rows, cudaMemcpyDeviceToHost, st));
      CU(cudaMemcpyAsync(h->head_val + (size_t)r0 * ARCS_HEAD, d.head_val, sizeof(float) * ARCS_HEAD * rows, cudaMemcpyDeviceToHost, st));
      CU(cudaMemcpyAsync(h->n_head + r0, d.n_head, sizeof(int32_t) * rows, cudaMemcpyDeviceToHost, st));
    }
  }
  return finish(c);
}

// Sampler::adjusted with host buffers: all pointers of `h` are host pointers.
extern "C" int arcs_adjusted_batch_host(arcs_host_ctx* c, const arcs_adjusted_args* h) {
  if (!c || !h || !h->logits || !h->params || !h->out || h->B <= 0 || h->V <= 0 || h->row_stride < h->V || h->out_stride < h->V)
    return set_error(ARCS_ERR_ARG, "adjusted_batch_host: bad argument");
  if (h->B > c->max_B || h->V > c->max_V || h->dtype != c->dtype)
    return set_error(ARCS_ERR_ARG, "adjusted_batch_host: batch larger than the context was created for");
  CU(cudaSetDevice(c->device));
  const int32_t B = h->B, V = h->V;
  const size_t es = c->dtype == ARCS_F32 ? 4 : 2;
  const int64_t nh = h->hist_off ? h->hist_off[B] : 0, nb = h->bias_off ? h->bias_off[B] : 0;
  if (nh > c->max_hist || nb > c->max_bias) return set_error(ARCS_ERR_ARG, "adjusted_batch_host: lists larger than the context was created for");
  if (!c->adj_out) CU(dalloc(&c->adj_out, (size_t)c->max_B * c->max_V));
  cudaStream_t st = c->st[0];
  CU(cudaMemcpyAsync(c->params, h->params, sizeof(arcs_row_params) * B, cudaMemcpyHostToDevice, st));
  if (h->hist_off) {
    CU(cudaMemcpyAsync(c->hist_off, h->hist_off, sizeof(int32_t) * (B + 1), cudaMemcpyHostToDevice, st));
    if (nh) CU(cudaMemcpyAsync(c->hist_ids, h->hist_ids, sizeof(int32_t) * nh, cudaMemcpyHostToDevice, st));
  }
  if (h->bias_off) {
    CU(cudaMemcpyAsync(c->bias_off, h->bias_off, sizeof(int32_t) * (B + 1), cudaMemcpyHostToDevice, st));
    if (nb) {
      CU(cudaMemcpyAsync(c->bias_ids, h->bias_ids, sizeof(int32_t) * nb, cudaMemcpyHostToDevice, st));
      CU(cudaMemcpyAsync(c->bias_vals, h->bias_vals, sizeof(float) * nb, cudaMemcpyHostToDevice, st));
    }
  }
  CU(cudaMemcpy2DAsync(c->logits, (size_t)V * es, h->logits, (size_t)h->row_stride * es, (size_t)V * es, B, cudaMemcpyHostToDevice, st));
  arcs_adjusted_args d = *h;
  d.logits = c->logits;
  d.row_stride = V;
  d.params = c->params;
  d.hist_off = h->hist_off ? c->hist_off : nullptr;
  d.hist_ids = c->hist_ids;
  d.bias_off = h->bias_off ? c->bias_off : nullptr;
  d.bias_ids = c->bias_ids;
  d.bias_vals = c->bias_vals;
  d.out = c->adj_out;
  d.out_stride = V;
  const int rc = arcs_adjusted_batch(&d, st);
  if (rc != ARCS_OK) return rc;
  CU(cudaMemcpy2DAsync(h->out, (size_t)h->out_stride * 4, c->adj_out, (size_t)V * 4, (size_t)V * 4, B, cudaMemcpyDeviceToHost, st));
  return finish(c);
}

// The last step of Sampler::sample_allowed (tools/sampler.h:121-143) for a host that called its
// predicate itself: n candidates in the order they were found (ids, adjusted logits; host
// pointers), the row's settings, the uniform draw; softmax, min-p / top-p cuts and the draw on the
// device. *token = -1 when n == 0.
extern "C" int arcs_draw_candidates_host(arcs_host_ctx* c, const int32_t* ids, const float* vals, int32_t n, const arcs_row_params* p,
                                         double u, int32_t v_global, int32_t* token, int32_t* n_kept) {
  if (!c || !p || !token || n < 0 || n > ARCS_KCAP || (n > 0 && (!ids || !vals)) || v_global <= 0)
    return set_error(ARCS_ERR_ARG, "draw_candidates_host: bad argument");
  if (n == 0) {
    *token = -1;
    if (n_kept) *n_kept = 0;
    return ARCS_OK;
  }
  CU(cudaSetDevice(c->device));
  if (!c->draw_id) {
    CU(dalloc(&c->draw_id, (size_t)ARCS_KCAP));
    CU(dalloc(&c->draw_val, (size_t)ARCS_KCAP));
    CU(dalloc(&c->draw_n, (size_t)1));
  }
  cudaStream_t st = c->st[0];
  CU(cudaMemcpyAsync(c->draw_id, ids, sizeof(int32_t) * n, cudaMemcpyHostToDevice, st));
  CU(cudaMemcpyAsync(c->draw_val, vals, sizeof(float) * n, cudaMemcpyHostToDevice, st));
  CU(cudaMemcpyAsync(c->draw_n, &n, sizeof(int32_t), cudaMemcpyHostToDevice, st));
  CU(cudaMemcpyAsync(c->params, p, sizeof(arcs_row_params), cudaMemcpyHostToDevice, st));
  CU(cudaMemcpyAsync(c->u, &u, sizeof(double), cudaMemcpyHostToDevice, st));
  arcs_merge_args m = {};
  m.G = 1;
  m.B = 1;
  m.cand_stride = ARCS_KCAP;
  m.cand_id = c->draw_id;
  m.cand_val = c->draw_val;
  m.n_cand = c->draw_n;
  m.params = c->params;
  m.u = c->u;
  m.v_global = v_global;
  m.token = c->token;
  m.n_kept = c->n_kept;
  m.status = c->status;
  const int rc = arcs_merge_batch(&m, st);
  if (rc != ARCS_OK) return rc;
  CU(cudaMemcpyAsync(token, c->token, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  if (n_kept) CU(cudaMemcpyAsync(n_kept, c->n_kept, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  return finish(c);
}

extern "C" int arcs_argmax_batch_host(arcs_host_ctx* c, const arcs_argmax_args* h) {
  if (!c || !h || !h->logits || !h->argmax || h->R <= 0 || h->V <= 0 || h->row_stride < h->V)
    return set_error(ARCS_ERR_ARG, "argmax_batch_host: bad argument");
  if (h->R > c->max_B || h->V > c->max_V || h->dtype != c->dtype || h->slots > c->max_B)
    return set_error(ARCS_ERR_ARG, "argmax_batch_host: batch larger than the context was created for");
  CU(cudaSetDevice(c->device));
  const size_t es = c->dtype == ARCS_F32 ? 4 : 2;
  cudaStream_t st = c->st[0];
  const int32_t R = h->R, V = h->V, S = h->slots;
  if (S > 0) {
    if (!h->row_off || !h->draft_off || !h->accepted || !h->next || h->draft_off[S] > c->max_B)
      return set_error(ARCS_ERR_ARG, "argmax_batch_host: slot lists missing or too long");
    CU(cudaMemcpyAsync(c->row_off, h->row_off, sizeof(int32_t) * (S + 1), cudaMemcpyHostToDevice, st));
    CU(cudaMemcpyAsync(c->draft_off, h->draft_off, sizeof(int32_t) * (S + 1), cudaMemcpyHostToDevice, st));
    if (h->draft_off[S] > 0)
      CU(cudaMemcpyAsync(c->draft, h->draft, sizeof(int32_t) * h->draft_off[S], cudaMemcpyHostToDevice, st));
  }
  if (h->row_stride == V) {
    CU(cudaMemcpyAsync(c->logits, h->logits, (size_t)R * V * es, cudaMemcpyHostToDevice, st));
  } else {
    CU(cudaMemcpy2DAsync(c->logits, (size_t)V * es, h->logits, (size_t)h->row_stride * es, (size_t)V * es, R,
                         cudaMemcpyHostToDevice, st));
  }
  arcs_argmax_args d = *h;
  d.logits = c->logits;
  d.row_stride = V;
  d.argmax = c->argmax;
  d.max_sumexp = h->max_sumexp ? c->max_sumexp : nullptr;
  d.row_off = c->row_off;
  d.draft = c->draft;
  d.draft_off = c->draft_off;
  d.accepted = c->accepted;
  d.next = c->next;
  d.workspace = c->ws_argmax;
  d.workspace_bytes = c->ws_bytes;
  d.status = c->status;
  const int rc = arcs_argmax_batch(&d, st);
  if (rc != ARCS_OK) return rc;
  CU(cudaMemcpyAsync(h->argmax, c->argmax, sizeof(int32_t) * R, cudaMemcpyDeviceToHost, st));
  if (h->max_sumexp) CU(cudaMemcpyAsync(h->max_sumexp, c->max_sumexp, sizeof(float) * 2 * R, cudaMemcpyDeviceToHost, st));
  if (S > 0) {
    CU(cudaMemcpyAsync(h->accepted, c->accepted, sizeof(int32_t) * S, cudaMemcpyDeviceToHost, st));
    CU(cudaMemcpyAsync(h->next, c->next, sizeof(int32_t) * S, cudaMemcpyDeviceToHost, st));
  }
  return finish(c);
}
