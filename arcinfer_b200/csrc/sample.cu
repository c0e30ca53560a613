// sample_batch: penalties + temperature / top-k / top-p / min-p (+ allowed-token mask) with one
// pass over the logits. Two launches on the caller's stream: stream (the pass itself, which also
// prepares each item's touched tokens ahead of the pass) and finish (per row: order, softmax,
// cuts, draw), which runs beside the stream kernel and takes each row as it is released. The
// kernels hand their results on through the workspace.
#include "sample_finish.cuh"
#include "sample_stream.cuh"

using namespace arcs;

// launch `kernel` so that it may start before the kernel ahead of it on the stream has finished
// (it waits on the device before reading that kernel's output)
template <typename K>
static cudaError_t launch_dependent(K kernel, unsigned grid, unsigned block, size_t smem, cudaStream_t st, const SampleDev& a, bool overlap) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap ? 1 : 0;  // (without the attribute: an ordinary launch, e.g. when the kernels are timed one by one)
  return cudaLaunchKernelEx(&cfg, kernel, a);
}

constexpr int kMaxRows = 65536;
constexpr int kItemsPerSm = 1;        // work items per SM that few rows are cut into
constexpr int kFinishThreads = 128;   // threads of the finish kernel's CTA (four rows per CTA; one with an allowed-token mask)

// Rows with an allowed-token mask are not cut: the ranked head needs the 512 best of the whole
// row, and every segment would have to keep 512 of its own (a list that a short segment cannot
// prune before it ends).
static void plan_items(int B, int V, bool masked, int* nseg, int* seg_len) {
  if (!masked) return plan_segments(B, V, nseg, seg_len, kItemsPerSm);
  *nseg = 1;
  *seg_len = ((V + 2047) / 2048) * 2048;
}
// Few rows: a CTA of the finish kernel takes one row, so that a row the warp path leaves does not
// wait for its neighbours.
static int finish_rows_per_cta(int B) { return B > 2 * kSmCount ? 4 : 1; }

static int table_slots(int max_list) {
  int slots = kGroup;
  while (slots < 2 * max_list && slots < kMaxTableSlots) slots <<= 1;
  return slots;
}

extern "C" size_t arcs_sample_workspace_bytes(int32_t B, int32_t V, int32_t masked, int32_t max_list) {
  if (B <= 0 || V <= 0 || max_list < 0) return 0;
  int nseg, seg_len;
  plan_items(B, V, masked != 0, &nseg, &seg_len);
  return (size_t)B * nseg * (size_t)item_block_bytes(masked != 0, table_slots(max_list));
}

// events[0..2], when given, are recorded before the first launch and after each of the two
static int sample_launch(const arcs_sample_args* g, void* stream, cudaEvent_t* events) {
  if (int inj = fault_injected()) return inj;
  if (!g || !g->logits || !g->params || !g->u || !g->token || g->B <= 0 || g->V <= 0 || g->row_stride < g->V ||
      (g->dtype != ARCS_F32 && g->dtype != ARCS_BF16))
    return set_error(ARCS_ERR_ARG, "sample_batch: bad argument");
  if ((g->hist_off && !g->hist_ids) || (g->bias_off && (!g->bias_ids || !g->bias_vals)))
    return set_error(ARCS_ERR_ARG, "sample_batch: list offsets without the list");
  if (g->max_hist < 0 || g->max_bias < 0 || g->max_hist > (1 << 19) || g->max_bias > (1 << 16))
    return set_error(ARCS_ERR_ARG, "sample_batch: max_hist / max_bias out of range");
  if (g->B > kMaxRows) return set_error(ARCS_ERR_ARG, "sample_batch: more than 65536 rows in one call");
  if ((int64_t)g->V + g->id_base >= (int64_t)kIdMask || g->v_global >= (int32_t)kIdMask)
    return set_error(ARCS_ERR_ARG, "sample_batch: token ids must stay below 2^29 - 1");
  const bool masked = g->mask != nullptr;
  if (masked && g->mask_stride < (g->V + 31) / 32) return set_error(ARCS_ERR_ARG, "sample_batch: mask_stride too small");
  if (masked && (g->id_base != 0 || (g->v_global != 0 && g->v_global != g->V)))
    return set_error(ARCS_ERR_ARG, "sample_batch: a mask cannot be combined with a vocabulary shard");
  if ((g->head_id || g->head_val || g->n_head) && !(masked && g->head_id && g->head_val && g->n_head))
    return set_error(ARCS_ERR_ARG, "sample_batch: the ranked head needs a mask and all three of head_id, head_val, n_head");
  if ((g->cand_id || g->cand_val || g->cand_pr) &&
      (g->cand_width < 0 || g->cand_width > ARCS_KCAP || g->cand_stride < (g->cand_width > 0 ? g->cand_width : ARCS_KCAP)))
    return set_error(ARCS_ERR_ARG, "sample_batch: cand_stride must be at least cand_width (ARCS_KCAP when that is 0)");

  SampleDev a;
  plan_items(g->B, g->V, masked, &a.nseg, &a.seg_len);
  a.rows_per_cta = finish_rows_per_cta(g->B);
  a.logits = g->logits;
  a.row_stride = g->row_stride;
  a.B = g->B;
  a.V = g->V;
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
  const int max_list = a.max_hist + a.max_bias;
  const int slots = table_slots(max_list);
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
  a.cand_width = g->cand_width > 0 ? g->cand_width : g->cand_stride;
  a.head_id = g->head_id;
  a.head_val = g->head_val;
  a.n_head = g->n_head;
  a.ws_items = static_cast<char*>(g->workspace);
  a.item_block = item_block_bytes(masked, slots);
  a.status = g->status;
  a.merge_G = 0;
  a.merge_stride = 0;
  a.merge_id = nullptr;
  a.merge_val = nullptr;
  a.merge_n = nullptr;
  a.merge_width = 0;
  a.merge_mz = nullptr;
  a.merge_mz_stride = 0;
  a.mz_out = nullptr;
  if (!g->workspace || g->workspace_bytes < arcs_sample_workspace_bytes(g->B, g->V, masked, max_list))
    return set_error(ARCS_ERR_WORKSPACE, "sample_batch: workspace too small");
  if ((reinterpret_cast<uintptr_t>(g->workspace) & 15u) != 0) return set_error(ARCS_ERR_WORKSPACE, "sample_batch: workspace must be 16-byte aligned");

  const size_t smem_s = stream_smem_bytes(masked, slots);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int items = a.nseg * a.B;
  const unsigned grid_s = (unsigned)(items < kSmCount ? items : kSmCount);
#define ARCS_LAUNCH(T, M)                                                                                          \
  do {                                                                                                             \
    static std::atomic<unsigned long long> attr_done{0};                                                           \
    const cudaError_t attr_rc = ensure_dynamic_smem(stream_kernel<T, M>, 227 * 1024, attr_done);                   \
    if (attr_rc != cudaSuccess) return set_error(ARCS_ERR_CUDA, cudaGetErrorString(attr_rc));                      \
    if (events) cudaEventRecord(events[0], st);                                                                    \
    stream_kernel<T, M><<<grid_s, kThreadsS, smem_s, st>>>(a);                                                     \
    if (events) cudaEventRecord(events[1], st);                                                                    \
    const cudaError_t e = launch_dependent(finish_kernel<T, M, kFinishThreads>, (unsigned)(M ? a.B : (a.B + a.rows_per_cta - 1) / a.rows_per_cta), kFinishThreads, 0, st, a, events == nullptr); \
    if (e != cudaSuccess) return set_error(ARCS_ERR_CUDA, cudaGetErrorString(e));                                  \
    if (events) cudaEventRecord(events[2], st);                                                                    \
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

extern "C" int arcs_sample_batch(const arcs_sample_args* g, void* stream) { return sample_launch(g, stream, nullptr); }

extern "C" int arcs_sample_batch_timed(const arcs_sample_args* g, void* stream, float* ms2) {
  if (!ms2) return set_error(ARCS_ERR_ARG, "sample_batch_timed: no output");
  cudaEvent_t ev[3];
  for (auto& e : ev)
    if (cudaEventCreate(&e) != cudaSuccess) return set_error(ARCS_ERR_CUDA, "sample_batch_timed: cannot create events");
  int rc = sample_launch(g, stream, ev);
  if (rc == ARCS_OK && cudaEventSynchronize(ev[2]) != cudaSuccess) rc = set_error(ARCS_ERR_CUDA, "sample_batch_timed: synchronize failed");
  for (int i = 0; i < 2 && rc == ARCS_OK; ++i)
    if (cudaEventElapsedTime(&ms2[i], ev[i], ev[i + 1]) != cudaSuccess) rc = set_error(ARCS_ERR_CUDA, "sample_batch_timed: elapsed time failed");
  for (auto& e : ev) cudaEventDestroy(e);
  return rc;
}

// ---- vocabulary shards: the global choice from the shards' gathered candidate lists
extern "C" int arcs_merge_batch(const arcs_merge_args* g, void* stream) {
  if (int inj = fault_injected()) return inj;
  if (!g || g->G <= 0 || g->G > 64 || g->B <= 0 || g->B > kMaxRows || g->cand_stride <= 0 || !g->cand_id || !g->cand_val ||
      g->cand_width < 0 || g->cand_width > g->cand_stride || (!g->n_cand && g->cand_width == 0) || (g->mz_out && (!g->shard_mz || g->mz_stride < 2)) ||
      !g->params || !g->u || !g->token || g->v_global <= 0 || g->v_global >= (int32_t)kIdMask)
    return set_error(ARCS_ERR_ARG, "merge_batch: bad argument");
  if (g->bias_off && !g->bias_vals) return set_error(ARCS_ERR_ARG, "merge_batch: bias offsets without the values");
  if ((g->out_id || g->out_val || g->out_pr) && g->out_stride < ARCS_KCAP)
    return set_error(ARCS_ERR_ARG, "merge_batch: out_stride must be at least ARCS_KCAP");
  SampleDev a = {};
  a.B = g->B;
  a.V = g->v_global;
  a.v_global = g->v_global;
  a.nseg = 1;
  a.params = g->params;
  a.u = g->u;
  a.bias_off = g->bias_off;
  a.bias_vals = g->bias_vals;
  a.max_bias = 1 << 30;
  a.hash_slots = kGroup;
  a.token = g->token;
  a.n_cand = g->n_cand_out;
  a.n_kept = g->n_kept;
  a.flags = g->flags;
  a.cand_id = g->out_id;
  a.cand_val = g->out_val;
  a.cand_pr = g->out_pr;
  a.cand_stride = g->out_stride;
  a.cand_width = g->out_stride;
  a.status = g->status;
  a.merge_G = g->G;
  a.merge_stride = g->cand_stride;
  a.merge_id = g->cand_id;
  a.merge_val = g->cand_val;
  a.merge_n = g->n_cand;
  a.merge_width = g->cand_width > 0 ? g->cand_width : g->cand_stride;
  a.merge_mz = g->shard_mz;
  a.merge_mz_stride = g->mz_stride;
  a.mz_out = g->mz_out;
  a.rows_per_cta = 4;
  finish_kernel<float, false, kFinishThreads><<<(unsigned)((g->B + 3) / 4), kFinishThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return check_launch("merge_batch");
}
