"""How the path is spread over the GPUs of one box. Rows are independent, so the default is row
sharding with no collective on the data path: rank g owns rows [lo, hi). (The reference has a
single device and no distributed code at all; this layer is new.)"""


def row_range(n_rows, rank, world):
    """Contiguous, balanced: the first n_rows % world ranks get one row more."""
    base, extra = divmod(n_rows, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def vocab_range(V, rank, world, align=2048):
    """Column range of a vocabulary shard, a multiple of `align` wide except for the last."""
    per = -(-V // world)
    per = -(-per // align) * align
    lo = min(V, rank * per)
    return lo, min(V, lo + per)


def gather_tokens(local_tokens, n_rows, world, all_gather):
    """Token ids of all rows from the per-rank pieces; `all_gather(tensor_list, tensor)` is
    torch.distributed.all_gather or a stand-in. Only ids travel (4 bytes per row)."""
    import torch

    sizes = [row_range(n_rows, r, world) for r in range(world)]
    width = max(hi - lo for lo, hi in sizes)
    pad = torch.full((width,), -1, dtype=local_tokens.dtype, device=local_tokens.device)
    pad[: local_tokens.numel()] = local_tokens
    parts = [torch.empty_like(pad) for _ in range(world)]
    all_gather(parts, pad)
    return torch.cat([p[: hi - lo] for p, (lo, hi) in zip(parts, sizes)])


def record_words(k):
    """int32 words of a packed per-row record: k ids, k values (bit patterns), (max, sum exp)."""
    return 2 * k + 2


def vocab_sharded_sample(local_logits, lo, v_global, params, u, all_gather_into, world, sample_batch, merge_records, k, **lists):
    """The vocabulary-sharded step on one rank: this rank's columns [lo, lo + local V) of every row
    go through sample_batch under global ids, which writes each row's candidates straight into a
    packed record of k * 8 + 8 bytes; the records of all ranks are gathered into one preallocated
    buffer (`all_gather_into(out, inp)`: torch.distributed.all_gather_into_tensor over NCCL, or a
    stand-in) that merge_records reads in place for the global choice. The one collective on the
    data path carries B * (k * 8 + 8) bytes per rank. k: at least the largest top_k of the rows."""
    import torch

    B = local_logits.shape[0]
    rec = torch.full((B, record_words(k)), -1, dtype=torch.int32, device=local_logits.device)
    sample_batch(local_logits, params, u, id_base=lo, v_global=v_global, records=rec, **lists)
    gathered = torch.empty((world, B, record_words(k)), dtype=torch.int32, device=local_logits.device)
    all_gather_into(gathered.view(world * B, -1), rec)  # (rank r's rows land at [r * B, (r + 1) * B))
    return merge_records(gathered, params, u, v_global, bias_off=lists.get("bias_off"), bias_vals=lists.get("bias_vals"), want_cands=True)


class VocabShardStep:
    """The same step with everything allocated once: the argument block of the local pass, the
    record buffer it writes, the gathered buffer the merge reads. step() enqueues three pieces of
    work on the current stream: local pass, all-gather, merge. want_mz: every rank also reduces its
    columns to (max, sum exp) per row (arcs_argmax_batch), the pairs travel in the records and the
    merge combines them (out["mz"]): the normaliser of log-probabilities over the whole vocabulary."""

    def __init__(self, local_logits, lo, v_global, params, u, world, k, want_mz=False, **lists):
        import torch

        from . import capi

        self.capi, self.world, self.k, self.want_mz = capi, world, k, want_mz
        self.logits, self.params, self.u, self.v_global, self.lists = local_logits, params, u, v_global, lists
        B = local_logits.shape[0]
        dev = local_logits.device
        self.rec = torch.full((B, record_words(k)), -1, dtype=torch.int32, device=dev)
        self.rec[:, 2 * k :] = 0
        self.gathered = torch.empty((world, B, record_words(k)), dtype=torch.int32, device=dev)
        self.plan = capi.SamplePlan(local_logits, params, u, id_base=lo, v_global=v_global, records=self.rec,
                                    hist_off=lists.get("hist_off"), hist_ids=lists.get("hist_ids"), max_hist=lists.get("max_hist", 0))
        self.collective_bytes_per_rank = B * record_words(k) * 4

    def step(self, all_gather_into):
        self.plan.launch()
        if self.want_mz:
            ms = self.capi.argmax_batch(self.logits, want_lse=True)["max_sumexp"]
            self.rec[:, 2 * self.k :] = ms.view(self.rec.dtype)
        all_gather_into(self.gathered.view(-1, self.rec.shape[1]), self.rec)
        return self.capi.merge_records(self.gathered, self.params, self.u, self.v_global, bias_off=self.lists.get("bias_off"),
                                       bias_vals=self.lists.get("bias_vals"), want_mz=self.want_mz)

    def capture(self, all_gather_into):
        """The three pieces of work of a step as one CUDA graph (call step() at least once before, so
        that the communicator exists). replay() of the returned graph runs the step on the current
        stream without the host between its launches; the outputs are self.out."""
        import torch

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.step(all_gather_into)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                self.out = self.step(all_gather_into)
        torch.cuda.current_stream().wait_stream(side)
        return graph
