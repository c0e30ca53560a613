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


def vocab_sharded_sample(local_logits, lo, v_global, params, u, all_gather, world, sample_batch, merge_batch, **lists):
    """The vocabulary-sharded step on one rank: this rank's columns [lo, lo + local V) of every row
    go through sample_batch under global ids, the per-row candidate lists of all ranks are gathered
    (`all_gather(list_of_tensors, tensor)`: torch.distributed.all_gather over NCCL, or a stand-in),
    and merge_batch takes the global choice. The one collective on the data path carries
    B * (k * 8 + 4) bytes per rank."""
    import torch

    out = sample_batch(local_logits, params, u, id_base=lo, v_global=v_global, want_cands=True, **lists)
    # one message per rank: ids, values (bit patterns) and list lengths side by side
    k = out["cand_id"].shape[1]
    mine = torch.cat([out["cand_id"], out["cand_val"].view(torch.int32), out["n_cand"][:, None]], dim=1).contiguous()
    got = [torch.empty_like(mine) for _ in range(world)]
    all_gather(got, mine)
    allp = torch.stack(got)
    cand_id = allp[:, :, :k].contiguous()
    cand_val = allp[:, :, k : 2 * k].contiguous().view(torch.float32)
    n_cand = allp[:, :, 2 * k].contiguous()
    return merge_batch(cand_id, cand_val, n_cand, params, u, v_global,
                       bias_off=lists.get("bias_off"), bias_vals=lists.get("bias_vals"), want_cands=True)
