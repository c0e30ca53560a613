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
