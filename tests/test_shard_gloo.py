"""Row sharding over ranks with a world of 2 on the gloo backend (CPU): every rank selects tokens for
its own rows (here with the CPU oracle standing in for the kernel, which needs a GPU), only token ids
are gathered, and the result equals the single-process result."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import orc
from arcinfer_b200 import shard, synth


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rows(seed, B, V):
    g = synth.rng(seed)
    x = synth.normal_logits(g, B, V, 3.0)
    p = synth.make_params(B, top_k=20, top_p=0.9, repeat_penalty=1.1, repeat_last_n=-1)
    hist = synth.uniform_history(g, B, V, 32)
    return x, p, hist, g.random(B)


def _tokens(x, p, hist, u, lo, hi):
    return np.array([orc.sample(x[b], p[b : b + 1], hist[b], float(u[b]))["token"] for b in range(lo, hi)], np.int32)


def _worker(rank, world, port, B, V, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, p, hist, u = _rows(5, B, V)
    lo, hi = shard.row_range(B, rank, world)
    mine = torch.from_numpy(_tokens(x, p, hist, u, lo, hi))
    allt = shard.gather_tokens(mine, B, world, dist.all_gather)
    if rank == 0:
        out.put(allt.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_row_ranges_cover_everything():
    for n in (1, 7, 8, 1024, 1025):
        for w in (1, 2, 4, 8):
            r = [shard.row_range(n, k, w) for k in range(w)]
            assert r[0][0] == 0 and r[-1][1] == n
            assert all(r[i][1] == r[i + 1][0] for i in range(w - 1))
            assert max(hi - lo for lo, hi in r) - min(hi - lo for lo, hi in r) <= 1
    for V in (151936, 262144, 1000):
        for w in (2, 4, 8):
            r = [shard.vocab_range(V, k, w) for k in range(w)]
            assert r[0][0] == 0 and r[-1][1] == V and all(r[i][1] == r[i + 1][0] for i in range(w - 1))


def test_two_ranks_equal_one_process():
    B, V, world = 7, 3000, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_worker, args=(r, world, port, B, V, q)) for r in range(world)]
    for p in ps:
        p.start()
    got = q.get(timeout=120)
    for p in ps:
        p.join(timeout=120)
        assert p.exitcode == 0
    x, p, hist, u = _rows(5, B, V)
    assert np.array_equal(got, _tokens(x, p, hist, u, 0, B))


# ---- the vocabulary-sharded step (shard.vocab_sharded_sample) with stand-ins for the two kernels:
# every rank ranks its own columns with the CPU oracle, the lists travel through one gloo
# all-gather in the packed layout the real path uses, and the merge picks from the gathered lists.
K = 64  # entries per packed record


def _fake_sample(x_rows, hist, p_rows):
    def f(local_logits, params, u, id_base=0, v_global=0, records=None, **_):
        B, Vl = local_logits.shape
        for b in range(B):
            adj = orc.adjusted(x_rows[b], p_rows[b : b + 1], hist[b])[id_base : id_base + Vl]
            k = min(int(p_rows[b]["top_k"]), Vl)
            order = np.lexsort((np.arange(Vl), -adj.astype(np.float64)))[:k]  # value desc, id asc
            records[b, :K] = -1
            records[b, :k] = torch.from_numpy((order + id_base).astype(np.int32))
            records[b, K : K + k] = torch.from_numpy(adj[order].view(np.int32))
        return {}

    return f


def _fake_merge(p_rows, V):
    def f(records, params, u, v_global, **_):
        G, B, _ = records.shape
        tok = torch.zeros(B, dtype=torch.int32)
        plain = p_rows.copy()
        for name in ("presence_penalty", "frequency_penalty"):
            plain[name] = 0.0
        plain["repeat_penalty"] = 1.0  # the gathered values are already adjusted
        for b in range(B):
            row = np.full(V, -3.0e38, np.float32)
            for g in range(G):
                ids = records[g, b, :K].numpy()
                k = int((ids >= 0).sum())  # (a list ends at its first negative id)
                row[ids[:k]] = records[g, b, K : K + k].numpy().view(np.float32)
            tok[b] = orc.sample(row, plain[b : b + 1], np.zeros(0, np.int32), float(u[b]))["token"]
        return {"token": tok}

    return f


def _vocab_worker(rank, world, port, B, V, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, p, hist, u = _rows(6, B, V)
    lo, hi = shard.vocab_range(V, rank, world, align=256)
    local = torch.from_numpy(np.ascontiguousarray(x[:, lo:hi]))
    res = shard.vocab_sharded_sample(local, lo, V, p, torch.from_numpy(u), dist.all_gather_into_tensor, world, _fake_sample(x, hist, p), _fake_merge(p, V), K)
    if rank == 0:
        out.put(res["token"].numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_vocab_shards_two_ranks_equal_one_process():
    B, V, world = 5, 3000, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_vocab_worker, args=(r, world, port, B, V, q)) for r in range(world)]
    for p in ps:
        p.start()
    got = q.get(timeout=120)
    for p in ps:
        p.join(timeout=120)
        assert p.exitcode == 0
    x, p, hist, u = _rows(6, B, V)
    assert np.array_equal(got, _tokens(x, p, hist, u, 0, B))
