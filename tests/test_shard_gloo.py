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
