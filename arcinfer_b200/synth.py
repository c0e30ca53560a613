"""Seeded synthetic inputs with the shapes and value distributions of the five measured
workloads (no model, tokenizer or dataset is involved in this path). Everything is numpy on
the host; bf16 data are fp32 draws rounded to nearest-even and carried as uint16 bit patterns.
"""
import numpy as np

from .params import PARAMS_DTYPE, make_params  # noqa: F401

BASE_SEED = 20261125


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def f32_to_bf16_bits(x):
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (b + (0x7FFF + ((b >> 16) & 1))) >> 16
    return r.astype(np.uint16)


def bf16_bits_to_f32(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def csr(lists):
    off = np.zeros(len(lists) + 1, np.int32)
    off[1:] = np.cumsum([len(x) for x in lists])
    ids = np.concatenate([np.asarray(x, np.int32) for x in lists]) if off[-1] else np.zeros(0, np.int32)
    return off, ids.astype(np.int32)


def normal_logits(g, B, V, sigma, bf16=False):
    x = (g.standard_normal((B, V), dtype=np.float32) * np.float32(sigma)).astype(np.float32)
    return f32_to_bf16_bits(x) if bf16 else x


def uniform_history(g, B, V, H):
    return [g.integers(0, V, H, dtype=np.int64).astype(np.int32) for _ in range(B)]


def config1(seed=BASE_SEED + 1):
    """Single row, V=151936 fp32 ~N(0,2.5^2) + 8 spikes at +12; T .7, top-k 20, top-p .8,
    repetition penalty 1.05 over a 64-token history."""
    g = rng(seed)
    V = 151936
    x = normal_logits(g, 1, V, 2.5)
    x[0, g.choice(V, 8, replace=False)] += np.float32(12.0)
    p = make_params(1, temperature=0.7, top_k=20, top_p=0.8, min_p=0.0, repeat_penalty=1.05, repeat_last_n=64)
    return dict(name="single-row", logits=x, bf16=False, params=p, hist=uniform_history(g, 1, V, 64), u=g.random(1))


def config2(seed=BASE_SEED + 2, B=8):
    """Multi-slot decode: B rows x V=262144 fp32 ~N(0,3^2), 256-token histories, presence .5,
    frequency .3, T 1, top-k 64, top-p .95, min-p .05."""
    g = rng(seed)
    V = 262144
    x = normal_logits(g, B, V, 3.0)
    p = make_params(B, temperature=1.0, top_k=64, top_p=0.95, min_p=0.05, presence_penalty=0.5, frequency_penalty=0.3)
    return dict(name="multi-slot", logits=x, bf16=False, params=p, hist=uniform_history(g, B, V, 256), u=g.random(B))


def config3(seed=BASE_SEED + 3, slots=8, rows_per_slot=8, V=151936):
    """Speculative verification: slots x rows bf16 ~N(0,2^2); 7 drafts per slot, each the row
    argmax with probability .7, otherwise a uniform id."""
    g = rng(seed)
    R = slots * rows_per_slot
    bits = normal_logits(g, R, V, 2.0, bf16=True)
    am = bf16_bits_to_f32(bits).argmax(axis=1).astype(np.int32)  # first maximum
    nd = rows_per_slot - 1
    drafts = []
    for s in range(slots):
        d = am[s * rows_per_slot : s * rows_per_slot + nd].copy()
        miss = g.random(nd) >= 0.7
        d[miss] = g.integers(0, V, int(miss.sum()))
        drafts.append(d.astype(np.int32))
    row_off = (np.arange(slots + 1) * rows_per_slot).astype(np.int32)
    draft_off, draft = csr(drafts)
    return dict(name="spec-verify", logits=bits, bf16=True, row_off=row_off, draft=draft, draft_off=draft_off)


def make_vocab(g, V):
    """Token byte strings: length ~ Geometric(.35) clipped to 1..16; each byte printable ASCII
    with probability .7, else uniform 0..255."""
    ln = np.clip(g.geometric(0.35, V), 1, 16).astype(np.int64)
    off = np.zeros(V + 1, np.uint32)
    off[1:] = np.cumsum(ln)
    n = int(off[-1])
    printable = g.integers(0x20, 0x7F, n).astype(np.uint8)
    anyb = g.integers(0, 256, n).astype(np.uint8)
    by = np.where(g.random(n) < 0.7, printable, anyb).astype(np.uint8)
    return off, by


def make_dfa(g, S=96, classes=12):
    """S states; bytes fall into 32 classes of 8 consecutive values; each state accepts `classes`
    of them, each with a random target state; everything else goes to the dead state S (a row
    of the table that maps to itself)."""
    table = np.full((S + 1, 256), S, np.uint16)
    for s in range(S):
        for c in g.choice(32, classes, replace=False):
            table[s, c * 8 : c * 8 + 8] = g.integers(0, S)
    return table, S


def config4(seed=BASE_SEED + 4, B=32, V=151936):
    """Constrained sampling: B rows x V fp32 ~N(0,3^2); synthetic vocabulary and a 96-state byte
    automaton, a current state per row; T .8, top-p .9 (top-k left at the default 20)."""
    g = rng(seed)
    x = normal_logits(g, B, V, 3.0)
    off, by = make_vocab(g, V)
    table, dead = make_dfa(g)
    states = g.integers(0, 96, B).astype(np.int32)
    p = make_params(B, temperature=0.8, top_p=0.9)
    return dict(name="constrained", logits=x, bf16=False, params=p, hist=[np.zeros(0, np.int32)] * B, u=g.random(B),
                byte_off=off, bytes=by, table=table, dead=dead, states=states)


def config5_rows(seed=BASE_SEED + 5, B=1024, V=262144, H=512):
    """Wide batch: B rows x V bf16 ~N(0,3^2); top-k 50, top-p .95, repetition penalty 1.1 over
    the whole 512-token history (repeat_last_n -1); temperature 1, min-p 0 (defaults)."""
    g = rng(seed)
    bits = normal_logits(g, B, V, 3.0, bf16=True)
    p = make_params(B, top_k=50, top_p=0.95, repeat_penalty=1.1, repeat_last_n=-1)
    return dict(name="wide-batch", logits=bits, bf16=True, params=p, hist=uniform_history(g, B, V, H), u=g.random(B))
