"""Random sampler cases in the spirit of the reference's own test (tests/test_sampler.cpp:156-194
there: logits continuous / few discrete levels / mostly one value; 0-80 recent tokens; temperature,
top_k, top_p, min_p from small sets; optional frequency / repeat / presence penalties and biases)."""
import numpy as np

from orc import PARAMS_DTYPE


def rand_logits(g, V, mode):
    if mode == 0:
        return (g.standard_normal(V, dtype=np.float32) * np.float32(3.0)).astype(np.float32)
    if mode == 1:  # a few levels: many exact ties
        return (0.5 * g.integers(0, 8, V)).astype(np.float32)
    hi = g.integers(0, 100, V) < 3
    return np.where(hi, 1.0 + 0.25 * g.integers(0, 8, V), -2.0).astype(np.float32)


def rand_recent(g, V, nmax=80):
    return g.integers(0, V, int(g.integers(0, nmax + 1))).astype(np.int32)


def rand_params(g, V, penalties, allow_k0=True):
    p = np.zeros(1, PARAMS_DTYPE)
    p["temperature"] = g.choice([0.0, 0.3, 0.7, 1.0, 1.5])
    k = int(g.choice([1, 5, 20, 40, 0]))
    if k == 0 and (V < 256 or not allow_k0):
        k = 20
    p["top_k"] = k
    p["top_p"] = g.choice(np.array([0.8, 0.95, 1.0], np.float32))
    p["min_p"] = g.choice(np.array([0.0, 0.0, 0.05], np.float32))
    p["repeat_penalty"], p["repeat_last_n"] = 1.0, 64
    bias = []
    if penalties:
        if g.integers(2):
            p["frequency_penalty"] = 0.3
        if g.integers(2):
            p["repeat_penalty"] = 1.1
            p["repeat_last_n"] = -1 if g.integers(2) else 64
        if g.integers(2):
            p["presence_penalty"] = 0.7 if g.integers(2) else -0.4
        if g.integers(2):
            bias.append((int(g.integers(V)), 2.5))
        if g.integers(2):
            bias.append((int(g.integers(V)), -7.0))
        if g.integers(4) == 0:
            bias.append((int(g.integers(V)), -100.0))
    return p, bias


def rand_mask(g, V, density):
    bits = g.random(V) < density
    pad = np.zeros(((V + 31) // 32) * 32, bool)
    pad[:V] = bits
    return np.packbits(pad.reshape(-1, 32), axis=1, bitorder="little").view(np.uint32).reshape(-1)
