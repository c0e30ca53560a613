"""Generates tests/golden/sampler_golden.npz from the reference's OWN Sampler (tools/sampler.h of
rizagp/arcinfer, compiled in place into oracle/_ref/libarcs_ref.so by `make -C oracle ref`).
Run from the repository root where the reference tree is present:  python tests/golden/make_golden.py
Only cases whose candidates have pairwise distinct logits are kept: there the reference's result
does not depend on its standard library's heap order."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import orc  # noqa: E402
from cases import rand_logits, rand_mask, rand_params, rand_recent  # noqa: E402


def main():
    assert orc.ref is not None, "build oracle/_ref first (make -C oracle ref)"
    g = np.random.default_rng(20261125)
    out = {}
    n = 0
    while n < 64:
        V = int(g.integers(40, 1200))
        l = rand_logits(g, V, 0)
        pen = bool(n % 2)
        p, bias = rand_params(g, V, pen)
        rec = rand_recent(g, V)
        masked = n % 4 >= 2
        mask = rand_mask(g, V, float(g.choice([1.0, 0.5, 0.05]))) if masked else None
        seed = int(g.integers(1, 2**62)) | 1
        u = float(orc.u_from_seed(seed, 1)[0])
        o = orc.sample(l, p, rec, u, bias, mask)
        if o["flags"] & (1 | 16):
            continue
        if masked:
            tok, _, first = orc.ref_sample_seq(l, p, rec, seed, 1, False, bias, mask)
            flag = int(first[0])
        else:
            tok = orc.ref_sample_seq(l, p, rec, seed, 1, False, bias)
            flag = 0
        out[f"logits_{n}"] = l
        out[f"params_{n}"] = p
        out[f"recent_{n}"] = rec
        out[f"bias_id_{n}"] = np.array([b[0] for b in bias], np.int32)
        out[f"bias_val_{n}"] = np.array([b[1] for b in bias], np.float32)
        out[f"mask_{n}"] = mask if masked else np.zeros(0, np.uint32)
        out[f"u_{n}"] = np.array([u])
        out[f"token_{n}"] = np.array([int(tok[0]), flag], np.int32)
        n += 1
    out["count"] = np.array([n])
    np.savez_compressed(os.path.join(HERE, "sampler_golden.npz"), **out)
    print("wrote", n, "cases")


if __name__ == "__main__":
    main()
