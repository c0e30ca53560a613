"""Golden vectors produced by the reference's own Sampler (tests/golden/make_golden.py): the CPU
oracle must reproduce them (here, without a GPU) and so must the CUDA path (on the GPU box, where the
reference tree does not exist)."""
import os

import numpy as np
import pytest

import orc

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sampler_golden.npz"))


def _case(i):
    bias = list(zip(G[f"bias_id_{i}"].tolist(), G[f"bias_val_{i}"].tolist()))
    mask = G[f"mask_{i}"]
    return (G[f"logits_{i}"], G[f"params_{i}"].view(orc.PARAMS_DTYPE), G[f"recent_{i}"], float(G[f"u_{i}"][0]), bias,
            mask if len(mask) else None, int(G[f"token_{i}"][0]), int(G[f"token_{i}"][1]))


def test_oracle_reproduces_reference_tokens():
    n = int(G["count"][0])
    assert n >= 32
    for i in range(n):
        l, p, rec, u, bias, mask, tok, first = _case(i)
        o = orc.sample(l, p, rec, u, bias, mask)
        assert o["token"] == tok, i
        if mask is not None and o["n_cand"] > 0 or (mask is not None and tok < 0):
            assert bool(o["flags"] & 2) == bool(first) or tok < 0, i


@pytest.mark.gpu
def test_cuda_reproduces_reference_tokens():
    from gpuutil import run_gpu_sample

    n = int(G["count"][0])
    for i in range(n):
        l, p, rec, u, bias, mask, tok, first = _case(i)
        out = run_gpu_sample(l[None, :], False, p, [rec], [u], [bias], masks=None if mask is None else mask[None, :],
                             want_cands=False)
        assert int(out["status"][0]) == 0
        assert int(out["token"][0]) == tok, i
