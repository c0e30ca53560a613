"""GPU parity: arcs_logprobs_batch through the C ABI against the CPU oracle (tools/server_chat.h:417-441).
Ids of the alternatives bit-exact (ties: lower id first); log probabilities within 1e-6 absolute
(the library sums float exponentials in fp64 in another order than the reference's fp64 loop)."""
import numpy as np
import pytest
import torch

import orc
from arcinfer_b200 import synth

pytestmark = pytest.mark.gpu
TOL = 1e-6


def _run(x, bf16, token, top_n, stride=None, offset=0):
    import arcinfer_b200 as ab
    from gpuutil import to_dev_logits

    lg, V = to_dev_logits(x, bf16, stride, offset)
    tok = None if token is None else torch.from_numpy(np.ascontiguousarray(token, dtype=np.int32)).cuda()
    out = ab.logprobs_batch(lg, tok, top_n, V=V)
    torch.cuda.synchronize()
    return {k: v.cpu().numpy() for k, v in out.items()}


def _check(x, bf16, token, top_n, **kw):
    xf = synth.bf16_bits_to_f32(x) if bf16 else x
    B, V = xf.shape
    got = _run(x, bf16, token, top_n, **kw)
    assert got["status"][0] == 0
    worst = 0.0
    for r in range(B):
        lse, lp, ids, tlp = orc.logprobs(xf[r], -1 if token is None else int(token[r]), min(top_n, V))
        assert abs(got["lse"][r] - lse) <= TOL, (r, got["lse"][r], lse)
        worst = max(worst, abs(got["lse"][r] - lse))
        if token is not None:
            if token[r] >= 0:
                assert abs(got["logprob"][r] - lp) <= TOL
            else:
                assert np.isnan(got["logprob"][r])
        n = min(top_n, V)
        if n:
            assert np.array_equal(got["top_id"][r, :n], ids), (r, V, got["top_id"][r, :n], ids)
            assert np.allclose(got["top_logprob"][r, :n], tlp, rtol=0, atol=TOL)
            assert (got["top_id"][r, n:] == -1).all()
    return worst


@pytest.mark.parametrize("bf16", [False, True])
def test_logprobs_edge_sizes(bf16):
    g = np.random.default_rng(21)
    for V in [1, 2, 7, 9, 33, 127, 129, 1000, 2049, 4097, 8193, 20000, 40961]:
        for B in [1, 3]:
            for mode in range(3):
                if mode == 0:
                    x = (g.standard_normal((B, V), dtype=np.float32) * 3).astype(np.float32)
                elif mode == 1:  # few levels: masses of exact ties
                    x = (0.5 * g.integers(0, 8, (B, V))).astype(np.float32)
                else:  # ascending: every element is a new maximum, the buffer is pruned all the time
                    x = np.tile(np.linspace(-20, 20, V, dtype=np.float32), (B, 1)) + g.standard_normal((B, 1), dtype=np.float32)
                xb = synth.f32_to_bf16_bits(x) if bf16 else x
                tok = g.integers(0, V, B).astype(np.int32)
                for top_n in [0, 1, 20]:
                    for stride, off in [(None, 0), (V + 3, 1)]:
                        _check(xb, bf16, tok, top_n, stride=stride, offset=off)


@pytest.mark.parametrize("bf16", [False, True])
def test_logprobs_full_rows(bf16):
    """rows of the reference's vocabularies; alternatives 20 (the reference's maximum) and 256"""
    g = np.random.default_rng(22)
    worst = 0.0
    for V, B, top_n in [(151936, 8, 20), (262144, 4, 20), (262144, 2, 256), (151936, 2, 5), (50000, 64, 20), (30000, 600, 3)]:
        x = (g.standard_normal((B, V), dtype=np.float32) * 3).astype(np.float32)
        x[0, :: max(1, V // 50)] += 9.0
        xb = synth.f32_to_bf16_bits(x) if bf16 else x
        tok = g.integers(0, V, B).astype(np.int32)
        tok[-1] = -1
        worst = max(worst, _check(xb, bf16, tok, top_n))
    assert worst <= 1e-7  # what the compensated float exponentials actually give


def test_logprobs_infinities_and_no_token():
    g = np.random.default_rng(23)
    V = 5000
    x = (g.standard_normal((2, V), dtype=np.float32) * 2).astype(np.float32)
    x[0, 100:4000] = -np.inf
    x[1, ::7] = -1e30
    _check(x, False, None, 10)


def test_logprobs_many_rows_sum_to_one():
    """size-independent property at a wide batch: the alternatives' probabilities are in
    descending order and exp(lse - max) >= 1; the full softmax sums to one."""
    import arcinfer_b200 as ab

    B, V = 512, 65536
    gen = torch.Generator(device="cuda").manual_seed(3)
    lg = (torch.randn(B, V, device="cuda", generator=gen) * 3).to(torch.bfloat16)
    out = ab.logprobs_batch(lg, None, 20)
    torch.cuda.synchronize()
    assert int(out["status"][0]) == 0
    lse = out["lse"]
    full = torch.exp(lg.double() - lse[:, None]).sum(1)
    assert torch.allclose(full, torch.ones_like(full), rtol=0, atol=1e-6)
    tl = out["top_logprob"]
    assert (tl[:, 1:] <= tl[:, :-1]).all()
    want = torch.topk(lg.float(), 20, dim=1).values.double() - lse[:, None]
    assert torch.allclose(tl, want, rtol=0, atol=1e-12)
