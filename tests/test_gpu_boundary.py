"""Entry points of the boundary beyond sample / argmax: the penalised row (Sampler::adjusted) and
the ranked head of a constrained row (the order in which Sampler::sample_allowed calls its
predicate), each against the CPU checker, bit for bit."""
import numpy as np
import pytest
import torch

import orc
from arcinfer_b200 import synth
from cases import rand_logits, rand_params, rand_recent

pytestmark = pytest.mark.gpu


def _lists(hists, biases):
    ho, hi = synth.csr(hists)
    bo, bi = synth.csr([[b[0] for b in bl] for bl in biases])
    bv = np.array([b[1] for bl in biases for b in bl], np.float32)
    t = lambda a, dt: torch.from_numpy(a if len(a) else np.zeros(1, dt)).cuda()
    return dict(hist_off=torch.from_numpy(ho).cuda(), hist_ids=t(hi, np.int32), bias_off=torch.from_numpy(bo).cuda(),
                bias_ids=t(bi, np.int32), bias_vals=t(bv, np.float32))


@pytest.mark.parametrize("bf16", [False, True])
def test_adjusted_rows_bit_exact(bf16):
    import arcinfer_b200 as ab

    g = np.random.default_rng(31)
    for V, B in [(37, 3), (5000, 16), (151936, 4)]:
        x = np.stack([rand_logits(g, V, b % 3) for b in range(B)])
        xb = synth.f32_to_bf16_bits(x) if bf16 else x
        xf = synth.bf16_bits_to_f32(xb) if bf16 else x
        params, biases, hists = [], [], []
        for b in range(B):
            p, bias = rand_params(g, V, True)
            if b % 4 == 1:  # duplicates, ids out of range, a ban
                bias += [(bias[0][0] if bias else 0, 1.25), (-3, 2.0), (V + 5, -100.0), (int(g.integers(V)), -100.0)]
            if b % 4 == 2:  # nothing set: the row itself
                p, bias = synth.make_params(1), []
            params.append(p)
            biases.append(bias)
            h = rand_recent(g, V, 300)
            hists.append(np.concatenate([h, np.array([-1, V, V + 7], np.int32)]) if b % 2 else h)
        params = np.concatenate(params)
        lg = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16) if bf16 else torch.from_numpy(xb).cuda()
        out = ab.adjusted_batch(lg, ab.capi.params_to_device(params, "cuda"), **_lists(hists, biases))
        torch.cuda.synchronize()
        out = out.cpu().numpy()
        for b in range(B):
            want = orc.adjusted(xf[b], params[b : b + 1], hists[b], biases[b])
            assert np.array_equal(out[b].view(np.uint32), want.view(np.uint32)), (V, b)


def test_ranked_head_is_the_order_of_the_adjusted_row():
    import arcinfer_b200 as ab

    g = np.random.default_rng(32)
    for V, B in [(100, 2), (513, 2), (40000, 6), (151936, 3)]:
        x = np.stack([rand_logits(g, V, 0) for _ in range(B)])
        params, biases, hists = [], [], []
        for b in range(B):
            p, bias = rand_params(g, V, b % 2 == 1)
            p["temperature"] = max(float(p["temperature"][0]), 0.3)
            params.append(p)
            biases.append(bias)
            hists.append(rand_recent(g, V))
        params = np.concatenate(params)
        W = (V + 31) // 32
        mask = torch.zeros(1, W, dtype=torch.int32, device="cuda")  # nothing allowed: only the ranking is asked for
        kw = _lists(hists, biases)
        out = ab.sample_batch(torch.from_numpy(x).cuda(), ab.capi.params_to_device(params, "cuda"), torch.zeros(B, dtype=torch.float64, device="cuda"),
                              mask=mask, mask_row=torch.zeros(B, dtype=torch.int32, device="cuda"), max_hist=80, max_bias=8, want_head=True, **kw)
        torch.cuda.synchronize()
        assert int(out["status"].item()) == 0
        for b in range(B):
            adj = orc.adjusted(x[b], params[b : b + 1], hists[b], biases[b])
            order = np.lexsort((np.arange(V), -adj.astype(np.float64)))[:512]
            n = int(out["n_head"][b])
            assert n == min(V, 512)
            assert np.array_equal(out["head_id"][b, :n].cpu().numpy(), order.astype(np.int32)), (V, b)
            assert np.array_equal(out["head_val"][b, :n].cpu().numpy().view(np.uint32), adj[order].view(np.uint32))
            assert int(out["token"][b]) == -1
