"""The DFlash2 candidate selector on the GPU (arcs_dflash_select) against the CPU restatement of
zero/engine_drafters.h:461-506 (pinned to the reference's own loop in test_oracle_pin.py): drafts
bit for bit, for many slots in one call, fp32 and bf16 logits, ties, the probability cut, rows
narrower than topk; the path probability within 2e-6 relative of the exact value."""
import numpy as np
import pytest
import torch

import orc
from arcinfer_b200 import synth
from test_oracle_pin import dflash_case

pytestmark = pytest.mark.gpu


def _run(logits, hproj, pred, succ, tok, topk, max_drafts, min_p, bf16=False):
    import arcinfer_b200 as ab

    lg = torch.from_numpy(synth.f32_to_bf16_bits(logits).view(np.int16)).cuda().view(torch.bfloat16) if bf16 else torch.from_numpy(logits).cuda()
    out = ab.dflash_select(lg, torch.from_numpy(hproj).cuda(), torch.from_numpy(pred.view(np.int16)).cuda(), torch.from_numpy(succ.view(np.int16)).cuda(),
                           torch.from_numpy(tok).cuda(), topk=topk, max_drafts=max_drafts, min_p=min_p)
    torch.cuda.synchronize()
    assert int(out["status"].item()) == 0
    return {k: v.cpu().numpy() for k, v in out.items()}


@pytest.mark.parametrize("bf16", [False, True])
def test_selector_matches_the_reference_loop(bf16):
    g = np.random.default_rng(300 + bf16)
    cuts = 0
    for V, rank, nd, topk, min_p, slots, sharp in [(3000, 64, 7, 16, 0.3, 5, 1.0), (151936, 256, 7, 16, 0.3, 8, 0.8), (5000, 250, 4, 64, 0.0, 3, 1.0),
                                                   (40, 16, 4, 64, 0.3, 2, 1.0), (262144, 256, 7, 16, 0.05, 4, 0.4), (4096, 1024, 2, 8, 0.9, 3, 1.0)]:
        lgs, hps = [], []
        for s in range(slots):
            l, h, pred, succ = dflash_case(g, V, rank, nd, sharp)  # (the codebooks of the last slot serve all)
            if s == 1:
                l[:, 5] = l[:, 9] = l.max(axis=1) + 1  # ties among the top logits
            lgs.append(l)
            hps.append(h)
        logits, hproj = np.stack(lgs), np.stack(hps)
        if bf16:
            logits = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(logits))
        tok = g.integers(0, V, slots).astype(np.int32)
        for max_drafts in (nd, 2):
            out = _run(logits, hproj, pred, succ, tok, topk, max_drafts, min_p, bf16)
            for s in range(slots):
                want, pp = orc.dflash_select(logits[s], hproj[s], pred, succ, topk, max_drafts, int(tok[s]), min_p)
                n = int(out["n_out"][s])
                assert n == len(want) and np.array_equal(out["tokens"][s, :n], want), (V, rank, nd, topk, s, max_drafts)
                assert (out["tokens"][s, n:] == -1).all()
                cuts += n < min(nd, max_drafts)
                if min_p > 0:
                    seen = ~np.isnan(pp)
                    assert np.array_equal(seen, ~np.isnan(out["path_p"][s]))
                    # the reference sums float exponentials in float blocks of 4096 (about 1e-6 of its own
                    # error per position); the exact sums are met ten times closer
                    assert np.allclose(out["path_p"][s][seen], pp[seen], rtol=2e-5, atol=0)
                    ld = logits[s].astype(np.float64)
                    exact = np.cumprod([np.exp(ld[t, want[t]] - ld[t].max()) / np.exp(ld[t] - ld[t].max()).sum() for t in range(len(want))])
                    assert np.allclose(out["path_p"][s][: len(want)], exact, rtol=2e-6, atol=0)
    assert cuts > 0


def test_arguments():
    import ctypes as C

    import arcinfer_b200 as ab

    a = ab.capi.DflashArgs()
    assert ab.lib.arcs_dflash_select(C.byref(a), None) == 1
    assert ab.lib.arcs_dflash_workspace_bytes(0, 7, 1000, 16) == 0
    g = np.random.default_rng(1)
    l, h, pred, succ = dflash_case(g, 500, 8, 3)
    with pytest.raises(ab.ArcsError):  # topk beyond 64
        _run(l[None], h[None], pred, succ, np.zeros(1, np.int32), 65, 3, 0.3)
    # a token outside the codebooks: reported in the status word, no draft
    lg = torch.from_numpy(l[None]).cuda()
    out = ab.dflash_select(lg, torch.from_numpy(h[None]).cuda(), torch.from_numpy(pred.view(np.int16)).cuda(), torch.from_numpy(succ.view(np.int16)).cuda(),
                           torch.tensor([500], dtype=torch.int32, device="cuda"))
    torch.cuda.synchronize()
    assert int(out["status"].item()) == 1 and int(out["n_out"].item()) == 0
    ab.capi.reset_workspaces()
