"""Draft verification under sampling (tools/server_chat.h:578-591) in one pass: every verification
row of every slot is sampled in one arcs_sample_batch call, row i of a slot with the slot's history
followed by its first i drafts, and arcs_accept_batch walks the tokens. Checked against the
reference's sequence restated with the CPU checker: sample a row, accept if it equals the draft,
append it to the history, go on to the next row."""
import numpy as np
import pytest
import torch

import orc
from arcinfer_b200 import synth
from arcinfer_b200.capi import verification_histories
from cases import rand_logits

pytestmark = pytest.mark.gpu


def _sequential(x_rows, p, hist, drafts, us):
    """what the server does for one slot: (accepted, next token)"""
    gen = list(hist)
    acc = 0
    for i in range(len(drafts) + 1):
        t = orc.sample(x_rows[i], p, np.asarray(gen, np.int32), float(us[i]))["token"]
        if i < len(drafts) and t == drafts[i]:
            acc += 1
            gen.append(t)
            continue
        return acc, t
    raise AssertionError


@pytest.mark.parametrize("bf16", [False, True])
def test_sampled_verification_in_one_pass(bf16):
    import arcinfer_b200 as ab
    from gpuutil import to_dev_logits

    g = np.random.default_rng(60 + bf16)
    for V, slots in [(5000, 6), (151936, 4)]:
        hists, drafts, rows, us, params = [], [], [], [], []
        for s in range(slots):
            k = int(g.integers(0, 8))
            p = synth.make_params(1, temperature=0.7, top_k=int(g.choice([1, 8, 40])), top_p=0.9, repeat_penalty=float(g.choice([1.0, 1.3])),
                                  presence_penalty=float(g.choice([0.0, 0.8])), frequency_penalty=float(g.choice([0.0, 0.4])), repeat_last_n=int(g.choice([-1, 16, 64])))
            hist = g.integers(0, V, int(g.integers(0, 40))).astype(np.int32)
            x = np.stack([rand_logits(g, V, 0) * 3 for _ in range(k + 1)]).astype(np.float32)
            if bf16:
                x = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(x))
            u = g.random(k + 1)
            # drafts: what the sequence itself would choose for a while (so that they are accepted), then a miss
            want, gen = [], list(hist)
            good = int(g.integers(0, k + 1))
            for i in range(k):
                t = orc.sample(x[i], p, np.asarray(gen, np.int32), float(u[i]))["token"]
                if i >= good:
                    t = (t + 1) % V
                want.append(t)
                gen.append(t)
            hists.append(hist)
            drafts.append(np.asarray(want, np.int32))
            rows.append(x)
            us.append(u)
            params.append(p)
        X = np.concatenate(rows)
        R = X.shape[0]
        prow = np.concatenate([np.repeat(params[s], len(drafts[s]) + 1) for s in range(slots)])
        ho, hi, row_off, d_off, dr = verification_histories(hists, drafts)
        lg, _ = to_dev_logits(synth.f32_to_bf16_bits(X) if bf16 else X, bf16)
        z = lambda a: torch.from_numpy(a).cuda() if len(a) else torch.zeros(1, dtype=torch.int32, device="cuda")
        out = ab.sample_batch(lg, ab.capi.params_to_device(prow, "cuda"), torch.from_numpy(np.concatenate(us)).cuda(), hist_off=z(ho), hist_ids=z(hi),
                              max_hist=int(np.diff(ho).max()), V=V)
        acc, nxt = ab.accept_batch(out["token"], z(row_off), z(dr), z(d_off))
        torch.cuda.synchronize()
        assert int(out["status"].item()) == 0 and R == row_off[-1]
        acc, nxt = acc.cpu().numpy(), nxt.cpu().numpy()
        n_acc = 0
        for s in range(slots):
            want = _sequential(rows[s], params[s], hists[s], drafts[s], us[s])
            assert (int(acc[s]), int(nxt[s])) == want, (V, s, drafts[s])
            n_acc += want[0]
        assert n_acc > 0
