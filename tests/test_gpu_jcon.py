"""Constrained JSON decoding end to end on the GPU: schema -> arcs_jcon_table -> arcs_dfa_mask
-> arcs_sample_batch with the mask, step after step, as tools/server_chat.h:548-560 runs it with
its per-candidate predicate. Checked each step: the device mask equals the host walk of the same
table bit for bit, the drawn token is an allowed one, the text stays a prefix for the reference's
own checker (when oracle/_ref is built); at the end the answer is complete, parses as JSON and is
DONE for the reference."""
import json

import numpy as np
import pytest
import torch

import orc
from arcinfer_b200 import jcon, synth
from arcinfer_b200.params import make_params
from test_jcon import SCHEMAS, json_vocab, ref_check

pytestmark = pytest.mark.gpu

V = 32768


def _vocab(g):
    toks, off, by = json_vocab(g, 4000)
    off2, by2 = synth.make_vocab(g, V - len(toks))  # filled up with tokens as the measured vocabulary has them
    off = np.concatenate([off, off2[1:] + off[-1]]).astype(np.uint32)
    by = np.concatenate([by, by2[: off2[-1]]])
    return off, by


@pytest.mark.parametrize("si", [0, 2, 4, 5, 7])
def test_constrained_decoding(si):
    import arcinfer_b200 as ab

    schema, obj = SCHEMAS[si]
    g = np.random.default_rng(700 + si)
    off, by = _vocab(g)
    lens = np.diff(off.astype(np.int64))
    jc = jcon.JsonConstraint(schema, obj, off, by)
    d_off, d_by = torch.from_numpy(off.view(np.int32)).cuda(), torch.from_numpy(by).cuda()
    params = torch.from_numpy(make_params(1, temperature=0.9, top_k=40, top_p=0.95).view(np.uint8)).cuda()
    mask_row = torch.zeros(1, dtype=torch.int32, device="cuda")
    states = torch.zeros(1, dtype=torch.int32, device="cuda")
    # closing and separating tokens are favoured after a while, so that the answer ends
    closers = np.array([t for t in range(V) if 0 < lens[t] <= 2 and all(c in b'"}],:' for c in by[off[t] : off[t + 1]].tobytes())])
    text, ended = b"", False
    for step in range(160):
        table, dead, done, ts = jc.table(text)
        if ts == jcon.DONE:  # tools/server_chat.h:550-551: the server ends the answer here
            ended = True
            break
        mask = ab.dfa_mask(torch.from_numpy(table.view(np.int16)).cuda(), dead, states, d_off, d_by)
        allowed, _ = jcon.walk_mask(table, dead, off, by)
        want = np.packbits(allowed, bitorder="little").view(np.uint32)
        assert np.array_equal(mask.cpu().numpy().view(np.uint32)[0], want), (si, step, text)
        assert allowed.any()
        logits = g.normal(0, 2.0, (1, V)).astype(np.float32)
        if step > 25:
            logits[0, closers] += 12.0
        u = torch.from_numpy(g.random(1)).cuda()
        out = ab.sample_batch(torch.from_numpy(logits).cuda(), params, u, mask=mask, mask_row=mask_row)
        torch.cuda.synchronize()
        assert int(out["status"].item()) == 0
        tok = int(out["token"].item())
        assert 0 <= tok < V and allowed[tok], (si, step, text, tok)
        text += by[off[tok] : off[tok + 1]].tobytes()
        if orc.ref is not None:
            assert ref_check(schema, obj, text) != jcon.FAIL, (si, step, text)
    assert ended, (si, text)
    if b"\\\x00" not in text:  # (a backslash before a NUL byte passes the reference's escape test; no JSON parser takes it)
        json.loads(text.decode("utf-8", errors="replace"))
    if orc.ref is not None:
        assert ref_check(schema, obj, text) == jcon.DONE
    hits, misses = jc.cache_stats()
    assert misses <= step + 1
