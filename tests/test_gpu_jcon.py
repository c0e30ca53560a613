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
from test_jcon import DOCS, SCHEMAS, json_vocab, ref_check

pytestmark = pytest.mark.gpu

V = 32768


def _vocab(g):
    toks, off, by = json_vocab(g, 4000)
    off2, by2 = synth.make_vocab(g, V - len(toks))  # filled up with tokens as the measured vocabulary has them
    off = np.concatenate([off, off2[1:] + off[-1]]).astype(np.uint32)
    by = np.concatenate([by, by2[: off2[-1]]])
    return off, by


def _decode(si, doc, steps, seed, tools=None, qwen=False):
    """One constrained decoding on the GPU. With `doc`, tokens that continue it are favoured so
    strongly that the answer spells it (the mask still decides what may be drawn); without, the
    walk is free. tools: a tool list, for the Gemma tool-call form instead of schema si.
    Returns (text, ended)."""
    import arcinfer_b200 as ab

    g = np.random.default_rng(seed)
    if tools is None:
        schema, obj = SCHEMAS[si]
        off, by = _vocab(g)
        jc = jcon.JsonConstraint(schema, obj, off, by)
        check = lambda text: ref_check(schema, obj, text)
    else:
        import test_tcon

        toks, off, by = (test_tcon.qwen_vocab if qwen else test_tcon.call_vocab)(g, 3000)
        off2, by2 = synth.make_vocab(g, V - len(toks))
        off = np.concatenate([off, off2[1:] + off[-1]]).astype(np.uint32)
        by = np.concatenate([by, by2[: off2[-1]]])
        jc = (jcon.JsonConstraint.qwen_call if qwen else jcon.JsonConstraint.gemma_call)(tools, off, by)
        check = test_tcon.ref_qcheck if qwen else test_tcon.ref_check
    lens = np.diff(off.astype(np.int64))
    pieces = [by[off[t] : off[t + 1]].tobytes() for t in range(V)]
    d_off, d_by = torch.from_numpy(off.view(np.int32)).cuda(), torch.from_numpy(by).cuda()
    params = torch.from_numpy(make_params(1, temperature=0.9, top_k=40, top_p=0.95).view(np.uint8)).cuda()
    mask_row = torch.zeros(1, dtype=torch.int32, device="cuda")
    states = torch.zeros(1, dtype=torch.int32, device="cuda")
    # a \\uXXXX escape inside a key of a closed object is a dead end in the reference too (the key's text gets a
    # '?' that no property has, tools/json_constraint.h:185): a free walk keeps away from backslashes
    escapes = np.array([t for t in range(V) if 0x5C in by[off[t] : off[t + 1]]])
    text, ended = b"", False
    for step in range(steps):
        table, dead, done, ts = jc.table(text)
        if ts == jcon.DONE:  # tools/server_chat.h:550-551: the server ends the answer here
            ended = True
            break
        mask = ab.dfa_mask(torch.from_numpy(table.view(np.int16)).cuda(), dead, states, d_off, d_by)
        allowed, _ = jcon.walk_mask(table, dead, off, by)
        want = np.packbits(allowed, bitorder="little").view(np.uint32)
        assert np.array_equal(mask.cpu().numpy().view(np.uint32)[0], want), (si, step, text)
        assert allowed.any(), (si, step, text)
        logits = g.normal(0, 2.0, (1, V)).astype(np.float32)
        if doc is None:
            logits[0, escapes] -= 40.0
        else:
            rest = doc[len(text):]
            follow = [t for t in range(V) if lens[t] and rest.startswith(pieces[t])]
            assert follow and allowed[follow].all(), (si, step, text)  # (a valid document is never cut off by the mask)
            logits[0, follow] += 60.0
        u = torch.from_numpy(g.random(1)).cuda()
        out = ab.sample_batch(torch.from_numpy(logits).cuda(), params, u, mask=mask, mask_row=mask_row)
        torch.cuda.synchronize()
        assert int(out["status"].item()) == 0
        tok = int(out["token"].item())
        assert 0 <= tok < V and allowed[tok], (si, step, text, tok)
        text += pieces[tok]
        if orc.ref is not None:
            assert check(text) != jcon.FAIL, (si, step, text)
    hits, misses = jc.cache_stats()
    assert hits + misses >= 1
    return text, ended


@pytest.mark.parametrize("si", [0, 2, 4, 5, 7])
def test_constrained_decoding_spells_a_valid_document(si):
    schema, obj = SCHEMAS[si]
    for k, doc in enumerate(DOCS[si][:2]):
        d = doc.strip().encode()
        text, ended = _decode(si, d, 4 * len(d) + 8, 700 + 10 * si + k)
        assert ended and text == d, (si, text)
        json.loads(text.decode())
        if orc.ref is not None:
            assert ref_check(schema, obj, text) == jcon.DONE


@pytest.mark.parametrize("si", [1, 3, 6])
def test_free_constrained_walk_stays_a_prefix(si):
    text, ended = _decode(si, None, 40, 900 + si)
    assert ended or len(text) > 0


def test_tool_call_decoding_spells_a_valid_call():
    """The Gemma tool-call form through the same pipeline (tools/tool_constraint.h:66-280)."""
    import test_tcon

    for k, call in enumerate(test_tcon.CALLS[:5]):
        d = call.encode()
        text, ended = _decode(0, d, 4 * len(d) + 8, 950 + k, tools=test_tcon.TOOLS)
        assert ended and text == d, text
        if orc.ref is not None:
            assert test_tcon.ref_check(text) == jcon.DONE


def test_qwen_tool_call_decoding_spells_a_valid_call():
    """The Qwen 3.x tool-call form through the same pipeline (tools/tool_constraint.h:285-371)."""
    import test_tcon

    for k, call in enumerate(test_tcon.QCALLS[:4]):
        d = call.encode()
        text, ended = _decode(0, d, 4 * len(d) + 8, 970 + k, tools=test_tcon.QTOOLS, qwen=True)
        assert ended and text == d, text
        if orc.ref is not None:
            assert test_tcon.ref_qcheck(text) == jcon.DONE
