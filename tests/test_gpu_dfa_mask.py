"""The automaton mask kernel (arcs_dfa_mask) against the CPU walk, bit for bit, on the branches
the constrained-sampling workload never reaches: empty pieces, control tokens with special_ok 0
and 1, vocabularies that are not a multiple of 32, a start state that is the dead state, many
start states in one call, and output rows wider than the mask."""
import numpy as np
import pytest
import torch

import orc
from arcinfer_b200 import synth

pytestmark = pytest.mark.gpu


def _vocab(g, V, empty_frac=0.1):
    """byte strings of length 0..16 (some empty), bytes as in the measured vocabulary"""
    off, by = synth.make_vocab(g, V)
    ln = np.diff(off.astype(np.int64))
    ln[g.random(V) < empty_frac] = 0
    off2 = np.zeros(V + 1, np.uint32)
    off2[1:] = np.cumsum(ln)
    by2 = np.concatenate([by[off[t] : off[t] + ln[t]] for t in range(V)] + [np.zeros(1, np.uint8)])
    return off2, by2


def _gpu(table, dead, states, off, by, special, special_ok, V, out_stride=None):
    import arcinfer_b200 as ab

    sp = None if special is None else torch.from_numpy(special).cuda()
    out = ab.dfa_mask(torch.from_numpy(table.view(np.int16)).cuda(), dead, torch.from_numpy(np.asarray(states, np.int32)).cuda(),
                      torch.from_numpy(off.view(np.int32)).cuda(), torch.from_numpy(by).cuda(), special=sp, special_ok=special_ok,
                      V=V, out_stride=out_stride)
    torch.cuda.synchronize()
    return out.cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("V", [1, 31, 33, 1000, 4097])
def test_mask_edges(V):
    g = np.random.default_rng(40 + V)
    table, dead = synth.make_dfa(g, S=24, classes=20)
    off, by = _vocab(g, V)
    special = (g.random(V) < 0.2).astype(np.uint8)
    states = list(range(0, 24, 5)) + [dead]  # the dead state as a start state: nothing is allowed
    W = (V + 31) // 32
    for sp, sp_ok in [(None, False), (special, False), (special, True)]:
        for stride in [None, W + 3]:
            got = _gpu(table, dead, states, off, by, sp, sp_ok, V, out_stride=stride)
            for i, s in enumerate(states):
                want = orc.dfa_mask(table, dead, int(s), off, by, sp, sp_ok)
                assert np.array_equal(got[i, :W], want), (V, s, sp is not None, sp_ok, stride)
                if stride is not None:
                    assert not got[i, W:].any()
            assert not got[len(states) - 1].any()
    # something was allowed and something refused, and the three variants differ
    a = _gpu(table, dead, states[:1], off, by, None, False, V)
    b = _gpu(table, dead, states[:1], off, by, special, False, V)
    c = _gpu(table, dead, states[:1], off, by, special, True, V)
    assert np.array_equal(a, c)
    if V >= 1000:
        assert a.any() and not np.array_equal(a, b)


def test_many_states_one_call():
    g = np.random.default_rng(77)
    V = 3001
    table, dead = synth.make_dfa(g, S=96, classes=12)
    off, by = _vocab(g, V, empty_frac=0.02)
    states = np.arange(97, dtype=np.int32)
    got = _gpu(table, dead, states, off, by, None, False, V, out_stride=(V + 31) // 32 + 1)
    for s in states:
        assert np.array_equal(got[s, : (V + 31) // 32], orc.dfa_mask(table, dead, int(s), off, by)), s
