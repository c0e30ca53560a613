"""Pins the plain-C oracle to the reference's own code: oracle/_ref/libarcs_ref.so is the
reference's Sampler compiled from its sources (built where the reference tree is present; it
travels with the repository's built files). Rows in which two candidates have exactly equal
logits are counted separately: there the reference's order is whatever its standard library's
heap code produces, and the oracle uses (value desc, id asc) instead."""
import numpy as np
import pytest

import orc
from arcinfer_b200 import synth
from cases import rand_logits, rand_mask, rand_params, rand_recent

needs_ref = pytest.mark.skipif(orc.ref is None, reason="oracle/_ref/libarcs_ref.so not built")
needs_slices = pytest.mark.skipif(orc.refslices is None, reason="oracle/_ref/libarcs_refslices.so not built")


@needs_ref
def test_uniform_draw_matches_libstdcxx():
    g = np.random.default_rng(1)
    for _ in range(200):
        seed = int(g.integers(1, 2**63))
        tot = float(g.random()) + 1e-3
        a = orc.u_from_seed(seed, 8) * tot
        b = orc.ref_uniform(seed, tot, 8)
        assert np.array_equal(a, b)


@needs_ref
def test_adjusted_bit_exact():
    g = np.random.default_rng(2)
    for c in range(300):
        V = int(g.integers(2, 3000))
        l = rand_logits(g, V, c % 3)
        p, bias = rand_params(g, V, True)
        rec = rand_recent(g, V)
        if c % 5 == 0:  # duplicate bias entries, ids out of range, a ban lifted by nothing
            bias += [(bias[0][0] if bias else 0, 1.25), (-3, 2.0), (V + 5, -100.0)]
            rec = np.concatenate([rec, np.array([-1, V, V + 7], np.int32)])
        assert np.array_equal(orc.adjusted(l, p, rec, bias).view(np.uint32), orc.ref_adjusted(l, p, rec, bias).view(np.uint32))


def _run_sample_cases(pen, n_cases, seed):
    g = np.random.default_rng(seed)
    bad = ties = n = 0
    for c in range(n_cases):
        V = 151936 if c % 40 == 0 else int(g.integers(64, 6064))
        l = rand_logits(g, V, 0 if pen else c % 3)
        p, bias = rand_params(g, V, pen)
        rec = list(rand_recent(g, V))
        s = int(g.integers(1, 2**62)) | 1
        want = orc.ref_sample_seq(l, p, np.array(rec, np.int32), s, ndraws=4, append=True, bias=bias)
        us = orc.u_from_seed(s, 4)
        draw = 0
        for d in range(4):
            r = orc.sample(l, p, np.array(rec, np.int32), us[draw], bias)
            if p["temperature"][0] > 0:
                draw += 1
            n += 1
            if r["flags"] & 1:
                ties += 1
                rec.append(int(want[d]))
                continue
            bad += r["token"] != want[d]
            rec.append(int(want[d]))
    return n, bad, ties


@needs_ref
@pytest.mark.parametrize("pen", [False, True])
def test_sample_matches_reference(pen):
    n, bad, ties = _run_sample_cases(pen, 160, 3 + pen)
    print(f"sample(): {n} draws, {ties} with tied candidates (not compared), {bad} differ")
    assert bad == 0
    assert n - ties > n // 3


@needs_ref
@pytest.mark.parametrize("pen", [False, True])
def test_sample_allowed_matches_reference(pen):
    g = np.random.default_rng(7 + pen)
    bad = badfirst = ties = n = tails = skipped = 0
    for c in range(200):
        V = 151936 if c % 50 == 0 else (int(g.integers(1, 600)) if c % 7 == 0 else int(g.integers(64, 20000)))
        l = rand_logits(g, V, 0 if pen else c % 3)
        p, bias = rand_params(g, V, pen, allow_k0=True)
        if p["top_k"][0] == 0 and V < 256:
            p["top_k"] = 20
        den = float(g.choice([1.0, 0.5, 0.05, 0.005, 0.001, 0.0]))
        mask = rand_mask(g, V, den)
        rec = list(rand_recent(g, V))
        s = int(g.integers(1, 2**62)) | 1
        want, calls, first = orc.ref_sample_seq(l, p, np.array(rec, np.int32), s, ndraws=3, append=True, bias=bias, mask=mask)
        us = orc.u_from_seed(s, 3)
        draw = 0
        for d in range(3):
            r = orc.sample(l, p, np.array(rec, np.int32), us[draw], bias, mask)
            if p["temperature"][0] > 0 and r["n_cand"] > 1:
                draw += 1  # the reference draws only when it has at least two candidates
            n += 1
            tails += bool(r["flags"] & 8)
            skipped += bool(r["flags"] & 4)
            if r["flags"] & (1 | 16):
                ties += 1
            else:
                bad += r["token"] != want[d]
                if calls[d] > 0:
                    badfirst += bool(r["flags"] & 2) != bool(first[d])
            if want[d] >= 0:
                rec.append(int(want[d]))
    print(f"sample_allowed(): {n} draws, {ties} tied (not compared), {tails} used the tail, {skipped} skipped it, "
          f"{bad} tokens differ, {badfirst} first-refused flags differ")
    assert bad == 0 and badfirst == 0
    assert tails > 0 and n - ties > n // 3


def test_logprobs_restatement_against_numpy():
    """orc_logprobs (tools/server_chat.h:417-441) against an independent fp64 computation: the
    reference's lambda sits inside Server::chat and cannot be compiled alone, so the restatement
    is pinned by numpy's log-sum-exp and a stable sort (ties: lower id first)."""
    g = np.random.default_rng(5)
    for V, top_n in [(1, 1), (5, 3), (1000, 20), (151936, 20), (4096, 256)]:
        for mode in range(2):
            x = (g.standard_normal(V) * 3).astype(np.float32) if mode == 0 else (0.5 * g.integers(0, 6, V)).astype(np.float32)
            tok = int(g.integers(0, V))
            lse, lp, ids, tlp = orc.logprobs(x, tok, min(top_n, V))
            xd = x.astype(np.float64)
            want_lse = xd.max() + np.log(np.exp(xd - xd.max()).sum())
            assert abs(lse - want_lse) <= 1e-12 * max(1.0, abs(want_lse))
            assert abs(lp - (xd[tok] - want_lse)) <= 1e-11
            order = np.argsort(-xd, kind="stable")[: min(top_n, V)]
            assert np.array_equal(ids, order.astype(np.int32))
            assert np.allclose(tlp, xd[order] - want_lse, rtol=0, atol=1e-11)


@needs_slices
def test_logprobs_pinned_to_the_reference_lines():
    """orc_logprobs against the reference's own lp_entry arithmetic (the lines are cut out of
    tools/server_chat.h at build time and compiled): lse and log probabilities bit for bit (the
    same fp64 operations in the same order), the alternatives' ids wherever the logits that
    decide the order are distinct (equal logits: the reference leaves the order to
    std::partial_sort, the restatement puts the lower id first)."""
    g = np.random.default_rng(7)
    ties = 0
    for V, top_n in [(1, 1), (5, 3), (1000, 20), (151936, 20), (262144, 20), (4096, 256), (3000, 0)]:
        for mode in range(3):
            x = rand_logits(g, V, mode)
            tok = int(g.integers(0, V))
            n = min(top_n, V)
            lse, lp, ids, tlp = orc.logprobs(x, tok, n)
            rlse, rlp, rids, rtlp = orc.ref_lp_entry(x, tok, n)
            assert lse == rlse and lp == rlp
            srt = np.sort(x)[::-1][: n + 1]
            if len(srt) > 1 and np.any(srt[1:] == srt[:-1]):
                ties += 1
                assert np.array_equal(np.sort(x[ids])[::-1], np.sort(x[rids])[::-1])  # the same values either way
            else:
                assert np.array_equal(ids, rids)
            assert np.array_equal(tlp, rtlp)
    assert ties > 0


@needs_slices
def test_softmax_den_pinned_to_the_reference_function():
    """orc_softmax_den against the reference's own softmax_den (zero/engine_drafters.h, cut out at
    build time): bit for bit, including rows that are not a multiple of the 4096-element block."""
    g = np.random.default_rng(8)
    for V in [1, 7, 4095, 4096, 4097, 50000, 151936, 262144]:
        for mode in range(3):
            x = rand_logits(g, V, mode)
            mx = float(x.max())
            assert orc.softmax_den(x, mx) == orc.ref_softmax_den(x, mx)


def dflash_case(g, V, rank, nd, sharp=1.0):
    """Inputs of the DFlash2 selector: logits with a few strong tokens per position (so that the
    path probability is neither 0 nor 1), small codebook entries that reorder the top candidates."""
    logits = (g.standard_normal((nd, V)) * 2.0).astype(np.float32)
    for t in range(nd):
        logits[t, g.integers(0, V, 3)] += np.float32(6.0 * sharp)
    hproj = g.standard_normal((nd, rank)).astype(np.float32)
    pred = synth.f32_to_bf16_bits((g.standard_normal((V, rank)) * 0.3).astype(np.float32))
    succ = synth.f32_to_bf16_bits((g.standard_normal((V, rank)) * 0.3).astype(np.float32))
    return logits, hproj, pred, succ


@pytest.mark.skipif(orc.refslices is None, reason="oracle/_ref/libarcs_refslices.so not built (needs the reference tree)")
def test_dflash_selector_restatement_is_the_reference_loop():
    g = np.random.default_rng(77)
    n_cut = 0
    for V, rank, nd, topk, min_p, sharp in [(3000, 64, 7, 16, 0.3, 1.0), (5000, 256, 5, 16, 0.3, 0.6), (2000, 32, 7, 64, 0.0, 1.0),
                                            (4096, 128, 3, 8, 0.9, 1.0), (40, 16, 4, 64, 0.3, 1.0), (3000, 64, 7, 16, 0.05, 0.3)]:
        for rep in range(4):
            logits, hproj, pred, succ = dflash_case(g, V, rank, nd, sharp)
            if rep == 1:  # ties among the top logits: the first of equals is kept and wins
                logits[:, 5] = logits[:, 9] = logits.max(axis=1) + 1
            tok = int(g.integers(0, V))
            for max_drafts in (nd, 2):
                got, _ = orc.dflash_select(logits, hproj, pred, succ, topk, max_drafts, tok, min_p)
                want = orc.ref_dflash_select(logits, hproj, pred, succ, topk, max_drafts, tok, min_p)
                assert np.array_equal(got, want), (V, rank, nd, topk, min_p, rep)
                n_cut += len(want) < min(nd, max_drafts)
    assert n_cut > 0  # the probability cut was taken somewhere
