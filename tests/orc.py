"""ctypes bindings of the CPU checker: oracle/_build/libarcs_oracle.so (plain-C restatement)
and, when present, oracle/_ref/libarcs_ref.so (the reference's own sampler compiled from its
sources). Test infrastructure: only tests, smoke() and the benchmark's CPU-baseline leg use it."""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORC_SO = os.path.join(ROOT, "oracle", "_build", "libarcs_oracle.so")
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libarcs_ref.so")
REFSLICES_SO = os.path.join(ROOT, "oracle", "_ref", "libarcs_refslices.so")

PARAMS_DTYPE = np.dtype(
    [("temperature", "<f4"), ("top_p", "<f4"), ("min_p", "<f4"), ("presence_penalty", "<f4"),
     ("frequency_penalty", "<f4"), ("repeat_penalty", "<f4"), ("repeat_last_n", "<i4"), ("top_k", "<i4")]
)  # fmt: skip


class Result(C.Structure):
    _fields_ = [("token", C.c_int32), ("n_cand", C.c_int32), ("n_kept", C.c_int32), ("flags", C.c_int32)]


def _build_oracle():
    if not os.path.exists(ORC_SO):
        subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "liboracle"], stdout=subprocess.DEVNULL)
    return C.CDLL(ORC_SO)


orc = _build_oracle()
ref = C.CDLL(REF_SO) if os.path.exists(REF_SO) else None
# fragments of reference files that do not compile here as a whole (oracle/ref_slices.cpp)
refslices = C.CDLL(REFSLICES_SO) if os.path.exists(REFSLICES_SO) else None

orc.orc_softmax_den.restype = C.c_double
orc.orc_softmax_den_exact.restype = C.c_double
orc.orc_argmax.restype = C.c_int32
orc.orc_logprobs.restype = C.c_double
if refslices is not None:
    refslices.ref_softmax_den.restype = C.c_double
    refslices.ref_lp_entry.restype = C.c_double
if ref is not None:
    ref.ref_sample_batch.restype = C.c_double
    ref.ref_hardware_threads.restype = C.c_int


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _bias(bias):
    if not bias:
        return np.zeros(0, np.int32), np.zeros(0, np.float32)
    return _i32([b[0] for b in bias]), _f32([b[1] for b in bias])


def u_from_seed(seed, n=1):
    out = np.zeros(n, np.float64)
    orc.orc_mt64_u01(C.c_uint64(seed), n, _p(out))
    return out


def adjusted(logits, p, hist, bias=None):
    logits, hist = _f32(logits), _i32(hist)
    bi, bv = _bias(bias)
    out = np.empty_like(logits)
    orc.orc_adjusted(_p(logits), len(logits), _p(p), _p(hist), len(hist), _p(bi), _p(bv), len(bi), _p(out))
    return out


def sample(logits, p, hist, u, bias=None, mask=None):
    """Oracle sample / sample_allowed for one row. p: one-element PARAMS_DTYPE array.
    Returns dict(token, n_cand, n_kept, flags, cand_id, cand_pr)."""
    logits, hist = _f32(logits), _i32(hist)
    bi, bv = _bias(bias)
    res = Result()
    k = max(int(p["top_k"][0]) if int(p["top_k"][0]) > 0 else 256, 1)
    cid = np.full(k + 2, -1, np.int32)
    cpr = np.zeros(k + 2, np.float64)
    if mask is None:
        orc.orc_sample(_p(logits), len(logits), _p(p), _p(hist), len(hist), _p(bi), _p(bv), len(bi), C.c_double(u),
                       C.byref(res), _p(cid), _p(cpr))
    else:
        mask = np.ascontiguousarray(mask, dtype=np.uint32)
        orc.orc_sample_allowed(_p(logits), len(logits), _p(p), _p(hist), len(hist), _p(bi), _p(bv), len(bi), _p(mask),
                               C.c_double(u), C.byref(res), _p(cid), _p(cpr))
    n = res.n_cand
    return dict(token=res.token, n_cand=n, n_kept=res.n_kept, flags=res.flags, cand_id=cid[:n].copy(), cand_pr=cpr[:n].copy())


def argmax(row):
    row = _f32(row)
    return orc.orc_argmax(_p(row), len(row))


def verify_greedy(sel, row_off, draft, draft_off):
    sel, row_off, draft, draft_off = _i32(sel), _i32(row_off), _i32(draft), _i32(draft_off)
    slots = len(row_off) - 1
    acc, nxt = np.zeros(slots, np.int32), np.zeros(slots, np.int32)
    orc.orc_verify_greedy(_p(sel), _p(row_off), _p(draft), _p(draft_off), slots, _p(acc), _p(nxt))
    return acc, nxt


def softmax_den(row, mx, exact=False):
    row = _f32(row)
    f = orc.orc_softmax_den_exact if exact else orc.orc_softmax_den
    return f(_p(row), C.c_int64(len(row)), C.c_float(mx))


def logprobs(row, token=-1, top_n=0):
    """lse, logprob of `token` (nan when token < 0), top ids, top log probabilities"""
    row = _f32(row)
    lp = np.full(1, np.nan, np.float64)
    ids, tlp = np.full(max(top_n, 1), -1, np.int32), np.full(max(top_n, 1), np.nan, np.float64)
    lse = orc.orc_logprobs(_p(row), len(row), int(token), int(top_n), _p(lp), _p(ids), _p(tlp))
    return lse, lp[0], ids[:top_n], tlp[:top_n]


def dfa_mask(table, dead, state, byte_off, by, special=None, special_ok=False):
    table = np.ascontiguousarray(table, dtype=np.uint16)
    byte_off = np.ascontiguousarray(byte_off, dtype=np.uint32)
    by = np.ascontiguousarray(by, dtype=np.uint8)
    V = len(byte_off) - 1
    out = np.zeros((V + 31) // 32, np.uint32)
    sp = None if special is None else np.ascontiguousarray(special, dtype=np.uint8)
    orc.orc_dfa_mask(_p(table), table.shape[0], dead, state, _p(byte_off), _p(by), _p(sp), int(special_ok), V, _p(out))
    return out


# ---- the reference's own Sampler (oracle/_ref), when it has been built
def ref_sample_seq(logits, p, hist, seed, ndraws=1, append=False, bias=None, mask=None):
    assert ref is not None
    logits, hist = _f32(logits), _i32(hist)
    bi, bv = _bias(bias)
    out = np.zeros(ndraws, np.int32)
    if mask is None:
        ref.ref_sample_seq(_p(p), C.c_uint64(seed), _p(bi), _p(bv), len(bi), _p(logits), len(logits), _p(hist), len(hist),
                           ndraws, int(append), _p(out))
        return out
    mask = np.ascontiguousarray(mask, dtype=np.uint32)
    calls, first = np.zeros(ndraws, np.int32), np.zeros(ndraws, np.int32)
    ref.ref_sample_allowed_seq(_p(p), C.c_uint64(seed), _p(bi), _p(bv), len(bi), _p(logits), len(logits), _p(hist),
                               len(hist), _p(mask), ndraws, int(append), _p(out), _p(calls), _p(first))
    return out, calls, first


def ref_adjusted(logits, p, hist, bias=None):
    assert ref is not None
    logits, hist = _f32(logits), _i32(hist)
    bi, bv = _bias(bias)
    out = np.empty_like(logits)
    ref.ref_adjusted(_p(p), _p(bi), _p(bv), len(bi), _p(logits), len(logits), _p(hist), len(hist), _p(out))
    return out


def ref_uniform(seed, tot, n):
    assert ref is not None
    out = np.zeros(n, np.float64)
    ref.ref_uniform(C.c_uint64(seed), C.c_double(tot), n, _p(out))
    return out


def ref_softmax_den(row, mx):
    """the reference's own softmax_den (zero/engine_drafters.h), cut out of its file at build time"""
    assert refslices is not None
    row = _f32(row)
    return refslices.ref_softmax_den(_p(row), C.c_int64(len(row)), C.c_float(mx))


def ref_lp_entry(row, token=-1, top_n=0):
    """the arithmetic of the reference's lp_entry lambda (tools/server_chat.h), cut out at build time"""
    assert refslices is not None
    row = _f32(row)
    lp = np.full(1, np.nan, np.float64)
    ids, tlp = np.full(max(top_n, 1), -1, np.int32), np.full(max(top_n, 1), np.nan, np.float64)
    lse = refslices.ref_lp_entry(_p(row), len(row), int(token), int(top_n), _p(lp), _p(ids), _p(tlp))
    return lse, lp[0], ids[:top_n], tlp[:top_n]


# ---- the DFlash2 candidate selector (zero/engine_drafters.h:461-506), one slot
def dflash_select(logits, hproj, pred, succ, topk, max_drafts, tok, min_p):
    """logits [nd, V] float32, hproj [nd, rank] float32, pred / succ [V, rank] uint16 (bf16 bits).
    Returns (drafts int32 array, path probabilities float64 [nd])."""
    logits, hproj = _f32(logits), _f32(hproj)
    pred, succ = np.ascontiguousarray(pred, np.uint16), np.ascontiguousarray(succ, np.uint16)
    nd, V = logits.shape
    out, pp = np.zeros(nd, np.int32), np.full(nd, np.nan)
    n = orc.orc_dflash_select(_p(logits), _p(hproj), _p(pred), _p(succ), V, hproj.shape[1], topk, nd, max_drafts, int(tok),
                              C.c_double(min_p), _p(out), _p(pp))
    return out[:n], pp


def ref_dflash_select(logits, hproj, pred, succ, topk, max_drafts, tok, min_p):
    """The reference's own loop (a fragment of zero/engine_drafters.h compiled by oracle/ref_slices.cpp)."""
    assert refslices is not None
    logits, hproj = _f32(logits), _f32(hproj)
    pred, succ = np.ascontiguousarray(pred, np.uint16), np.ascontiguousarray(succ, np.uint16)
    nd, V = logits.shape
    out = np.zeros(nd, np.int32)
    n = refslices.ref_dflash_select(_p(logits), _p(hproj), _p(pred), _p(succ), V, hproj.shape[1], topk, nd, max_drafts, int(tok),
                                    C.c_double(min_p), _p(out))
    return out[:n]
