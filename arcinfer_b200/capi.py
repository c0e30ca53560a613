"""ctypes binding of include/arcsample.h. Tensors are torch CUDA tensors; every call enqueues
on torch's current stream of the tensors' device and returns without synchronising."""
import ctypes as C
import os

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libarcsample.so")

KCAP = 256
HEAD = 512
F32, BF16 = 0, 1
FLAG_TIE_TOPK, FLAG_FIRST_REFUSED, FLAG_TAIL_SKIPPED, FLAG_TAIL_USED = 1, 2, 4, 8

from .params import PARAMS_DTYPE, make_params  # noqa: E402,F401


class ArcsError(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C arcinfer_b200/csrc` "
            "(or __graft_entry__.build()); there is no CPU fallback"
        )
    return C.CDLL(LIB_PATH)


lib = _load()


class SampleArgs(C.Structure):
    _fields_ = [
        ("logits", C.c_void_p), ("dtype", C.c_int32), ("B", C.c_int32), ("V", C.c_int32),
        ("row_stride", C.c_int64), ("params", C.c_void_p),
        ("hist_off", C.c_void_p), ("hist_ids", C.c_void_p),
        ("bias_off", C.c_void_p), ("bias_ids", C.c_void_p), ("bias_vals", C.c_void_p),
        ("u", C.c_void_p), ("mask", C.c_void_p), ("mask_row", C.c_void_p), ("mask_stride", C.c_int64),
        ("max_hist", C.c_int32), ("max_bias", C.c_int32), ("id_base", C.c_int32), ("v_global", C.c_int32),
        ("token", C.c_void_p), ("n_cand", C.c_void_p), ("n_kept", C.c_void_p), ("flags", C.c_void_p),
        ("cand_id", C.c_void_p), ("cand_val", C.c_void_p), ("cand_pr", C.c_void_p), ("cand_stride", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("status", C.c_void_p),
        ("head_id", C.c_void_p), ("head_val", C.c_void_p), ("n_head", C.c_void_p),
        ("cand_width", C.c_int32),
    ]  # fmt: skip


class ArgmaxArgs(C.Structure):
    _fields_ = [
        ("logits", C.c_void_p), ("dtype", C.c_int32), ("R", C.c_int32), ("V", C.c_int32),
        ("row_stride", C.c_int64), ("argmax", C.c_void_p), ("max_sumexp", C.c_void_p),
        ("slots", C.c_int32), ("row_off", C.c_void_p), ("draft", C.c_void_p), ("draft_off", C.c_void_p),
        ("accepted", C.c_void_p), ("next", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("status", C.c_void_p),
    ]  # fmt: skip


lib.arcs_last_error.restype = C.c_char_p
lib.arcs_version.restype = C.c_int
lib.arcs_sample_workspace_bytes.restype = C.c_size_t
lib.arcs_sample_workspace_bytes.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32]
lib.arcs_sample_batch.restype = C.c_int
lib.arcs_sample_batch.argtypes = [C.POINTER(SampleArgs), C.c_void_p]


class MergeArgs(C.Structure):
    _fields_ = [
        ("G", C.c_int32), ("B", C.c_int32), ("cand_stride", C.c_int32),
        ("cand_id", C.c_void_p), ("cand_val", C.c_void_p), ("n_cand", C.c_void_p),
        ("params", C.c_void_p), ("u", C.c_void_p), ("bias_off", C.c_void_p), ("bias_vals", C.c_void_p),
        ("v_global", C.c_int32),
        ("token", C.c_void_p), ("n_cand_out", C.c_void_p), ("n_kept", C.c_void_p), ("flags", C.c_void_p),
        ("out_id", C.c_void_p), ("out_val", C.c_void_p), ("out_pr", C.c_void_p), ("out_stride", C.c_int32),
        ("status", C.c_void_p),
        ("cand_width", C.c_int32), ("shard_mz", C.c_void_p), ("mz_stride", C.c_int32), ("mz_out", C.c_void_p),
    ]


lib.arcs_merge_batch.restype = C.c_int
lib.arcs_merge_batch.argtypes = [C.POINTER(MergeArgs), C.c_void_p]
lib.arcs_sample_batch_timed.restype = C.c_int
lib.arcs_sample_batch_timed.argtypes = [C.POINTER(SampleArgs), C.c_void_p, C.POINTER(C.c_float)]
lib.arcs_argmax_workspace_bytes.restype = C.c_size_t
lib.arcs_argmax_workspace_bytes.argtypes = [C.c_int32, C.c_int32]
lib.arcs_argmax_batch.restype = C.c_int
lib.arcs_argmax_batch.argtypes = [C.POINTER(ArgmaxArgs), C.c_void_p]
lib.arcs_argmax_batch_static.restype = C.c_int
lib.arcs_argmax_batch_static.argtypes = [C.POINTER(ArgmaxArgs), C.c_void_p]
lib.arcs_argmax_static_scratch_bytes.restype = C.c_size_t
lib.arcs_accept_batch.restype = C.c_int
lib.arcs_accept_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]
lib.arcs_dfa_mask.restype = C.c_int
lib.arcs_dfa_mask.argtypes = [
    C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
    C.c_int32, C.c_int32, C.c_void_p, C.c_int64, C.c_void_p,
]  # fmt: skip


def _check(rc, what):
    if rc != 0:
        raise ArcsError(f"{what}: status {rc}: {lib.arcs_last_error().decode()}")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(device):
    return torch.cuda.current_stream(device).cuda_stream


def _dtype_code(t):
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise ArcsError(f"logits must be float32 or bfloat16, not {t.dtype}")


def params_to_device(p, device):
    return torch.from_numpy(np.ascontiguousarray(p).view(np.uint8).copy()).to(device)


_workspaces = {}


def _workspace(kind, device, nbytes, shape=None):
    """One zero-initialised scratch buffer per (kind, device), grown on demand. The kernels leave
    their counters zeroed again, but where the counters lie depends on the call's shape: the buffer
    is cleared when it is (re)allocated and when a call of another shape takes it over."""
    key = (kind, str(device))
    w, last = _workspaces.get(key, (None, None))
    if w is None or w.numel() < nbytes:
        w = torch.zeros(max(nbytes, 1024), dtype=torch.uint8, device=device)
    elif shape != last:
        w.zero_()
    _workspaces[key] = (w, shape)
    return w


def reset_workspaces():
    """Zero every cached scratch buffer (needed after a launch that reported a device status)."""
    for w, _ in _workspaces.values():
        w.zero_()


def sample_batch(logits, params, u, hist_off=None, hist_ids=None, bias_off=None, bias_ids=None, bias_vals=None,
                 mask=None, mask_row=None, max_hist=0, max_bias=0, id_base=0, v_global=0, V=None,
                 want_cands=False, want_head=False, status=None, records=None):
    """arcs_sample_batch on device tensors. logits: [B, >=V] float32/bfloat16 (row stride =
    logits.stride(0)); params: uint8 tensor holding B arcs_row_params; u: float64 [B].
    records: an int32 tensor [B, 2k + 2] that receives each row's candidates as a packed record
    (k ids, k values as bit patterns; the last two words are left to the caller), see pack_width."""
    assert logits.is_cuda and logits.dim() == 2 and logits.stride(1) == 1
    dev = logits.device
    B = logits.shape[0]
    V = logits.shape[1] if V is None else V
    out = {
        "token": torch.empty(B, dtype=torch.int32, device=dev),
        "n_cand": torch.empty(B, dtype=torch.int32, device=dev),
        "n_kept": torch.empty(B, dtype=torch.int32, device=dev),
        "flags": torch.empty(B, dtype=torch.int32, device=dev),
    }
    if want_cands:
        out["cand_id"] = torch.empty(B, KCAP, dtype=torch.int32, device=dev)
        out["cand_val"] = torch.empty(B, KCAP, dtype=torch.float32, device=dev)
        out["cand_pr"] = torch.empty(B, KCAP, dtype=torch.float32, device=dev)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=dev)
    out["status"] = status
    masked = mask is not None
    max_list = (max_hist if hist_off is not None else 0) + (max_bias if bias_off is not None else 0)
    nbytes = lib.arcs_sample_workspace_bytes(B, V, int(masked), max_list)
    ws = _workspace("sample", dev, nbytes)
    a = SampleArgs()
    a.logits, a.dtype, a.B, a.V, a.row_stride = logits.data_ptr(), _dtype_code(logits), B, V, logits.stride(0)
    a.params = params.data_ptr()
    a.hist_off, a.hist_ids = _ptr(hist_off), _ptr(hist_ids)
    a.bias_off, a.bias_ids, a.bias_vals = _ptr(bias_off), _ptr(bias_ids), _ptr(bias_vals)
    a.u = u.data_ptr()
    a.mask, a.mask_row = _ptr(mask), _ptr(mask_row)
    a.mask_stride = (mask.stride(0) if mask.shape[0] > 1 else mask.shape[1]) if masked else 0
    a.max_hist, a.max_bias, a.id_base, a.v_global = max_hist, max_bias, id_base, v_global
    a.token, a.n_cand, a.n_kept, a.flags = (out[k].data_ptr() for k in ("token", "n_cand", "n_kept", "flags"))
    if want_cands:
        a.cand_id, a.cand_val, a.cand_pr = out["cand_id"].data_ptr(), out["cand_val"].data_ptr(), out["cand_pr"].data_ptr()
    a.cand_stride = KCAP
    if records is not None:
        _point_at_records(a, records)
    if want_head:  # (constrained rows only) the 512 most likely tokens in the order the reference calls its predicate
        out["head_id"] = torch.empty(B, HEAD, dtype=torch.int32, device=dev)
        out["head_val"] = torch.empty(B, HEAD, dtype=torch.float32, device=dev)
        out["n_head"] = torch.empty(B, dtype=torch.int32, device=dev)
        a.head_id, a.head_val, a.n_head = out["head_id"].data_ptr(), out["head_val"].data_ptr(), out["n_head"].data_ptr()
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.status = status.data_ptr()
    _check(lib.arcs_sample_batch(C.byref(a), _stream(dev)), "arcs_sample_batch")
    return out


def accept_batch(token, row_off, draft, draft_off):
    """arcs_accept_batch: the acceptance walk over chosen tokens (int32 device tensors): returns
    (accepted [slots], next [slots])."""
    slots = row_off.numel() - 1
    dev = token.device
    acc = torch.empty(slots, dtype=torch.int32, device=dev)
    nxt = torch.empty(slots, dtype=torch.int32, device=dev)
    _check(lib.arcs_accept_batch(token.data_ptr(), row_off.data_ptr(), draft.data_ptr(), draft_off.data_ptr(), slots, acc.data_ptr(), nxt.data_ptr(),
                                 _stream(dev)), "arcs_accept_batch")
    return acc, nxt


def verification_histories(histories, drafts):
    """The CSR history of every verification row when drafts are verified under sampling: row i of
    a slot sees the slot's history followed by its first i drafts (tools/server_chat.h:593: an
    accepted draft is appended to `gen` before the next row is sampled). histories / drafts: one
    int32 array per slot; a slot has len(drafts) + 1 rows. Returns (hist_off, hist_ids, row_off,
    draft_off, draft_ids) as numpy arrays."""
    offs, ids, row_off, d_off = [0], [], [0], [0]
    for h, d in zip(histories, drafts):
        h, d = np.asarray(h, np.int32), np.asarray(d, np.int32)
        for i in range(len(d) + 1):
            ids.append(h)
            ids.append(d[:i])
            offs.append(offs[-1] + len(h) + i)
        row_off.append(row_off[-1] + len(d) + 1)
        d_off.append(d_off[-1] + len(d))
    cat = np.concatenate(ids).astype(np.int32) if ids else np.zeros(0, np.int32)
    dr = np.concatenate([np.asarray(d, np.int32) for d in drafts]) if drafts else np.zeros(0, np.int32)
    return (np.asarray(offs, np.int32), cat, np.asarray(row_off, np.int32), np.asarray(d_off, np.int32), dr.astype(np.int32))


def pack_width(records):
    """k of a record tensor [.., 2k + 2]: k ids, k values, (max, sum exp)."""
    assert records.dtype == torch.int32 and records.shape[-1] % 2 == 0 and records.is_contiguous()
    return (records.shape[-1] - 2) // 2


def _point_at_records(a, records):
    k = pack_width(records)
    a.cand_id, a.cand_val, a.cand_pr = records.data_ptr(), records.data_ptr() + 4 * k, None
    a.cand_stride, a.cand_width = records.shape[-1], k


def argmax_batch(logits, V=None, want_lse=False, row_off=None, draft=None, draft_off=None, status=None, static_scratch=False):
    """arcs_argmax_batch: first maximum per row, optional (max, sumexp), optional greedy
    acceptance for rows grouped into slots (row_off / draft / draft_off int32 device tensors)."""
    assert logits.is_cuda and logits.dim() == 2 and logits.stride(1) == 1
    dev = logits.device
    R = logits.shape[0]
    V = logits.shape[1] if V is None else V
    out = {"argmax": torch.empty(R, dtype=torch.int32, device=dev)}
    if want_lse:
        out["max_sumexp"] = torch.empty(R, 2, dtype=torch.float32, device=dev)
    slots = 0 if row_off is None else row_off.numel() - 1
    if slots:
        out["accepted"] = torch.empty(slots, dtype=torch.int32, device=dev)
        out["next"] = torch.empty(slots, dtype=torch.int32, device=dev)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=dev)
    out["status"] = status
    ws = None if static_scratch else _workspace("argmax", dev, lib.arcs_argmax_workspace_bytes(R, V), (R, V))
    a = ArgmaxArgs()
    a.logits, a.dtype, a.R, a.V, a.row_stride = logits.data_ptr(), _dtype_code(logits), R, V, logits.stride(0)
    a.argmax, a.max_sumexp = out["argmax"].data_ptr(), _ptr(out.get("max_sumexp"))
    a.slots, a.row_off, a.draft, a.draft_off = slots, _ptr(row_off), _ptr(draft), _ptr(draft_off)
    a.accepted, a.next = _ptr(out.get("accepted")), _ptr(out.get("next"))
    a.status = status.data_ptr()
    if static_scratch:  # the entry point that allocates nothing: scratch is a fixed array inside the library
        _check(lib.arcs_argmax_batch_static(C.byref(a), _stream(dev)), "arcs_argmax_batch_static")
        return out
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    _check(lib.arcs_argmax_batch(C.byref(a), _stream(dev)), "arcs_argmax_batch")
    return out


def dfa_mask(table, dead, states, byte_off, bytes_, special=None, special_ok=False, V=None, out_stride=None, out=None):
    """arcs_dfa_mask: table [S,256] uint16-as-int16 tensor, states int32 [n], byte_off
    uint32-as-int32 [V+1], bytes_ uint8. Returns int32 [n, out_stride] packed bits (out_stride
    defaults to ceil(V/32); words past that are left zero). out: a tensor of that shape to write
    into instead of a new one (its words past ceil(V/32) are left as they are)."""
    dev = table.device
    V = byte_off.numel() - 1 if V is None else V
    W = (V + 31) // 32 if out_stride is None else out_stride
    if out is None:
        out = torch.zeros(states.numel(), W, dtype=torch.int32, device=dev)
    assert out.shape == (states.numel(), W) and out.dtype == torch.int32 and out.is_contiguous()
    _check(
        lib.arcs_dfa_mask(table.data_ptr(), table.shape[0], dead, states.data_ptr(), states.numel(), byte_off.data_ptr(),
                          bytes_.data_ptr(), _ptr(special), int(special_ok), V, out.data_ptr(), W, _stream(dev)),
        "arcs_dfa_mask",
    )
    return out


class AdjustedArgs(C.Structure):
    _fields_ = [
        ("logits", C.c_void_p), ("dtype", C.c_int32), ("B", C.c_int32), ("V", C.c_int32), ("row_stride", C.c_int64),
        ("params", C.c_void_p), ("hist_off", C.c_void_p), ("hist_ids", C.c_void_p),
        ("bias_off", C.c_void_p), ("bias_ids", C.c_void_p), ("bias_vals", C.c_void_p),
        ("out", C.c_void_p), ("out_stride", C.c_int64),
    ]  # fmt: skip


lib.arcs_adjusted_batch.restype = C.c_int
lib.arcs_adjusted_batch.argtypes = [C.POINTER(AdjustedArgs), C.c_void_p]


def adjusted_batch(logits, params, hist_off=None, hist_ids=None, bias_off=None, bias_ids=None, bias_vals=None, V=None):
    """arcs_adjusted_batch: the penalised logits of whole rows (Sampler::adjusted) as float32 [B, V]."""
    dev = logits.device
    B = logits.shape[0]
    V = logits.shape[1] if V is None else V
    out = torch.empty(B, V, dtype=torch.float32, device=dev)
    a = AdjustedArgs()
    a.logits, a.dtype, a.B, a.V, a.row_stride = logits.data_ptr(), _dtype_code(logits), B, V, logits.stride(0)
    a.params = params.data_ptr()
    a.hist_off, a.hist_ids = _ptr(hist_off), _ptr(hist_ids)
    a.bias_off, a.bias_ids, a.bias_vals = _ptr(bias_off), _ptr(bias_ids), _ptr(bias_vals)
    a.out, a.out_stride = out.data_ptr(), V
    _check(lib.arcs_adjusted_batch(C.byref(a), _stream(dev)), "arcs_adjusted_batch")
    return out


class LogprobArgs(C.Structure):
    _fields_ = [
        ("logits", C.c_void_p), ("dtype", C.c_int32), ("B", C.c_int32), ("V", C.c_int32),
        ("row_stride", C.c_int64), ("token", C.c_void_p), ("top_n", C.c_int32), ("top_stride", C.c_int32),
        ("logprob", C.c_void_p), ("lse", C.c_void_p), ("top_id", C.c_void_p), ("top_logprob", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("status", C.c_void_p),
    ]  # fmt: skip


lib.arcs_logprobs_workspace_bytes.restype = C.c_size_t
lib.arcs_logprobs_workspace_bytes.argtypes = [C.c_int32, C.c_int32, C.c_int32]
lib.arcs_logprobs_batch.restype = C.c_int
lib.arcs_logprobs_batch.argtypes = [C.POINTER(LogprobArgs), C.c_void_p]


def logprobs_batch(logits, token=None, top_n=0, V=None, status=None):
    """arcs_logprobs_batch: logits [B, >=V] fp32 / bf16 on the device, token int32 [B] or None.
    Returns a dict: lse [B] float64, logprob [B] float64 (when token is given), top_id [B, top_n]
    int32 and top_logprob [B, top_n] float64 (when top_n > 0), status."""
    dev = logits.device
    B = logits.shape[0]
    V = logits.shape[1] if V is None else V
    out = {"lse": torch.empty(B, dtype=torch.float64, device=dev)}
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=dev)
    out["status"] = status
    if token is not None:
        out["logprob"] = torch.empty(B, dtype=torch.float64, device=dev)
    if top_n > 0:
        out["top_id"] = torch.full((B, top_n), -1, dtype=torch.int32, device=dev)
        out["top_logprob"] = torch.full((B, top_n), float("nan"), dtype=torch.float64, device=dev)
    a = LogprobArgs()
    a.logits, a.dtype, a.B, a.V, a.row_stride = logits.data_ptr(), _dtype_code(logits), B, V, logits.stride(0)
    a.token, a.top_n, a.top_stride = _ptr(token), top_n, top_n
    a.logprob, a.lse = _ptr(out.get("logprob")), out["lse"].data_ptr()
    a.top_id, a.top_logprob = _ptr(out.get("top_id")), _ptr(out.get("top_logprob"))
    ws = _workspace("logprobs", dev, lib.arcs_logprobs_workspace_bytes(B, V, top_n), (B, V, top_n))
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.status = status.data_ptr()
    _check(lib.arcs_logprobs_batch(C.byref(a), _stream(dev)), "arcs_logprobs_batch")
    return out


class DflashArgs(C.Structure):
    _fields_ = [
        ("logits", C.c_void_p), ("dtype", C.c_int32), ("slots", C.c_int32), ("nd", C.c_int32), ("V", C.c_int32),
        ("row_stride", C.c_int64), ("hproj", C.c_void_p), ("pred", C.c_void_p), ("succ", C.c_void_p),
        ("rank", C.c_int32), ("topk", C.c_int32), ("max_drafts", C.c_int32), ("tok", C.c_void_p), ("min_p", C.c_double),
        ("n_out", C.c_void_p), ("out_tokens", C.c_void_p), ("out_stride", C.c_int32), ("path_p", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("status", C.c_void_p),
    ]  # fmt: skip


lib.arcs_dflash_workspace_bytes.restype = C.c_size_t
lib.arcs_dflash_workspace_bytes.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32]
lib.arcs_dflash_select.restype = C.c_int
lib.arcs_dflash_select.argtypes = [C.POINTER(DflashArgs), C.c_void_p]


def dflash_select(logits, hproj, pred, succ, tok, topk=16, max_drafts=7, min_p=0.3, status=None):
    """arcs_dflash_select: logits [slots, nd, >=V] fp32 / bf16, hproj [slots, nd, rank] float32,
    pred / succ [V, rank] bf16 codebooks (int16 tensors holding the bit patterns), tok int32
    [slots]. Returns n_out [slots], tokens [slots, nd] (-1 past n_out), path_p [slots, nd], status."""
    dev = logits.device
    slots, nd = logits.shape[0], logits.shape[1]
    V, rank = pred.shape
    assert logits.stride(2) == 1 and (slots == 1 or logits.stride(0) == nd * logits.stride(1)) and hproj.is_contiguous() and pred.is_contiguous() and succ.is_contiguous()
    out = {"n_out": torch.zeros(slots, dtype=torch.int32, device=dev), "tokens": torch.full((slots, nd), -1, dtype=torch.int32, device=dev),
           "path_p": torch.full((slots, nd), float("nan"), dtype=torch.float64, device=dev)}
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=dev)
    out["status"] = status
    a = DflashArgs()
    a.logits, a.dtype, a.slots, a.nd, a.V, a.row_stride = logits.data_ptr(), _dtype_code(logits), slots, nd, V, logits.stride(1)
    a.hproj, a.pred, a.succ, a.rank, a.topk, a.max_drafts = hproj.data_ptr(), pred.data_ptr(), succ.data_ptr(), rank, topk, max_drafts
    a.tok, a.min_p = tok.data_ptr(), min_p
    a.n_out, a.out_tokens, a.out_stride, a.path_p = out["n_out"].data_ptr(), out["tokens"].data_ptr(), nd, out["path_p"].data_ptr()
    ws = _workspace("dflash", dev, lib.arcs_dflash_workspace_bytes(slots, nd, V, topk), (slots, nd, V, topk))
    a.workspace, a.workspace_bytes, a.status = ws.data_ptr(), ws.numel(), status.data_ptr()
    _check(lib.arcs_dflash_select(C.byref(a), _stream(dev)), "arcs_dflash_select")
    return out


# ---------------------------------------------------------------- host-buffer entry points
lib.arcs_host_create.restype = C.c_int
lib.arcs_host_create.argtypes = [C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_int64]
lib.arcs_host_destroy.restype = None
lib.arcs_host_destroy.argtypes = [C.c_void_p]
lib.arcs_sample_batch_host.restype = C.c_int
lib.arcs_sample_batch_host.argtypes = [C.c_void_p, C.POINTER(SampleArgs)]
lib.arcs_argmax_batch_host.restype = C.c_int
lib.arcs_argmax_batch_host.argtypes = [C.c_void_p, C.POINTER(ArgmaxArgs)]
lib.arcs_host_last_status.restype = C.c_int
lib.arcs_host_last_status.argtypes = [C.c_void_p]


def _hp(a):
    """host pointer of a numpy array or a (pinned) CPU torch tensor"""
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        assert a.flags["C_CONTIGUOUS"]
        return a.ctypes.data
    assert not a.is_cuda and a.is_contiguous()
    return a.data_ptr()


class HostContext:
    """arcs_host_ctx: the call a host application makes when its logits live in host memory.
    Inputs and outputs are numpy arrays or CPU torch tensors (pinned memory lets the copies of
    one chunk of rows overlap the kernel of the previous chunk)."""

    def __init__(self, device, max_B, max_V, bf16, max_hist_total=0, max_bias_total=0, max_mask_words=0):
        self._h = C.c_void_p()
        _check(lib.arcs_host_create(C.byref(self._h), device, max_B, max_V, BF16 if bf16 else F32, max_hist_total,
                                    max_bias_total, max_mask_words), "arcs_host_create")
        self.bf16 = bf16

    def close(self):
        if self._h:
            lib.arcs_host_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        self.close()

    def sample(self, logits, params, u, token, V=None, hist_off=None, hist_ids=None, bias_off=None, bias_ids=None,
               bias_vals=None, mask=None, mask_row=None, max_hist=0, max_bias=0, n_cand=None, n_kept=None, flags=None,
               cand_id=None, cand_val=None, cand_pr=None):
        B = logits.shape[0]
        a = SampleArgs()
        a.logits, a.dtype, a.B = _hp(logits), BF16 if self.bf16 else F32, B
        a.V = logits.shape[1] if V is None else V
        a.row_stride = logits.shape[1]
        a.params, a.u, a.token = _hp(params), _hp(u), _hp(token)
        a.hist_off, a.hist_ids, a.bias_off, a.bias_ids, a.bias_vals = _hp(hist_off), _hp(hist_ids), _hp(bias_off), _hp(bias_ids), _hp(bias_vals)
        a.mask, a.mask_row = _hp(mask), _hp(mask_row)
        a.mask_stride = mask.shape[1] if mask is not None else 0
        a.max_hist, a.max_bias = max_hist, max_bias
        a.n_cand, a.n_kept, a.flags = _hp(n_cand), _hp(n_kept), _hp(flags)
        a.cand_id, a.cand_val, a.cand_pr, a.cand_stride = _hp(cand_id), _hp(cand_val), _hp(cand_pr), KCAP
        _check(lib.arcs_sample_batch_host(self._h, C.byref(a)), "arcs_sample_batch_host")

    def argmax(self, logits, argmax, V=None, max_sumexp=None, row_off=None, draft=None, draft_off=None, accepted=None, next_=None):
        a = ArgmaxArgs()
        a.logits, a.dtype, a.R = _hp(logits), BF16 if self.bf16 else F32, logits.shape[0]
        a.V = logits.shape[1] if V is None else V
        a.row_stride = logits.shape[1]
        a.argmax, a.max_sumexp = _hp(argmax), _hp(max_sumexp)
        a.slots = 0 if row_off is None else len(row_off) - 1
        a.row_off, a.draft, a.draft_off, a.accepted, a.next = _hp(row_off), _hp(draft), _hp(draft_off), _hp(accepted), _hp(next_)
        _check(lib.arcs_argmax_batch_host(self._h, C.byref(a)), "arcs_argmax_batch_host")


def merge_batch(cand_id, cand_val, n_cand, params, u, v_global, bias_off=None, bias_vals=None, want_cands=False, status=None):
    """arcs_merge_batch: the global choice from the shards' gathered candidate lists.
    cand_id / cand_val: [G, B, stride] int32 / float32; n_cand: [G, B] int32 (device tensors)."""
    G, B, stride = cand_id.shape
    return _merge(G, B, stride, cand_id.data_ptr(), cand_val.data_ptr(), n_cand.data_ptr(), 0, None, cand_id.device, params, u, v_global,
                  bias_off, bias_vals, want_cands, status)


def merge_records(records, params, u, v_global, bias_off=None, bias_vals=None, want_cands=False, want_mz=False, status=None):
    """arcs_merge_batch on gathered packed records [G, B, 2k + 2] (int32), read in place: k ids,
    k values, (max, sum exp) of every shard and row. want_mz: also combine the pairs into out["mz"]."""
    G, B, stride = records.shape
    k = pack_width(records)
    return _merge(G, B, stride, records.data_ptr(), records.data_ptr() + 4 * k, None, k, records.data_ptr() + 8 * k if want_mz else None,
                  records.device, params, u, v_global, bias_off, bias_vals, want_cands, status)


def _merge(G, B, stride, p_id, p_val, p_n, width, p_mz, dev, params, u, v_global, bias_off, bias_vals, want_cands, status):
    out = {k: torch.empty(B, dtype=torch.int32, device=dev) for k in ("token", "n_cand", "n_kept", "flags")}
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=dev)
    out["status"] = status
    a = MergeArgs()
    a.G, a.B, a.cand_stride = G, B, stride
    a.cand_id, a.cand_val, a.n_cand = p_id, p_val, p_n
    a.cand_width = width
    if p_mz is not None:
        out["mz"] = torch.empty(B, 2, dtype=torch.float32, device=dev)
        a.shard_mz, a.mz_stride, a.mz_out = p_mz, stride, out["mz"].data_ptr()
    a.params, a.u = params.data_ptr(), u.data_ptr()
    a.bias_off, a.bias_vals = _ptr(bias_off), _ptr(bias_vals)
    a.v_global = v_global
    a.token, a.n_cand_out, a.n_kept, a.flags = (out[k].data_ptr() for k in ("token", "n_cand", "n_kept", "flags"))
    if want_cands:
        out["cand_id"] = torch.empty(B, KCAP, dtype=torch.int32, device=dev)
        out["cand_val"] = torch.empty(B, KCAP, dtype=torch.float32, device=dev)
        out["cand_pr"] = torch.empty(B, KCAP, dtype=torch.float32, device=dev)
        a.out_id, a.out_val, a.out_pr = out["cand_id"].data_ptr(), out["cand_val"].data_ptr(), out["cand_pr"].data_ptr()
    a.out_stride = KCAP
    a.status = status.data_ptr()
    _check(lib.arcs_merge_batch(C.byref(a), _stream(dev)), "arcs_merge_batch")
    return out


class SamplePlan:
    """A prepared arcs_sample_batch call: the argument block and the output tensors are built
    once, launch() only enqueues the kernel (what a serving loop does every step)."""

    def __init__(self, logits, params, u, hist_off=None, hist_ids=None, max_hist=0, mask=None, mask_row=None, V=None,
                 id_base=0, v_global=0, want_cands=False, records=None):
        dev = logits.device
        B = logits.shape[0]
        V = logits.shape[1] if V is None else V
        self.device = dev
        self.keep = (logits, params, u, hist_off, hist_ids, mask, mask_row)
        self.out = {k: torch.empty(B, dtype=torch.int32, device=dev) for k in ("token", "n_cand", "n_kept", "flags")}
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.out["status"] = self.status
        masked = mask is not None
        max_list = max_hist if hist_off is not None else 0
        self.ws = _workspace("sample", dev, lib.arcs_sample_workspace_bytes(B, V, int(masked), max_list))
        a = SampleArgs()
        a.logits, a.dtype, a.B, a.V, a.row_stride = logits.data_ptr(), _dtype_code(logits), B, V, logits.stride(0)
        a.params, a.u = params.data_ptr(), u.data_ptr()
        a.hist_off, a.hist_ids, a.max_hist = _ptr(hist_off), _ptr(hist_ids), max_hist
        a.mask, a.mask_row = _ptr(mask), _ptr(mask_row)
        a.mask_stride = (mask.stride(0) if mask.shape[0] > 1 else mask.shape[1]) if masked else 0
        a.id_base, a.v_global = id_base, v_global
        a.token, a.n_cand, a.n_kept, a.flags = (self.out[k].data_ptr() for k in ("token", "n_cand", "n_kept", "flags"))
        if want_cands:
            for k, dt in (("cand_id", torch.int32), ("cand_val", torch.float32), ("cand_pr", torch.float32)):
                self.out[k] = torch.empty(B, KCAP, dtype=dt, device=dev)
            a.cand_id, a.cand_val, a.cand_pr = (self.out[k].data_ptr() for k in ("cand_id", "cand_val", "cand_pr"))
        a.cand_stride = KCAP
        if records is not None:  # candidates straight into packed records (see sample_batch)
            _point_at_records(a, records)
            self.keep += (records,)
        a.workspace, a.workspace_bytes, a.status = self.ws.data_ptr(), self.ws.numel(), self.status.data_ptr()
        self.args = a

    def launch(self, stream=None):
        s = _stream(self.device) if stream is None else stream
        _check(lib.arcs_sample_batch(C.byref(self.args), s), "arcs_sample_batch")
        return self.out

    def launch_timed(self, stream=None):
        """One call with CUDA events between its kernels: (stream, finish) milliseconds."""
        s = _stream(self.device) if stream is None else stream
        ms = (C.c_float * 2)()
        _check(lib.arcs_sample_batch_timed(C.byref(self.args), s, ms), "arcs_sample_batch_timed")
        return tuple(ms)
