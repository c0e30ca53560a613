"""Helpers shared by the GPU parity tests: run a batch through the C ABI and through the oracle."""
import numpy as np
import torch

import arcinfer_b200 as ab
import orc
from arcinfer_b200 import synth


def to_dev_logits(x, bf16, stride=None, offset=0):
    """x: [B,V] fp32 array, or uint16 bf16 bit patterns when bf16. stride (elements) > V and a
    non-zero element offset give rows that are not 16-byte aligned."""
    B, V = x.shape
    stride = V if stride is None else stride
    if bf16:
        buf = torch.zeros(B * stride + offset + 8, dtype=torch.int16, device="cuda")
        view = buf[offset : offset + B * stride].view(B, stride)
        view[:, :V] = torch.from_numpy(x.view(np.int16)).cuda()
        return view.view(torch.bfloat16)[:, :V] if stride == V else view.view(torch.bfloat16), V
    buf = torch.zeros(B * stride + offset + 8, dtype=torch.float32, device="cuda")
    view = buf[offset : offset + B * stride].view(B, stride)
    view[:, :V] = torch.from_numpy(x).cuda()
    return view, V


def widen(x, bf16):
    return synth.bf16_bits_to_f32(x) if bf16 else x


def run_gpu_sample(x, bf16, params, hists, us, biases=None, masks=None, mask_row=None, stride=None, offset=0, want_cands=True):
    B = x.shape[0]
    lg, V = to_dev_logits(x, bf16, stride, offset)
    p = ab.capi.params_to_device(params, "cuda")
    u = torch.from_numpy(np.ascontiguousarray(us, dtype=np.float64)).cuda()
    kw = {}
    if hists is not None:
        ho, hi = synth.csr(hists)
        kw.update(hist_off=torch.from_numpy(ho).cuda(), hist_ids=torch.from_numpy(hi).cuda() if len(hi) else torch.zeros(1, dtype=torch.int32, device="cuda"),
                  max_hist=int(max(len(h) for h in hists)))
    if biases is not None:
        bo, bi = synth.csr([[b[0] for b in bl] for bl in biases])
        bv = np.array([b[1] for bl in biases for b in bl], np.float32)
        kw.update(bias_off=torch.from_numpy(bo).cuda(),
                  bias_ids=torch.from_numpy(bi).cuda() if len(bi) else torch.zeros(1, dtype=torch.int32, device="cuda"),
                  bias_vals=torch.from_numpy(bv).cuda() if len(bv) else torch.zeros(1, dtype=torch.float32, device="cuda"),
                  max_bias=int(max(len(b) for b in biases)))
    if masks is not None:
        kw.update(mask=torch.from_numpy(np.ascontiguousarray(masks).view(np.int32)).cuda())
        if mask_row is not None:
            kw.update(mask_row=torch.from_numpy(np.asarray(mask_row, np.int32)).cuda())
    out = ab.sample_batch(lg, p, u, V=V, want_cands=want_cands, **kw)
    torch.cuda.synchronize()
    return {k: v.cpu().numpy() for k, v in out.items()}


def check_rows(out, x, bf16, params, hists, us, biases=None, masks=None, mask_row=None, rows=None, pr_rtol=1e-6, tag=""):
    """Bit-exact ids / counts / adjusted logits, probabilities within pr_rtol relative."""
    B = x.shape[0]
    assert int(out["status"][0]) == 0
    xf = widen(x, bf16)
    for b in (range(B) if rows is None else rows):
        m = None if masks is None else masks[b if mask_row is None else mask_row[b]]
        r = orc.sample(xf[b], params[b : b + 1], hists[b] if hists is not None else np.zeros(0, np.int32), float(us[b]),
                       biases[b] if biases is not None else None, m)
        ctx = f"{tag} V={x.shape[1]} row {b} params {params[b]} got token {out['token'][b]} want {r['token']} n_cand {out['n_cand'][b]}/{r['n_cand']}"
        assert out["token"][b] == r["token"], ctx
        assert out["n_cand"][b] == r["n_cand"], ctx
        assert out["n_kept"][b] == r["n_kept"], ctx
        n = r["n_cand"]
        if "cand_id" in out:
            assert np.array_equal(out["cand_id"][b][:n], r["cand_id"]), ctx
            assert np.all(out["cand_id"][b][n:] == -1), ctx
            adj = orc.adjusted(xf[b], params[b : b + 1], hists[b] if hists is not None else np.zeros(0, np.int32),
                               biases[b] if biases is not None else None)
            assert np.array_equal(out["cand_val"][b][:n].view(np.uint32), adj[r["cand_id"]].view(np.uint32)), ctx
            if n:
                np.testing.assert_allclose(out["cand_pr"][b][:n], r["cand_pr"], rtol=pr_rtol, atol=1e-30, err_msg=ctx)
        gflags, oflags = int(out["flags"][b]), r["flags"]
        assert (gflags & 0xE) == (oflags & 0xE), (ctx, gflags, oflags)
