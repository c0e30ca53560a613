"""GPU parity on the five measured workloads at their full shapes (seeded synthetic inputs), through
the C ABI against the CPU oracle; plus the host-buffer entry points and the automaton mask."""
import numpy as np
import pytest
import torch

import orc
from arcinfer_b200 import synth

pytestmark = pytest.mark.gpu


def test_config1_single_row():
    from gpuutil import check_rows, run_gpu_sample

    c = synth.config1()
    out = run_gpu_sample(c["logits"], False, c["params"], c["hist"], c["u"])
    check_rows(out, c["logits"], False, c["params"], c["hist"], c["u"])


def test_config2_multi_slot():
    from gpuutil import check_rows, run_gpu_sample

    c = synth.config2()
    out = run_gpu_sample(c["logits"], False, c["params"], c["hist"], c["u"])
    check_rows(out, c["logits"], False, c["params"], c["hist"], c["u"])


def test_config4_constrained_dfa():
    import arcinfer_b200 as ab
    from gpuutil import check_rows, run_gpu_sample

    c = synth.config4()
    V = c["logits"].shape[1]
    states, inv = np.unique(c["states"], return_inverse=True)
    masks = ab.dfa_mask(torch.from_numpy(c["table"].view(np.int16)).cuda(), c["dead"], torch.from_numpy(states.astype(np.int32)).cuda(),
                        torch.from_numpy(c["byte_off"].view(np.int32)).cuda(), torch.from_numpy(c["bytes"]).cuda(), V=V)
    torch.cuda.synchronize()
    masks = masks.cpu().numpy().view(np.uint32)
    for i, s in enumerate(states):  # mask bits bit-exact against the CPU walk
        assert np.array_equal(masks[i], orc.dfa_mask(c["table"], c["dead"], int(s), c["byte_off"], c["bytes"])), s
    dens = [bin(int(w)).count("1") for w in masks[0]]
    assert 0 < sum(dens) < V
    for top_k in (20, 0):  # SamplingParams default 20; 0 means the 40 most likely allowed tokens
        p = c["params"].copy()
        p["top_k"] = top_k
        out = run_gpu_sample(c["logits"], False, p, c["hist"], c["u"], masks=masks, mask_row=inv.astype(np.int32))
        check_rows(out, c["logits"], False, p, c["hist"], c["u"], masks=masks, mask_row=inv)


def test_config5_wide_batch_subset_and_properties():
    import arcinfer_b200 as ab
    from gpuutil import check_rows, run_gpu_sample

    c = synth.config5_rows(B=160)  # one and a bit items per SM; full width and history
    out = run_gpu_sample(c["logits"], True, c["params"], c["hist"], c["u"])
    check_rows(out, c["logits"], True, c["params"], c["hist"], c["u"], rows=range(0, 160, 5))
    # size-independent properties on every row
    assert int(out["status"][0]) == 0
    val, pr, n_c, n_k = out["cand_val"], out["cand_pr"], out["n_cand"], out["n_kept"]
    for b in range(160):
        k = n_c[b]
        assert k == 50 and 1 <= n_k[b] <= k
        assert np.all(np.diff(val[b, :k]) <= 0)                      # sorted
        assert abs(pr[b, :k].sum() - 1.0) < 1e-5                     # a distribution
        assert out["token"][b] in out["cand_id"][b, : n_k[b]]          # drawn from the kept prefix
        assert len(set(out["cand_id"][b, :k].tolist())) == k
    # idempotence: the same launch again gives the same answer (scratch left clean)
    out2 = run_gpu_sample(c["logits"], True, c["params"], c["hist"], c["u"])
    assert np.array_equal(out["token"], out2["token"])


def test_config5_full_shape_rows_spread_over_every_cta():
    """The measured shape itself: 1024 x 262144 bf16, 512-id histories. Every eighth row (128 rows:
    every persistent CTA and each of its three rotating sets of per-item state is hit) is compared
    with the CPU checker; inputs are generated on the device and the checked rows copied back."""
    import arcinfer_b200 as ab

    B, V, H = 1024, 262144, 512
    gen = torch.Generator(device="cuda").manual_seed(synth.BASE_SEED + 55)
    logits = torch.empty(B, V, dtype=torch.bfloat16, device="cuda")
    for r0 in range(0, B, 128):
        logits[r0 : r0 + 128] = (torch.randn(128, V, generator=gen, device="cuda") * 3.0).to(torch.bfloat16)
    hist = torch.randint(0, V, (B, H), generator=gen, device="cuda", dtype=torch.int32)
    hist_off = (torch.arange(B + 1, device="cuda", dtype=torch.int32) * H).contiguous()
    u = torch.rand(B, generator=gen, device="cuda", dtype=torch.float64)
    params = synth.make_params(B, top_k=50, top_p=0.95, repeat_penalty=1.1, repeat_last_n=-1)
    out = ab.sample_batch(logits, ab.capi.params_to_device(params, "cuda"), u, hist_off=hist_off, hist_ids=hist.reshape(-1),
                          max_hist=H, want_cands=True)
    torch.cuda.synchronize()
    assert int(out["status"].item()) == 0
    rows = list(range(0, B, 8)) + [B - 1]
    idx = torch.tensor(rows, device="cuda")
    xf = logits[idx].float().cpu().numpy()
    hh, uu = hist[idx].cpu().numpy(), u[idx].cpu().numpy()
    tok, ncand, cid = out["token"].cpu().numpy(), out["n_cand"].cpu().numpy(), out["cand_id"].cpu().numpy()
    ties = 0
    for i, b in enumerate(rows):
        want = orc.sample(xf[i], params[b : b + 1], hh[i], float(uu[i]))
        ties += (want["flags"] & 1) != 0
        assert tok[b] == want["token"] and ncand[b] == want["n_cand"], (b, tok[b], want["token"])
        assert np.array_equal(cid[b][: want["n_cand"]], want["cand_id"]), b
    assert ties > 0  # bf16 logits: the 50 best of a row live in about as many representable values
    assert int(tok.min()) >= 0 and int(tok.max()) < V


def test_host_buffer_entry_points():
    import arcinfer_b200 as ab

    c = synth.config5_rows(B=40, V=50000, H=64)
    B, V = c["logits"].shape
    ho, hi = synth.csr(c["hist"])
    ctx = ab.capi.HostContext(0, B, V, True, max_hist_total=len(hi))
    tok = np.zeros(B, np.int32)
    ncand = np.zeros(B, np.int32)
    ctx.sample(c["logits"], c["params"], np.ascontiguousarray(c["u"]), tok, hist_off=ho, hist_ids=hi, max_hist=64, n_cand=ncand)
    xf = synth.bf16_bits_to_f32(c["logits"])
    for b in range(B):
        assert tok[b] == orc.sample(xf[b], c["params"][b : b + 1], c["hist"][b], float(c["u"][b]))["token"]
    am = np.zeros(B, np.int32)
    ctx.argmax(c["logits"], am)
    assert np.array_equal(am, np.array([orc.argmax(r) for r in xf], np.int32))
    ctx.close()


def test_host_status_of_the_second_stream_is_reported_by_the_same_call():
    """Row chunks alternate between the context's two streams. A row of the second chunk that asks
    for more candidates than a row can keep must make THIS call return ARCS_ERR_TOPK, and the next
    call must be clean."""
    import arcinfer_b200 as ab

    B, V = 12, 400000  # 1.6 MB rows of fp32: two chunks of six rows
    g = synth.rng(91)
    x = synth.normal_logits(g, B, V, 3.0)
    params = synth.make_params(B, top_k=20)
    params["top_k"][B - 2] = 300
    us = g.random(B)
    ctx = ab.capi.HostContext(0, B, V, False)
    tok = np.zeros(B, np.int32)
    with pytest.raises(ab.ArcsError) as e:
        ctx.sample(x, params, us, tok)
    assert "status 2" in str(e.value)
    params["top_k"][B - 2] = 20
    ctx.sample(x, params, us, tok)
    for b in range(B):
        assert tok[b] == orc.sample(x[b], params[b : b + 1], np.zeros(0, np.int32), float(us[b]))["token"]
    ctx.close()


def test_injected_failure_is_reported(monkeypatch):
    """host-side fault injection: the N-th entry-point call of a process fails before any launch"""
    import subprocess
    import sys

    code = ("import torch, arcinfer_b200 as ab\n"
            "lg = torch.zeros(2, 64, device='cuda')\n"
            "ab.argmax_batch(lg)\n"
            "try:\n    ab.argmax_batch(lg)\n    print('no error')\n"
            "except ab.ArcsError as e:\n    print('caught', 'injected' in str(e))\n"
            "print(ab.argmax_batch(lg)['argmax'].tolist())\n")
    import os

    env = dict(os.environ, ARCS_FAIL_CALL="2")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert "caught True" in r.stdout and "[0, 0]" in r.stdout, r.stdout + r.stderr
