"""Vocabulary-sharded sampling: G shards of the columns, each through arcs_sample_batch under global
ids, their candidate lists gathered and merged by arcs_merge_batch, must give exactly what the
oracle gives for the whole rows. One GPU plays all the shards here (the all-gather is a list copy);
with two or more GPUs the same helper runs over NCCL (second test, skipped on one GPU)."""
import os
import subprocess
import sys

import numpy as np
import pytest

from arcinfer_b200 import shard, synth
from cases import rand_logits, rand_params, rand_recent

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lists(hists, biases, lo, hi):
    import torch

    ho, hi_ = synth.csr(hists)
    bo, bi = synth.csr([[b[0] for b in bl] for bl in biases])
    bv = np.array([b[1] for bl in biases for b in bl], np.float32)
    z = lambda a, dt: torch.from_numpy(a).cuda() if len(a) else torch.zeros(1, dtype=dt, device="cuda")
    return dict(hist_off=torch.from_numpy(ho).cuda(), hist_ids=z(hi_, torch.int32), max_hist=int(max(len(h) for h in hists)),
                bias_off=torch.from_numpy(bo).cuda(), bias_ids=z(bi, torch.int32), bias_vals=z(bv, torch.float32),
                max_bias=int(max(len(b) for b in biases)))


@pytest.mark.parametrize("bf16", [False, True])
def test_shards_on_one_gpu_match_the_oracle(bf16):
    import torch

    import arcinfer_b200 as ab
    from gpuutil import check_rows, to_dev_logits

    g = np.random.default_rng(500 + bf16)
    for V, B, G in [(5000, 6, 2), (40000, 5, 4), (151936, 3, 8), (262144, 2, 3)]:
        x = np.stack([rand_logits(g, V, b % 3) for b in range(B)])
        ps, biases, hists = [], [], []
        for b in range(B):
            p, bias = rand_params(g, V, True)
            ps.append(p)
            biases.append(bias)
            hists.append(rand_recent(g, V))
        params = np.concatenate(ps)
        us = g.random(B)
        xb = synth.f32_to_bf16_bits(x) if bf16 else x
        p_dev = ab.capi.params_to_device(params, "cuda")
        u_dev = torch.from_numpy(us).cuda()
        ids, vals, ns = [], [], []
        for r in range(G):  # what every rank would do on its own columns
            lo, hi = shard.vocab_range(V, r, G)
            if hi <= lo:
                ids.append(torch.full((B, ab.capi.KCAP), -1, dtype=torch.int32, device="cuda"))
                vals.append(torch.zeros(B, ab.capi.KCAP, device="cuda"))
                ns.append(torch.zeros(B, dtype=torch.int32, device="cuda"))
                continue
            lg, Vl = to_dev_logits(np.ascontiguousarray(xb[:, lo:hi]), bf16)
            o = ab.sample_batch(lg, p_dev, u_dev, V=Vl, id_base=lo, v_global=V, want_cands=True, **_lists(hists, biases, lo, hi))
            assert int(o["status"].item()) == 0
            ids.append(o["cand_id"])
            vals.append(o["cand_val"])
            ns.append(o["n_cand"])
        kw = _lists(hists, biases, 0, V)
        out = ab.merge_batch(torch.stack(ids), torch.stack(vals), torch.stack(ns), p_dev, u_dev, V,
                             bias_off=kw["bias_off"], bias_vals=kw["bias_vals"], want_cands=True)
        torch.cuda.synchronize()
        out = {k: v.cpu().numpy() for k, v in out.items()}
        check_rows(out, xb, bf16, params, hists, us, biases, tag=f"G={G}")


def test_packed_records_read_in_place():
    """The layout the shards exchange: every shard writes k ids and k values per row straight into
    a record of k * 8 + 8 bytes whose last two words carry (max, sum exp) of its raw columns; the
    merge reads the gathered records where they lie, without list lengths, and combines the pairs."""
    import torch

    import arcinfer_b200 as ab
    from gpuutil import check_rows, to_dev_logits

    g = np.random.default_rng(540)
    for V, B, G, k in [(40000, 7, 4, 64), (262144, 130, 2, 50), (151936, 5, 8, 20)]:
        x = np.stack([rand_logits(g, V, b % 3) for b in range(B)])
        params = synth.make_params(B, top_k=k, top_p=0.9, min_p=0.02, repeat_penalty=1.2, presence_penalty=0.3, temperature=0.8)
        params["top_k"][::3] = max(1, k // 2)
        hists = [rand_recent(g, V) for _ in range(B)]
        biases = [[] for _ in range(B)]
        us = g.random(B)
        xb = synth.f32_to_bf16_bits(x)
        p_dev = ab.capi.params_to_device(params, "cuda")
        u_dev = torch.from_numpy(us).cuda()
        gathered = torch.empty(G, B, shard.record_words(k), dtype=torch.int32, device="cuda")
        for r in range(G):
            lo, hi = shard.vocab_range(V, r, G)
            lg, Vl = to_dev_logits(np.ascontiguousarray(xb[:, lo:hi]), True)
            kw = _lists(hists, biases, lo, hi)
            o = ab.sample_batch(lg, p_dev, u_dev, V=Vl, id_base=lo, v_global=V, records=gathered[r],
                                hist_off=kw["hist_off"], hist_ids=kw["hist_ids"], max_hist=kw["max_hist"])
            assert int(o["status"].item()) == 0
            gathered[r, :, 2 * k :] = ab.argmax_batch(lg, V=Vl, want_lse=True)["max_sumexp"].view(torch.int32)
        out = ab.merge_records(gathered, p_dev, u_dev, V, want_cands=True, want_mz=True)
        torch.cuda.synchronize()
        assert int(out["status"].item()) == 0
        mz = out.pop("mz").cpu().numpy().astype(np.float64)
        out = {kk: v.cpu().numpy() for kk, v in out.items()}
        check_rows(out, xb, True, params, hists, us, biases, tag=f"packed G={G}")
        xf = synth.bf16_bits_to_f32(xb).astype(np.float64)
        m = xf.max(axis=1)
        lse = m + np.log(np.exp(xf - m[:, None]).sum(axis=1))
        assert np.array_equal(mz[:, 0], m)
        assert np.abs(mz[:, 0] + np.log(mz[:, 1]) - lse).max() < 1e-5  # (fp32 sums of exponentials per shard)
    # a row that keeps more candidates than the record holds is reported, not written past the record
    lg, Vl = to_dev_logits(np.ascontiguousarray(xb[:, :4096]), True)
    small = torch.empty(B, shard.record_words(4), dtype=torch.int32, device="cuda")
    o = ab.sample_batch(lg, p_dev, u_dev, V=Vl, records=small)
    torch.cuda.synchronize()
    assert int(o["status"].item()) == 2  # ARCS_ERR_TOPK


def test_two_ranks_over_nccl():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29531", os.path.join(ROOT, "tests", "vocab_shard_worker.py")],
                       cwd=ROOT, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "VOCAB_SHARD_OK" in r.stdout
