#!/usr/bin/env python
"""Benchmark of the token-selection hot path on B200.

Workload (config.workload = "wide-batch"): B=1024 rows x V=262144 bf16 logits ~N(0,3^2), top-k 50,
top-p .95, repetition penalty 1.1 over each row's whole 512-token history, one uniform draw per
row: the fused penalty + top-k/top-p sampling pass, two kernel launches per step (the single pass
over the logits, and a small per-row finish that runs beside it). Rows are
independent, so with N GPUs every rank runs its own 1024-row batch (weak scaling, no data-path
collective) and the value is the rows all ranks sampled per second.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line (rank 0). `value` is timed with CUDA events over K launches with the
inputs resident in HBM (512 MiB of logits per step: larger than L2); `e2e` is the same metric
through the host-buffer entry point (pinned host logits copied in every step, token ids copied
back); `roofline` is the dominant kernel's (the pass over the logits) algorithmic bytes over its
average launch time, measured with CUDA events between the kernels, against the measured copy
bandwidth (MEASURED_PEAKS.json), with the whole step's figure beside it; `parity` compares the
tokens of 129 rows spread over the whole batch with the CPU checker after the timed region;
`cpu_baseline` is the reference's own CPU sampler (compiled from its sources into oracle/_ref)
timed on this box's host cores. With more than one rank the line also carries `vocab_shard`: the
same 1024 rows split by vocabulary columns over the ranks (strong scaling: local pass, one
all-gather of packed records, merge), timed after the main region.

  --workload logprobs | single-row | multi-slot | spec-verify | constrained | dflash   (one GPU)

print a line of their own for the other entry points and the reference's own small shapes; the
latency shapes are timed as CUDA graph replays with L2 flushed between calls.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

B_ROWS, VOCAB, HIST = 1024, 262144, 512
METRIC, UNIT = "sampled_rows_per_sec", "rows/s"


def algorithmic_bytes(B, V, H, elt):
    """bytes one launch must read: every logit once, every history id once"""
    return B * V * elt + B * H * 4


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def ncu_traffic(key):
    """DRAM bytes per launch from the committed ncu summary (profiles/traffic.json), if any"""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            return json.load(f).get(key)
    except Exception:
        return None


class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                       "-i", str(index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.f.read().splitlines():
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1]))
                mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        self.f.close()
        os.unlink(self.f.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_rate(logits_f32, params, hist_off, hist_ids, seeds, threads, min_seconds):
    """rows/s of the reference's Sampler::sample over the given rows, repeated until min_seconds"""
    import ctypes as C

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import numpy as np

    import orc

    if orc.ref is None:
        return None
    rows = logits_f32.shape[0]
    out = np.zeros(rows, np.int32)
    total_t, total_rows = 0.0, 0
    while total_rows == 0 or total_t < min_seconds:
        t = orc.ref.ref_sample_batch(params.ctypes.data_as(C.c_void_p), seeds.ctypes.data_as(C.c_void_p),
                                     logits_f32.ctypes.data_as(C.c_void_p), C.c_int64(rows), logits_f32.shape[1],
                                     hist_off.ctypes.data_as(C.c_void_p), hist_ids.ctypes.data_as(C.c_void_p), None,
                                     C.c_int64(0), threads, out.ctypes.data_as(C.c_void_p))
        total_t += t
        total_rows += rows
    return total_rows / total_t, out


def bench_logprobs(args):
    """Secondary workload (--workload logprobs, one GPU): arcs_logprobs_batch, the log probability
    of one token per row and the 20 most likely alternatives (tools/server_chat.h:417-441), on the
    same 1024 x 262144 bf16 logits. Prints its own JSON line."""
    import numpy as np
    import torch

    import arcinfer_b200 as ab
    sys.path.insert(0, os.path.join(ROOT, "tests"))

    B, V, top_n = args.rows, args.vocab, 20
    torch.cuda.set_device(0)
    gen = torch.Generator(device="cuda").manual_seed(20261125)
    logits = (torch.randn(B, V, device="cuda", generator=gen) * 3).to(torch.bfloat16)
    token = torch.randint(0, V, (B,), device="cuda", dtype=torch.int32, generator=gen)
    for _ in range(args.warmup):
        out = ab.logprobs_batch(logits, token, top_n)
    torch.cuda.synchronize()
    assert int(out["status"][0]) == 0
    clocks = ClockSampler(0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        ab.logprobs_batch(logits, token, top_n)
    e1.record()
    torch.cuda.synchronize()
    t_end = time.perf_counter() + 0.6  # (the timed steps take milliseconds: keep the same load up until the clocks have been sampled)
    while time.perf_counter() < t_end:
        ab.logprobs_batch(logits, token, top_n)
        torch.cuda.synchronize()
    clk = clocks.stop()
    ms = e0.elapsed_time(e1) / args.steps
    peak, which = measured_peak()
    by = B * V * logits.element_size()
    line = {
        "metric": "logprob_rows_per_sec", "value": B / (ms * 1e-3), "unit": "rows/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 logits, fp32 exponentials, fp64 sums", "data": "synthetic",
        "config": {"workload": "logprobs", "rows_per_gpu": B, "vocab": V, "top_logprobs": top_n,
                   "l2": "inputs (%d MiB) larger than L2" % (by >> 20)},
        "roofline": {"bound": "hbm", "kernel": "logprob_kernel", "achieved": by / (ms * 1e-3) / 1e9, "peak": peak,
                     "peak_source": which, "unit": "GB/s", "frac": by / (ms * 1e-3) / 1e9 / peak, "traffic": ncu_traffic("logprob_kernel_bf16_wide_batch"),
                     "note": "issue-bound on the exponentials, not on HBM"},
        "gpu_launches": args.steps, "clocks": clk,
    }
    if not args.no_cpu:
        import orc  # the CPU restatement, as the timed baseline only

        x = logits[:4].float().cpu().numpy()
        tk = token[:4].cpu().numpy()
        t0 = time.perf_counter()
        for r in range(4):
            orc.logprobs(x[r], int(tk[r]), top_n)
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": 4 / dt, "unit": "rows/s", "cores": 1, "kind": "port", "sample": "4 rows of the workload, one thread"}
    print(json.dumps(line), flush=True)


def bench_small(args):
    """The four latency workloads (--workload single-row | multi-slot | spec-verify | constrained, one
    GPU): the shapes the reference itself runs (at most 16 rows a pass, zero/engine.h:2910, scaled as
    the measured configurations say). One step = one call on device-resident inputs; `e2e` = the same
    call through the host-buffer entry point; every row's result is compared with the CPU checker;
    `cpu_baseline` = the reference's own code on one host thread, which is how the reference runs it."""
    import ctypes as C

    import numpy as np
    import torch

    import arcinfer_b200 as ab
    from arcinfer_b200 import synth

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import orc

    torch.cuda.set_device(0)
    dev = "cuda"
    wl = args.workload
    c = {"single-row": synth.config1, "multi-slot": synth.config2, "spec-verify": synth.config3, "constrained": synth.config4}[wl]()
    x = c["logits"]
    bf16 = c["bf16"]
    B, V = x.shape
    lg = torch.from_numpy(x.view(np.int16)).to(dev).view(torch.bfloat16) if bf16 else torch.from_numpy(x).to(dev)
    xf = synth.bf16_bits_to_f32(x) if bf16 else x
    elt = 2 if bf16 else 4
    launches_per_step, extra_bytes = 2, 0
    if wl == "spec-verify":
        kw = dict(row_off=torch.from_numpy(c["row_off"]).to(dev), draft=torch.from_numpy(c["draft"]).to(dev), draft_off=torch.from_numpy(c["draft_off"]).to(dev))
        step = lambda: ab.argmax_batch(lg, **kw)
        launches_per_step, extra_bytes = 1, c["draft"].nbytes
        kernel = "argmax_kernel"
    else:
        p_dev = ab.capi.params_to_device(c["params"], dev)
        u = torch.from_numpy(np.ascontiguousarray(c["u"])).to(dev)
        ho, hi = synth.csr(c["hist"])
        H = int(max(len(h) for h in c["hist"]))
        kw = {}
        if H:
            kw = dict(hist_off=torch.from_numpy(ho).to(dev), hist_ids=torch.from_numpy(hi).to(dev), max_hist=H)
            extra_bytes += hi.nbytes
        if wl == "constrained":
            states, inv = np.unique(c["states"], return_inverse=True)
            tab = torch.from_numpy(c["table"].view(np.int16)).to(dev)
            st_dev = torch.from_numpy(states.astype(np.int32)).to(dev)
            off_dev, by_dev = torch.from_numpy(c["byte_off"].view(np.int32)).to(dev), torch.from_numpy(c["bytes"]).to(dev)
            mrow = torch.from_numpy(inv.astype(np.int32)).to(dev)
            launches_per_step = 3
            extra_bytes += c["bytes"].nbytes + c["byte_off"].nbytes + c["table"].nbytes + len(states) * ((V + 31) // 32) * 4

            # the argument blocks are built once (a caller that decodes step after step does the same)
            m_dev = ab.dfa_mask(tab, c["dead"], st_dev, off_dev, by_dev, V=V)
            plan = ab.capi.SamplePlan(lg, p_dev, u, mask=m_dev, mask_row=mrow, **kw)

            def step():  # the mask of every distinct automaton state, then the constrained selection
                ab.dfa_mask(tab, c["dead"], st_dev, off_dev, by_dev, V=V, out=m_dev)
                return plan.launch()
        else:
            plan = ab.capi.SamplePlan(lg, p_dev, u, **kw)
            step = plan.launch
        kernel = "stream_kernel"
    for _ in range(max(args.warmup, 5)):
        out = step()
    torch.cuda.synchronize()
    # The step is captured in a CUDA graph and replayed: at these sizes the host's work between two
    # launches (tens of microseconds in Python) would otherwise sit inside the timed region.
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            out = step()
    torch.cuda.synchronize()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than L2: written between timed calls
    clocks = ClockSampler(0)
    times = []
    for _ in range(args.steps):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    t_end = time.perf_counter() + 0.5
    while time.perf_counter() < t_end:
        graph.replay()
        torch.cuda.synchronize()
    clk = clocks.stop()
    ms = float(np.median(times))
    assert int(out["status"].item()) == 0
    # ---- every row against the CPU checker
    bad = 0
    masks_h = None
    if wl == "spec-verify":
        sel = np.array([orc.argmax(r) for r in xf], np.int32)
        acc, nxt = orc.verify_greedy(sel, c["row_off"], c["draft"], c["draft_off"])
        bad = int((out["argmax"].cpu().numpy() != sel).sum() + (out["accepted"].cpu().numpy() != acc).sum() + (out["next"].cpu().numpy() != nxt).sum())
    else:
        if wl == "constrained":
            masks_h = ab.dfa_mask(tab, c["dead"], st_dev, off_dev, by_dev, V=V).cpu().numpy().view(np.uint32)
            for i, sidx in enumerate(states):
                bad += int(not np.array_equal(masks_h[i], orc.dfa_mask(c["table"], c["dead"], int(sidx), c["byte_off"], c["bytes"])))
        tok = out["token"].cpu().numpy()
        for b in range(B):
            m = None if masks_h is None else masks_h[inv[b]]
            bad += int(tok[b] != orc.sample(xf[b], c["params"][b:b + 1], c["hist"][b], float(c["u"][b]), None, m)["token"])
    parity = {"rows_checked": B, "mismatches": bad, "against": "oracle/arcs_oracle.c on the same inputs"}
    if bad:
        print(json.dumps({"parity": parity}), flush=True)
        sys.exit(3)
    # ---- end to end: host buffers in, results out
    ctx = ab.capi.HostContext(0, B, V, bf16, max_hist_total=max(1, extra_bytes), max_mask_words=(B * ((V + 31) // 32)) if wl == "constrained" else 0)
    h_x = torch.from_numpy(x.view(np.int16) if bf16 else x).pin_memory().numpy()
    if bf16:
        h_x = h_x.view(np.uint16)
    if wl == "spec-verify":
        am, ac, nx = np.zeros(B, np.int32), np.zeros(len(c["row_off"]) - 1, np.int32), np.zeros(len(c["row_off"]) - 1, np.int32)
        host_step = lambda: ctx.argmax(h_x, am, row_off=c["row_off"], draft=c["draft"], draft_off=c["draft_off"], accepted=ac, next_=nx)
        d2h = am.nbytes + ac.nbytes + nx.nbytes
    else:
        tk = np.zeros(B, np.int32)
        hkw = dict(hist_off=ho, hist_ids=hi, max_hist=H) if H else {}
        if wl == "constrained":
            hkw.update(mask=np.ascontiguousarray(masks_h), mask_row=inv.astype(np.int32))
        us = np.ascontiguousarray(c["u"])
        host_step = lambda: ctx.sample(h_x, c["params"], us, tk, **hkw)
        d2h = tk.nbytes + 4
    for _ in range(3):
        host_step()
    t0 = time.perf_counter()
    esteps = max(5, min(args.steps, 20))
    for _ in range(esteps):
        host_step()
    e_ms = 1e3 * (time.perf_counter() - t0) / esteps
    ctx.close()
    # ---- the reference's own code, one host thread
    cpu = None
    if not args.no_cpu:
        t0 = time.perf_counter()
        reps = 0
        while reps == 0 or time.perf_counter() - t0 < 3.0:
            if wl == "spec-verify":
                sel = np.array([orc.argmax(r) for r in xf], np.int32)
                orc.verify_greedy(sel, c["row_off"], c["draft"], c["draft_off"])
            elif orc.ref is not None:
                seeds = np.arange(1, B + 1, dtype=np.uint64)
                outc = np.zeros(B, np.int32)
                mk = None if masks_h is None else np.ascontiguousarray(masks_h[inv])
                orc.ref.ref_sample_batch(c["params"].ctypes.data_as(C.c_void_p), seeds.ctypes.data_as(C.c_void_p), np.ascontiguousarray(xf).ctypes.data_as(C.c_void_p),
                                         C.c_int64(B), V, ho.ctypes.data_as(C.c_void_p), (hi if len(hi) else np.zeros(1, np.int32)).ctypes.data_as(C.c_void_p),
                                         None if mk is None else mk.ctypes.data_as(C.c_void_p), C.c_int64(0 if mk is None else mk.shape[1]), 1,
                                         outc.ctypes.data_as(C.c_void_p))
            else:
                for b in range(B):
                    orc.sample(xf[b], c["params"][b:b + 1], c["hist"][b], float(c["u"][b]), None, None if masks_h is None else masks_h[inv[b]])
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        kind = "reference" if (orc.ref is not None and wl != "spec-verify") else "port"
        cpu = {"value": B / dt, "unit": UNIT, "cores": 1, "kind": kind, "sample": f"the whole workload ({B} rows), repeated for >= 3 s, one thread"}
    peak, which = measured_peak()
    abytes = B * V * elt + extra_bytes
    line = {
        "metric": METRIC, "value": B / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 5),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if bf16 else "f32",
        "data": "synthetic", "config": {"workload": wl, "rows": B, "vocab": V, "l2": "L2 flushed (256 MiB written) between timed calls; median of the calls", "launch": "CUDA graph replay of the step"},
        "gpu_launches": launches_per_step * args.steps, "clocks": clk,
        "e2e": {"value": B / (e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": B * V * elt + extra_bytes, "d2h_bytes_per_step": d2h, "ms_per_step": e_ms},
        "roofline": {"bound": "hbm", "kernel": kernel, "achieved": abytes / (ms * 1e-3) / 1e9, "peak": peak, "peak_source": f"of {which}", "unit": "GB/s",
                     "frac": abytes / (ms * 1e-3) / 1e9 / peak, "traffic": None, "algorithmic_bytes_per_launch": abytes,
                     "note": "a latency case: launch and per-row dependency chains, not HBM, bound it"},
        "cpu_baseline": cpu, "parity": parity,
    }
    print(json.dumps(line), flush=True)


def bench_dflash(args):
    """--workload dflash (one GPU): the DFlash2 candidate selector (zero/engine_drafters.h:461-506)
    for 8 slots x 7 draft positions of a 151936-token vocabulary, rank-256 codebooks, top-16
    candidates, min_p 0.3. One step = arcs_dflash_select on device-resident inputs (a CUDA graph
    replay, L2 flushed between calls); every slot's drafts are compared with the CPU checker."""
    import numpy as np
    import torch

    import arcinfer_b200 as ab
    from arcinfer_b200 import synth

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import orc

    torch.cuda.set_device(0)
    dev = "cuda"
    slots, nd, V, rank, topk, min_p = 8, 7, 151936, 256, 16, 0.3
    g = np.random.default_rng(synth.BASE_SEED + 31)
    logits = (g.standard_normal((slots, nd, V)) * 2.0).astype(np.float32)
    for s_ in range(slots):
        for t in range(nd):
            logits[s_, t, g.integers(0, V, 3)] += np.float32(5.0)
    hproj = g.standard_normal((slots, nd, rank)).astype(np.float32)
    pred = synth.f32_to_bf16_bits((g.standard_normal((V, rank)) * 0.3).astype(np.float32))
    succ = synth.f32_to_bf16_bits((g.standard_normal((V, rank)) * 0.3).astype(np.float32))
    tok = g.integers(0, V, slots).astype(np.int32)
    d = [torch.from_numpy(a).to(dev) for a in (logits, hproj, pred.view(np.int16), succ.view(np.int16), tok)]
    step = lambda: ab.dflash_select(d[0], d[1], d[2], d[3], d[4], topk=topk, max_drafts=nd, min_p=min_p)
    for _ in range(max(args.warmup, 5)):
        out = step()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            out = step()
    torch.cuda.synchronize()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    clocks = ClockSampler(0)
    times = []
    for _ in range(args.steps):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    clk = clocks.stop()
    ms = float(np.median(times))
    assert int(out["status"].item()) == 0
    n_out, toks = out["n_out"].cpu().numpy(), out["tokens"].cpu().numpy()
    bad = 0
    t0 = time.perf_counter()
    for s_ in range(slots):
        want, _ = orc.dflash_select(logits[s_], hproj[s_], pred, succ, topk, nd, int(tok[s_]), min_p)
        bad += int(n_out[s_] != len(want) or not np.array_equal(toks[s_, : len(want)], want))
    cpu_dt = time.perf_counter() - t0
    parity = {"rows_checked": slots, "mismatches": bad, "against": "oracle/arcs_oracle.c (pinned to the reference's loop) on the same inputs"}
    if bad:
        print(json.dumps({"parity": parity}), flush=True)
        sys.exit(3)
    peak, which = measured_peak()
    R = slots * nd
    abytes = R * V * 4 + R * rank * 4 + R * (topk + 1) * rank * 2
    print(json.dumps({
        "metric": "draft_rows_per_sec", "value": R / (ms * 1e-3), "unit": "rows/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 5),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 logits, bf16 codebooks, fp64 scores",
        "data": "synthetic", "config": {"workload": "dflash", "slots": slots, "positions": nd, "vocab": V, "rank": rank, "topk": topk, "min_p": min_p,
                                        "l2": "L2 flushed (256 MiB written) between timed calls; median of the calls", "launch": "CUDA graph replay of the step"},
        "gpu_launches": 3 * args.steps, "clocks": clk, "e2e": None,
        "roofline": {"bound": "hbm", "kernel": "logprob_kernel", "achieved": abytes / (ms * 1e-3) / 1e9, "peak": peak, "peak_source": f"of {which}", "unit": "GB/s",
                     "frac": abytes / (ms * 1e-3) / 1e9 / peak, "traffic": None, "algorithmic_bytes_per_launch": abytes,
                     "note": "a latency case: 56 rows in one pass, then a sequential walk of 7 positions per slot"},
        "cpu_baseline": {"value": R / cpu_dt, "unit": "rows/s", "cores": 1, "kind": "port", "sample": f"the whole workload ({slots} slots), once, one thread"},
        "parity": parity}), flush=True)


def vocab_shard_leg(ab, synth, dist, rank, world, dev, B, V, H, params, steps, warmup, check_rows=4):
    """The vocabulary-sharded step (strong scaling): every rank holds its columns of ALL B rows,
    runs the selection on them under global ids into packed records, one all-gather of
    B * (k * 8 + 8) bytes per rank, then the merge. Timed on the device, max over ranks. Rank 0
    checks a few rows against the CPU checker on the rows' full width (their columns are gathered
    from all ranks for that, outside the timed region)."""
    import numpy as np
    import torch

    from arcinfer_b200 import shard

    lo, hi = shard.vocab_range(V, rank, world)
    gen = torch.Generator(device=dev)
    gen.manual_seed(synth.BASE_SEED + 7 + 1000 * rank)
    local_logits = torch.empty(B, hi - lo, dtype=torch.bfloat16, device=dev)
    for r0 in range(0, B, 128):
        r1 = min(B, r0 + 128)
        local_logits[r0:r1] = (torch.randn(r1 - r0, hi - lo, generator=gen, device=dev) * 3.0).to(torch.bfloat16)
    gen.manual_seed(synth.BASE_SEED + 8)  # lists and draws are the same on every rank
    hist = torch.randint(0, V, (B, H), generator=gen, device=dev, dtype=torch.int32)
    hist_off = (torch.arange(B + 1, device=dev, dtype=torch.int32) * H).contiguous()
    u = torch.rand(B, generator=gen, device=dev, dtype=torch.float64)
    p_dev = ab.capi.params_to_device(params, dev)
    k = int(params["top_k"].max())
    st = shard.VocabShardStep(local_logits, lo, V, p_dev, u, world, k, hist_off=hist_off, hist_ids=hist.reshape(-1), max_hist=H)
    for _ in range(max(warmup, 3)):
        out = st.step(dist.all_gather_into_tensor)
    dist.barrier()
    torch.cuda.synchronize()
    # the step as a CUDA graph (local pass, collective, merge): no host between its launches
    launch = "CUDA graph replay"
    try:
        graph = st.capture(dist.all_gather_into_tensor)
        run = graph.replay
    except Exception as e:  # (a stack that cannot capture the collective: the eager step is timed instead)
        launch = f"eager ({type(e).__name__})"
        graph, run = None, (lambda: st.step(dist.all_gather_into_tensor))
    for _ in range(3):
        run()
    dist.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        run()
    ev1.record()
    if graph is not None:
        out = st.out
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / steps
    assert int(out["status"].item()) == 0 and int(st.plan.status.item()) == 0
    toks = [torch.empty_like(out["token"]) for _ in range(world)]
    dist.all_gather(toks, out["token"])
    same = all(bool((x == toks[0]).all()) for x in toks)
    # ---- a few rows on their full width against the CPU checker (rank 0)
    rows = sorted(set(np.linspace(0, B - 1, check_rows).astype(int).tolist()))
    width = shard.vocab_range(V, 0, world)[1]
    mine = torch.zeros(len(rows), width, dtype=torch.bfloat16, device=dev)
    mine[:, : hi - lo] = local_logits[torch.tensor(rows, device=dev)]
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    bad = 0
    if rank == 0:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import orc  # the checker; never on the timed path

        full = torch.cat([parts[r][:, : shard.vocab_range(V, r, world)[1] - shard.vocab_range(V, r, world)[0]] for r in range(world)], dim=1)
        xf = full.float().cpu().numpy()
        hh, uu, tk = hist.cpu().numpy(), u.cpu().numpy(), out["token"].cpu().numpy()
        for i, b in enumerate(rows):
            bad += int(tk[b] != orc.sample(xf[i], params[b:b + 1], hh[b], float(uu[b]))["token"])
    return {"ms_per_step": ms_step, "value": B / (ms_step * 1e-3), "unit": UNIT, "scaling": "strong", "rows": B,
            "all_ranks_agree": same, "collective_bytes_per_rank": st.collective_bytes_per_rank, "record_entries": k,
            "parity": {"rows_checked": len(rows), "mismatches": bad, "against": "oracle/arcs_oracle.c on the rows' full width"},
            "launches_per_step": 3, "launch": launch, "note": "local pass (stream + finish kernels), all_gather_into_tensor of packed records, merge kernel"}


def bind_near_gpu(torch, local):
    """Run this process (and allocate its pinned host memory: first touch) on the CPU cores the
    GPU hangs off. With several ranks on a multi-socket host, a rank left on the wrong socket copies
    its batch to its GPU across the socket link. Only the process's own CPU affinity is set (a
    property of this process, read from NVML; nothing of the GPU is changed). Returns what was done."""
    try:
        import pynvml

        pynvml.nvmlInit()
        pr = torch.cuda.get_device_properties(local)
        bus = f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (w >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return "no cores in common with the allowed set"
        os.sched_setaffinity(0, cpus)
        return f"{len(cpus)} cores near GPU {local}"
    except Exception as e:  # (no NVML, no permission: the run goes on unbound)
        return f"unbound ({type(e).__name__})"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=B_ROWS, help="rows per GPU (default: the measured workload)")
    ap.add_argument("--vocab", type=int, default=VOCAB)
    ap.add_argument("--shard", default="rows", choices=["rows", "vocab"],
                    help="how N GPUs split the work: rows (default, no collective) or vocabulary columns (one all-gather)")
    ap.add_argument("--workload", default="wide-batch", choices=["wide-batch", "logprobs", "single-row", "multi-slot", "spec-verify", "constrained", "dflash"],
                    help="wide-batch: the sampling step (the headline); logprobs: arcs_logprobs_batch on the same logits; the other four: "
                         "the latency workloads of the measured configurations 1-4 (one GPU)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of the timed launch's tokens")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.workload == "logprobs" and args.impl == "ours":
        if int(os.environ.get("RANK", "0")) == 0:
            bench_logprobs(args)
        return
    if args.workload == "dflash" and args.impl == "ours":
        if int(os.environ.get("RANK", "0")) == 0:
            bench_dflash(args)
        return
    if args.workload in ("single-row", "multi-slot", "spec-verify", "constrained") and args.impl == "ours":
        if int(os.environ.get("RANK", "0")) == 0:
            bench_small(args)
        return

    import numpy as np
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    B, V, H = args.rows, args.vocab, HIST
    config = {"workload": "wide-batch", "rows_per_gpu": B, "vocab": V, "history": H, "top_k": 50, "top_p": 0.95,
              "repeat_penalty": 1.1, "logits": "bf16 ~N(0,3^2)", "partition": f"rows x{world}",
              "l2": "inputs (512 MiB per step) larger than L2"}

    from arcinfer_b200 import synth

    params = synth.make_params(B, top_k=50, top_p=0.95, repeat_penalty=1.1, repeat_last_n=-1)

    if args.impl == "reference":
        # the reference's own CPU sampler on this box's host cores; rank 0 only
        if rank != 0:
            return
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import orc

        if orc.ref is None:
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libarcs_ref.so not built (reference tree absent at build time)"}))
            return
        threads = int(orc.ref.ref_hardware_threads()) or os.cpu_count() or 1
        S = max(threads, min(B, 128))  # rows per step: a bounded sample of the 1024-row batch
        g = synth.rng(synth.BASE_SEED + 5)
        x = synth.bf16_bits_to_f32(synth.normal_logits(g, S, V, 3.0, bf16=True))
        hist = g.integers(0, V, (S, H)).astype(np.int32)
        hoff = (np.arange(S + 1) * H).astype(np.int32)
        seeds = g.integers(1, 2**62, S).astype(np.uint64)
        p = params[:1].repeat(S)
        for _ in range(min(args.warmup, 1)):
            cpu_reference_rate(x, p, hoff, hist.reshape(-1), seeds, threads, 0.0)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            cpu_reference_rate(x, p, hoff, hist.reshape(-1), seeds, threads, 0.0)
        dt = time.perf_counter() - t0
        val = S * args.steps / dt
        sample = f"{S} rows of the workload per step (widened to fp32), {threads} threads, one Sampler per row"
        print(json.dumps({"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
                          "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                          "data": "synthetic", "config": config,
                          "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "reference", "sample": sample},
                          "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    import arcinfer_b200 as ab

    assert torch.cuda.is_available(), "bench.py needs a CUDA device: there is no CPU fallback"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    bound = bind_near_gpu(torch, local) if world > 1 else "single rank: not bound"
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.shard == "vocab" and world > 1:
        leg = vocab_shard_leg(ab, synth, dist, rank, world, dev, B, V, H, params, args.steps, args.warmup)
        if rank == 0:
            config["partition"] = f"vocabulary columns x{world}"
            config["rows_per_gpu"] = B
            print(json.dumps({"metric": METRIC, "value": leg["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
                              "warmup": args.warmup, "ms_per_step": leg["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                              "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
                              "gpu_launches": 3 * args.steps, "vocab_shard": leg}))
        dist.destroy_process_group()
        return

    # ---- synthetic inputs, generated on the device from a per-rank seed
    gen = torch.Generator(device=dev)
    gen.manual_seed(synth.BASE_SEED + 5 + 1000 * rank)
    logits = torch.empty(B, V, dtype=torch.bfloat16, device=dev)
    for r0 in range(0, B, 128):
        r1 = min(B, r0 + 128)
        logits[r0:r1] = (torch.randn(r1 - r0, V, generator=gen, device=dev) * 3.0).to(torch.bfloat16)
    hist = torch.randint(0, V, (B, H), generator=gen, device=dev, dtype=torch.int32)
    hist_off = (torch.arange(B + 1, device=dev, dtype=torch.int32) * H).contiguous()
    u = torch.rand(B, generator=gen, device=dev, dtype=torch.float64)
    p_dev = ab.capi.params_to_device(params, dev)
    plan = ab.capi.SamplePlan(logits, p_dev, u, hist_off=hist_off, hist_ids=hist.reshape(-1), max_hist=H)

    for _ in range(args.warmup):
        plan.launch()
    barrier()
    clocks = ClockSampler(local) if rank == 0 else None
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        out = plan.launch()
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    status = int(plan.status.item())
    tok = out["token"]
    assert status == 0, f"device status {status}"
    assert int(tok.min()) >= 0 and int(tok.max()) < V
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / args.steps
    value = world * B / (ms_step * 1e-3)

    # ---- parity of the timed launch itself (rank 0): every eighth row of the batch, so that every
    # persistent CTA and each of its rotating sets of per-item state is hit, against the CPU checker
    parity = None
    if rank == 0 and not args.no_parity:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import orc  # the checker; never on the timed path

        rows = sorted(set(list(range(0, B, max(1, B // 128))) + [B - 1]))
        idx = torch.tensor(rows, device=dev)
        xf = logits[idx].float().cpu().numpy()
        hh, uu, tk = hist[idx].cpu().numpy(), u[idx].cpu().numpy(), tok[idx].cpu().numpy()
        bad, ties = [], 0
        for i, b in enumerate(rows):
            want = orc.sample(xf[i], params[b:b + 1], hh[i], float(uu[i]))
            ties += int((want["flags"] & 1) != 0)
            if int(tk[i]) != int(want["token"]):
                bad.append(b)
        parity = {"rows_checked": len(rows), "mismatches": len(bad), "tie_rows": ties,
                  "against": "oracle/arcs_oracle.c (value desc, id asc), same logits, histories and uniform draws"}
        if bad:
            print(json.dumps({"parity": parity, "mismatched_rows": bad[:16]}), flush=True)
            sys.exit(3)

    # ---- end to end through the host-buffer entry point: pinned host logits in, token ids out
    e2e = None
    if not args.no_e2e:
        h_logits = torch.empty(B, V, dtype=torch.bfloat16).pin_memory()
        h_logits.copy_(logits)
        h_hist = hist.reshape(-1).cpu().pin_memory()
        h_off = hist_off.cpu().pin_memory()
        h_u = u.cpu().pin_memory()
        h_tok = torch.empty(B, dtype=torch.int32).pin_memory()
        ctx = ab.capi.HostContext(local, B, V, True, max_hist_total=B * H)
        esteps = max(3, min(args.steps, 10))
        for _ in range(2):
            ctx.sample(h_logits, params, h_u, h_tok, hist_off=h_off, hist_ids=h_hist, max_hist=H)
        same = bool((h_tok.to(dev) == tok).all())
        barrier()
        t0 = time.perf_counter()
        for _ in range(esteps):
            ctx.sample(h_logits, params, h_u, h_tok, hist_off=h_off, hist_ids=h_hist, max_hist=H)
        barrier()
        dt = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([dt], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        h2d = B * V * 2 + B * H * 4 + (B + 1) * 4 + B * 8 + B * 32
        e2e = {"value": world * B * esteps / dt, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": B * 4 + 4,
               "steps": esteps, "ms_per_step": 1e3 * dt / esteps, "same_tokens_as_device_path": same,
               # every rank copies its own batch from its own pinned buffer: the step is the host-to-device
               # copy, and what N ranks reach together is bounded by the host side they share
               "h2d_gbs_per_rank": h2d / dt * esteps / 1e9, "h2d_gbs_all_ranks": world * h2d / dt * esteps / 1e9,
               "host_cores": bound}
        ctx.close()
        del h_logits
    clk = clocks.stop() if clocks else None
    # ---- the two kernels of a step, each timed with CUDA events on the launching stream (after
    # the timed region, same inputs: the dominant one, the stream kernel, carries the roofline)
    kms = np.array([plan.launch_timed() for _ in range(max(3, min(args.steps, 20)))], dtype=np.float64)
    k_stream, k_fin = (float(x) for x in np.median(kms, axis=0))

    # ---- more than one GPU: the vocabulary-sharded variant of the step as well (the same B rows
    # spread by columns over the ranks: strong scaling, one collective), after the main region
    vleg = None
    if world > 1:
        del logits, plan
        torch.cuda.empty_cache()
        try:
            vleg = vocab_shard_leg(ab, synth, dist, rank, world, dev, B, V, H, params, args.steps, args.warmup)
        except Exception as e:  # (the main measurement above stands on its own: its line is printed whatever happens here)
            vleg = {"error": f"{type(e).__name__}: {e}"[:300]}

    # ---- the reference's CPU sampler on this box's host cores (rank 0, one GPU only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import orc

        if orc.ref is not None:
            threads = int(orc.ref.ref_hardware_threads()) or os.cpu_count() or 1
            S = min(B, max(64, threads))
            x = logits[:S].float().cpu().numpy()
            hh = hist[:S].cpu().numpy().reshape(-1)
            hoff = (np.arange(S + 1) * H).astype(np.int32)
            seeds = np.arange(1, S + 1, dtype=np.uint64)
            rate_all, _ = cpu_reference_rate(x, params[:S].copy(), hoff, hh, seeds, threads, 8.0)
            rate_one, _ = cpu_reference_rate(x[:8], params[:8].copy(), hoff[:9], hh[: 8 * H], seeds[:8], 1, 2.0)
            cpu = {"value": rate_all, "unit": UNIT, "cores": threads, "kind": "reference",
                   "sample": f"first {S} rows of the batch (widened to fp32), repeated for >= 8 s, {threads} threads",
                   "single_thread_value": rate_one}
        else:
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "reference", "sample": "oracle/_ref not built"}

    if rank == 0:
        peak, which = measured_peak()
        abytes = algorithmic_bytes(B, V, H, 2)
        achieved = abytes / (k_stream * 1e-3) / 1e9
        step_gbs = abytes / (ms_step * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": config, "gpu_launches": 2 * args.steps, "clocks": clk, "e2e": e2e,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": ncu_traffic("stream_kernel_bf16_wide_batch"), "peak_source": f"of {which}",
                         "kernel": "stream_kernel", "algorithmic_bytes_per_launch": abytes,
                         "kernel_ms": {"stream": k_stream, "finish": k_fin, "note": "each alone, one after the other; in a step the finish kernel runs beside the stream kernel"},
                         "whole_step": {"achieved": step_gbs, "frac": step_gbs / peak}},
            "cpu_baseline": cpu, "parity": parity,
        }
        if vleg is not None:
            line["vocab_shard"] = vleg
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
