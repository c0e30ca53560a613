"""The C++ mirror of the reference's Sampler (arcinfer_b200/host/sampler_b200.hpp): it compiles
against the C ABI alone (checked here without a GPU), and a compiled program that replays call
sequences through it gives the tokens of the CPU oracle, generator handling included (GPU)."""
import os
import struct
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "sampler_replay.cpp")


def test_wrapper_compiles_without_cuda_headers():
    subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-Wall", SRC], check=True, cwd=ROOT)


def orc_default_params():
    import orc

    p = np.zeros(1, orc.PARAMS_DTYPE)
    p["temperature"], p["top_p"], p["repeat_penalty"], p["repeat_last_n"], p["top_k"] = 1.0, 0.95, 1.0, 64, 20
    return p


def _write_case(path, logits, p, recent, bias, mask, seed, n_calls, append):
    with open(path, "wb") as f:
        f.write(struct.pack("<6i", len(logits), len(recent), len(bias), n_calls, int(mask is not None), int(append)))
        f.write(struct.pack("<6f2iQ", float(p["temperature"][0]), float(p["top_p"][0]), float(p["min_p"][0]),
                            float(p["presence_penalty"][0]), float(p["frequency_penalty"][0]), float(p["repeat_penalty"][0]),
                            int(p["repeat_last_n"][0]), int(p["top_k"][0]), seed))
        f.write(np.asarray(logits, np.float32).tobytes())
        f.write(np.asarray(recent, np.int32).tobytes())
        f.write(np.asarray([t for t, _ in bias], np.int32).tobytes())
        f.write(np.asarray([b for _, b in bias], np.float32).tobytes())
        if mask is not None:
            f.write(np.asarray(mask, np.uint32).tobytes())


@pytest.mark.gpu
def test_wrapper_replays_like_the_oracle(tmp_path):
    import orc
    from cases import rand_logits, rand_mask, rand_params, rand_recent

    exe = str(tmp_path / "sampler_replay")
    libdir = os.path.join(ROOT, "arcinfer_b200", "lib")
    subprocess.run(["g++", "-std=c++17", "-O1", SRC, "-o", exe, "-L" + libdir, "-larcsample", "-Wl,-rpath," + libdir],
                   check=True, cwd=ROOT)
    g = np.random.default_rng(77)
    for case in range(12):
        V = int(g.choice([300, 5000, 40000]))
        masked = case % 3 == 2
        logits = rand_logits(g, V, 0)
        p, bias = rand_params(g, V, True, allow_k0=not masked)
        recent = rand_recent(g, V)
        if case == 10:  # a long answer with default parameters: the history is never read (tools/sampler.h:151)
            p, bias = orc_default_params(), []
            recent = g.integers(0, V, 5000).astype(np.int32)
        if case == 11:  # ... and with the repeat penalty alone, which reads the last 64 ids
            p, bias = orc_default_params(), []
            p["repeat_penalty"] = 1.3
            recent = g.integers(0, V, 70000).astype(np.int32)
        mask = rand_mask(g, V, 0.3) if masked else None
        seed, n_calls, append = int(g.integers(1, 1 << 40)), 5, case % 2 == 0
        path = str(tmp_path / f"case{case}.bin")
        _write_case(path, logits, p, recent, bias, mask, seed, n_calls, append)
        got = [int(x) for x in subprocess.run([exe, path], check=True, capture_output=True, text=True).stdout.split()]
        # the oracle with the reference's draw sequence: a draw is consumed by every non-greedy call,
        # except a constrained call left with at most one candidate (tools/sampler.h:38, :122)
        us = orc.u_from_seed(seed, n_calls)
        hist, k, want = list(recent), 0, []
        for _ in range(n_calls):
            o = orc.sample(logits, p, np.asarray(hist, np.int32), float(us[k]), bias, mask)
            want.append(int(o["token"]))
            if float(p["temperature"][0]) > 0.0 and not (masked and o["n_cand"] <= 1):
                k += 1
            if append and o["token"] >= 0:
                hist.append(int(o["token"]))
        assert got == want, (case, got, want)
