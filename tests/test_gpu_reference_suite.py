"""The reference's own sampler test (tests/test_sampler.cpp of the reference) run against the
CUDA-backed C++ mirror: oracle/_ref/test_sampler_mirror is that file, derived by
oracle/make_sampler_test.py (its `Sampler` bound to the mirror, its random rows made free of exactly
equal logits) and built where the reference tree is present. Every check of it compares with the
test's verbatim copy of the earlier implementation: greedy and banned-token behaviour, 2400 seeded
draws of sample(), and 4500 draws of sample_allowed() whose PREDICATE-CALL SEQUENCES must equal
the earlier implementation's (or be the prefix the e^-20 rule allows)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "oracle", "_ref", "test_sampler_mirror")


@pytest.mark.gpu
@pytest.mark.skipif(not os.path.exists(EXE), reason="oracle/_ref/test_sampler_mirror not built (reference tree absent at build time)")
def test_reference_sampler_test_passes_on_the_mirror():
    r = subprocess.run([EXE], capture_output=True, text=True, timeout=1500)
    tail = "\n".join(r.stdout.splitlines()[-25:])
    assert r.returncode == 0 and "ALL OK" in r.stdout, tail + r.stderr[-2000:]
    assert "FAIL" not in r.stdout, tail
    assert "rows with equal logits made distinct" in r.stdout
