"""The C-ABI library loads without a GPU and exports every entry point include/arcsample.h declares;
argument checks that need no device work the same everywhere."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    import arcinfer_b200 as ab

    hdr = open(os.path.join(ROOT, "include", "arcsample.h")).read()
    names = set(re.findall(r"\b(arcs_[a-z_0-9]+)\s*\(", hdr))
    assert {"arcs_sample_batch", "arcs_argmax_batch", "arcs_dfa_mask", "arcs_sample_batch_host",
            "arcs_argmax_batch_static", "arcs_logprobs_batch"} <= names
    for n in sorted(names):
        assert hasattr(ab.lib, n), n
    assert ab.lib.arcs_version() == 1


def test_argument_checks_need_no_device():
    import arcinfer_b200 as ab

    a = ab.capi.SampleArgs()
    assert ab.lib.arcs_sample_batch(C.byref(a), None) == 1  # ARCS_ERR_ARG
    assert b"bad argument" in ab.lib.arcs_last_error()
    g = ab.capi.ArgmaxArgs()
    assert ab.lib.arcs_argmax_batch(C.byref(g), None) == 1
    lp = ab.capi.LogprobArgs()
    assert ab.lib.arcs_logprobs_batch(C.byref(lp), None) == 1
    assert ab.lib.arcs_sample_workspace_bytes(1024, 262144, 0, 0) >= 1024 * 4
    # (many rows: one block a row either way, a masked one with the head ranking's list on top)
    assert ab.lib.arcs_sample_workspace_bytes(1024, 262144, 1, 0) > ab.lib.arcs_sample_workspace_bytes(1024, 262144, 0, 0)
    assert ab.lib.arcs_sample_workspace_bytes(8, 262144, 0, 512) > ab.lib.arcs_sample_workspace_bytes(8, 262144, 0, 0)


def test_struct_layout_matches_header():
    import arcinfer_b200 as ab

    assert ab.capi.PARAMS_DTYPE.itemsize == 32
    # pointer / int64 fields first-order check: the C struct is 8-byte aligned with no surprises
    assert C.sizeof(ab.capi.SampleArgs) % 8 == 0 and C.sizeof(ab.capi.ArgmaxArgs) % 8 == 0
