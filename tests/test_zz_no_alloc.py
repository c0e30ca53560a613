"""The entry point that allocates nothing (arcs_argmax_batch_static): for hosts that have closed
their device allocator (all of HBM belongs to their own pool) or must not call it between the
kernels of a step. Its scratch is a fixed array inside the library, so its results must equal the
plain entry point's on calls in a row, which also shows that each call leaves the array clean.
Collected last on purpose: a run that stops at the first failure has then run everything else."""
import numpy as np
import pytest
import torch

import orc
from arcinfer_b200 import synth

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_workspace_entry_point():
    import arcinfer_b200 as ab

    c = synth.config3(slots=4, rows_per_slot=4, V=50000)
    lg = torch.from_numpy(c["logits"].view(np.int16)).cuda().view(torch.bfloat16)
    kw = dict(row_off=torch.from_numpy(c["row_off"]).cuda(), draft=torch.from_numpy(c["draft"]).cuda(),
              draft_off=torch.from_numpy(c["draft_off"]).cuda(), want_lse=True)
    want = ab.argmax_batch(lg, **kw)
    torch.cuda.synchronize()
    # the plain entry point itself against the CPU checker
    xf = synth.bf16_bits_to_f32(c["logits"])
    sel = np.array([orc.argmax(r) for r in xf], np.int32)
    acc, nxt = orc.verify_greedy(sel, c["row_off"], c["draft"], c["draft_off"])
    assert np.array_equal(want["argmax"].cpu().numpy(), sel)
    assert np.array_equal(want["accepted"].cpu().numpy(), acc) and np.array_equal(want["next"].cpu().numpy(), nxt)
    for call in range(2):  # two calls in a row share the array
        got = ab.argmax_batch(lg, static_scratch=True, **kw)
        torch.cuda.synchronize()
        assert int(got["status"].item()) == 0
        for k in ("argmax", "accepted", "next"):
            assert torch.equal(got[k], want[k]), (call, k)
        assert torch.equal(got["max_sumexp"][:, 0], want["max_sumexp"][:, 0])
        torch.testing.assert_close(got["max_sumexp"][:, 1], want["max_sumexp"][:, 1], rtol=1e-6, atol=0)
        assert np.array_equal(got["argmax"].cpu().numpy(), sel)  # and against the CPU checker directly
        assert np.array_equal(got["accepted"].cpu().numpy(), acc) and np.array_equal(got["next"].cpu().numpy(), nxt)


def test_static_scratch_refuses_oversized_shapes():
    import ctypes as C

    import arcinfer_b200 as ab

    cap = ab.lib.arcs_argmax_static_scratch_bytes()
    R, V = 100000, 8192  # so many rows need more scratch than the fixed array holds
    assert ab.lib.arcs_argmax_workspace_bytes(R, V) > cap
    a = ab.capi.ArgmaxArgs()
    dummy = torch.zeros(8, device="cuda")  # never read: the call is refused before any launch
    a.logits, a.dtype, a.R, a.V, a.row_stride = dummy.data_ptr(), 0, R, V, V
    a.argmax = dummy.data_ptr()
    rc = ab.lib.arcs_argmax_batch_static(C.byref(a), None)
    assert rc == 3  # ARCS_ERR_WORKSPACE
    assert b"fixed array" in ab.lib.arcs_last_error()
