"""GPU parity for sample_batch through the C ABI against the CPU oracle: token ids, candidate
lists, counts and adjusted logits bit-exact; probabilities within 1e-6 relative."""
import numpy as np
import pytest

import orc
from arcinfer_b200 import synth
from cases import rand_logits, rand_mask, rand_params, rand_recent

pytestmark = pytest.mark.gpu


def _batch(g, B, V, pen, modes, masked=False, allow_k0=True):
    x = np.stack([rand_logits(g, V, modes[b % len(modes)]) for b in range(B)])
    ps, biases, hists = [], [], []
    for b in range(B):
        p, bias = rand_params(g, V, pen, allow_k0=allow_k0)
        if masked and p["top_k"][0] > 256:
            p["top_k"] = 40
        ps.append(p)
        biases.append(bias)
        hists.append(rand_recent(g, V))
    params = np.concatenate(ps)
    us = g.random(B)
    masks = None
    if masked:
        masks = np.stack([rand_mask(g, V, float(g.choice([1.0, 0.5, 0.05, 0.005, 0.001, 0.0]))) for _ in range(B)])
    return x, params, hists, us, biases, masks


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("pen", [False, True])
def test_sample_random_battery(bf16, pen):
    from gpuutil import check_rows, run_gpu_sample

    g = np.random.default_rng(100 + 2 * bf16 + pen)
    for V, B in [(2, 3), (33, 4), (257, 5), (1000, 8), (4099, 6), (8192, 4), (20000, 6), (151936, 3), (262144, 2)]:
        x, params, hists, us, biases, _ = _batch(g, B, V, pen, [0, 1, 2])
        xb = synth.f32_to_bf16_bits(x) if bf16 else x
        for stride, off in [(None, 0), (V + 5, 3)]:
            out = run_gpu_sample(xb, bf16, params, hists, us, biases, stride=stride, offset=off)
            check_rows(out, xb, bf16, params, hists, us, biases, tag=f"stride={stride} off={off}")


@pytest.mark.parametrize("bf16", [False, True])
def test_sample_allowed_random_battery(bf16):
    from gpuutil import check_rows, run_gpu_sample

    g = np.random.default_rng(200 + bf16)
    for V, B in [(1, 2), (40, 4), (600, 6), (5000, 8), (20000, 8), (151936, 4)]:
        for pen in (False, True):
            x, params, hists, us, biases, masks = _batch(g, B, V, pen, [0, 1, 2], masked=True)
            xb = synth.f32_to_bf16_bits(x) if bf16 else x
            out = run_gpu_sample(xb, bf16, params, hists, us, biases, masks=masks)
            check_rows(out, xb, bf16, params, hists, us, biases, masks=masks)


def test_many_rows_one_segment():
    """enough rows that every row is one segment (no merge), with long histories"""
    from gpuutil import check_rows, run_gpu_sample

    g = np.random.default_rng(300)
    B, V = 700, 12000
    x = (g.standard_normal((B, V), dtype=np.float32) * 3).astype(np.float32)
    xb = synth.f32_to_bf16_bits(x)
    params = synth.make_params(B, top_k=50, top_p=0.95, repeat_penalty=1.1, repeat_last_n=-1)
    hists = [g.integers(0, V, 512).astype(np.int32) for _ in range(B)]
    us = g.random(B)
    out = run_gpu_sample(xb, True, params, hists, us)
    check_rows(out, xb, True, params, hists, us, rows=range(0, B, 9))


@pytest.mark.parametrize("masked", [False, True])
def test_ascending_rows_overflow_the_lists(masked):
    """ascending logits make every element a survivor of the stream: the per-item lists overflow
    and the rows are read again by the finishing step; same results as ever"""
    from gpuutil import check_rows, run_gpu_sample

    g = np.random.default_rng(310 + masked)
    B, V = 5, 40000
    x = np.sort((g.standard_normal((B, V), dtype=np.float32) * 3).astype(np.float32), axis=1)
    x[1] = x[1, ::-1]  # one descending row: nothing after the first elements survives
    x[2, ::7] = x[2, 5]  # and one with masses of equal values
    ps, biases, hists = [], [], []
    for b in range(B):
        p, bias = rand_params(g, V, True, allow_k0=not masked)
        if masked and p["top_k"][0] > 256:
            p["top_k"] = 40
        ps.append(p)
        biases.append(bias)
        hists.append(np.concatenate([g.integers(0, V, 60), np.arange(V - 40, V)]).astype(np.int32))  # the best tokens are penalised
    params = np.concatenate(ps)
    us = g.random(B)
    masks = np.stack([rand_mask(g, V, d) for d in (1.0, 0.5, 0.05, 0.5, 0.001)]) if masked else None
    for bf16 in (False, True):
        xb = synth.f32_to_bf16_bits(x) if bf16 else x
        out = run_gpu_sample(xb, bf16, params, hists, us, biases, masks=masks)
        check_rows(out, xb, bf16, params, hists, us, biases, masks=masks)


def test_reference_property_cases():
    """the reference's own property tests (tests/test_sampler.cpp:215-301 there): presence penalty in
    greedy mode, bans by logit_bias <= -100, nothing allowed -> -1"""
    from gpuutil import run_gpu_sample

    l = np.zeros((1, 100), np.float32)
    l[0, :3] = [5.0, 4.9, 4.0]
    pg = synth.make_params(1, temperature=0.0, presence_penalty=0.5)
    one = lambda x, p, h, bias=None, mask=None: int(run_gpu_sample(x, False, p, [np.array(h, np.int32)], [0.5], [bias or []], masks=mask)["token"][0])
    assert one(l, pg, [0, 0, 7]) == 1
    assert one(l, pg, [0, 0, 0, 1]) == 0
    assert one(l, pg, [3]) == 0
    assert one(l, synth.make_params(1, temperature=0.0, presence_penalty=-2.0), [2]) == 2
    g = np.random.default_rng(5)
    x = (g.standard_normal((1, 1000), dtype=np.float32) * 3).astype(np.float32)
    x[0, 3] = 1000.0
    ban = [(3, -100.0)]
    p0 = synth.make_params(1, temperature=0.0)
    assert one(x, p0, [], ban) != 3
    m37 = np.zeros((1, 32), np.uint32)
    m37[0, 0] = (1 << 3) | (1 << 7)
    assert one(x, p0, [], ban, m37) == 7
    m3 = np.zeros((1, 32), np.uint32)
    m3[0, 0] = 1 << 3
    assert one(x, p0, [], ban, m3) == -1
    assert one(x, synth.make_params(1, temperature=0.0, presence_penalty=-5000.0), [3], [(3, -250.0)]) != 3
    # most of the vocabulary banned: banned tokens reach the top k, still never drawn
    x2 = (g.standard_normal((1, 300), dtype=np.float32) * 3).astype(np.float32)
    q = synth.make_params(1, temperature=1.5, top_k=20, top_p=1.0)
    bans = [(t, -100.0) for t in range(290)]
    for u in np.linspace(0, 0.999999, 50):
        assert int(run_gpu_sample(x2, False, q, [np.zeros(0, np.int32)], [u], [bans])["token"][0]) >= 290


def test_error_paths():
    import torch

    import arcinfer_b200 as ab

    lg = torch.zeros(2, 1000, device="cuda")
    p = ab.capi.params_to_device(synth.make_params(2, top_k=5000), "cuda")
    u = torch.zeros(2, dtype=torch.float64, device="cuda")
    out = ab.sample_batch(lg, p, u)
    torch.cuda.synchronize()
    # top_k is clipped to V = 1000, still above the 256-candidate cap: reported, no token chosen
    assert int(out["status"][0].item()) == 2
    assert out["token"].tolist() == [-1, -1]
    with pytest.raises(ab.ArcsError):
        ab.sample_batch(lg, p, u, V=0)
