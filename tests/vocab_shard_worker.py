"""Worker of tests/test_gpu_vocab_shard.py::test_two_ranks_over_nccl (one process per GPU under
torchrun): every rank samples its columns, the packed records travel through one NCCL all-gather,
every rank merges, and rank 0 compares with the CPU oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import arcinfer_b200 as ab  # noqa: E402
from arcinfer_b200 import shard, synth  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    g = np.random.default_rng(900)  # the same inputs on every rank
    B, V, H = 16, 262144, 64
    x = (g.standard_normal((B, V), dtype=np.float32) * 3).astype(np.float32)
    xb = synth.f32_to_bf16_bits(x)
    params = synth.make_params(B, top_k=50, top_p=0.95, repeat_penalty=1.1, repeat_last_n=-1)
    hists = [g.integers(0, V, H).astype(np.int32) for _ in range(B)]
    us = g.random(B)
    lo, hi = shard.vocab_range(V, rank, world)
    local_logits = torch.from_numpy(np.ascontiguousarray(xb[:, lo:hi]).view(np.int16)).cuda().view(torch.bfloat16)
    ho, hi_ = synth.csr(hists)
    lists = dict(hist_off=torch.from_numpy(ho).cuda(), hist_ids=torch.from_numpy(hi_).cuda(), max_hist=H)
    p_dev = ab.capi.params_to_device(params, "cuda")
    u_dev = torch.from_numpy(us).cuda()
    out = shard.vocab_sharded_sample(local_logits, lo, V, p_dev, u_dev, dist.all_gather_into_tensor, world, ab.sample_batch, ab.merge_records, 50, **lists)
    torch.cuda.synchronize()
    tok = out["token"].cpu().numpy()
    step = shard.VocabShardStep(local_logits, lo, V, p_dev, u_dev, world, 50, want_mz=True, **lists)  # the prebuilt form, with the normaliser
    for _ in range(2):
        out2 = step.step(dist.all_gather_into_tensor)
    torch.cuda.synchronize()
    assert np.array_equal(out2["token"].cpu().numpy(), tok)
    mz = out2["mz"].cpu().numpy().astype(np.float64)
    if rank == 0:
        import orc

        xf = synth.bf16_bits_to_f32(xb)
        for b in range(B):
            want = orc.sample(xf[b], params[b : b + 1], hists[b], float(us[b]))
            assert tok[b] == want["token"], (b, tok[b], want["token"])
        xd = xf.astype(np.float64)
        m = xd.max(axis=1)
        assert np.abs(mz[:, 0] + np.log(mz[:, 1]) - (m + np.log(np.exp(xd - m[:, None]).sum(axis=1)))).max() < 1e-5
        print("VOCAB_SHARD_OK")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
