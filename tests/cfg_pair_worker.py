"""Child process of tests/test_cfg_pair_gpu.py: one rank of a guidance pair (run under torchrun, 2 GPUs)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))
from conftest import load_package  # noqa: E402


def rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / np.linalg.norm(b.astype(np.float64)))


def main():
    fx = load_package()
    import flux2_c_b200.dp as dp
    import flux2_c_b200.synth as synth
    from oracle import flux_oracle as fo
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = fx.Context(local)
    d = synth.Dims.tiny()
    W = synth.make_transformer_weights(d, seed=3, sharp=True, std=0.08)
    model = fx.Model.from_tensors(ctx, d, W)
    h, w, ntxt, steps, g = 6, 6, 48, 5, 4.0
    z0 = fx.init_noise(d.latent_ch, h, w, 7)
    cc = synth.make_context(41, ntxt, d.text_dim)
    cu = synth.make_context(42, ntxt, d.text_dim)
    sch = fx.official_schedule(steps, h * w)
    _, is_cond = dp.pair_of_rank(rank)
    group = dp.pair_groups(dist.get_world_size())

    mine = cc if is_cond else cu
    sampler = fx.Sampler(model, h, w, ntxt, batch=1, max_steps=steps)
    sampler.upload(z0.ctypes.data, mine.ctypes.data)
    v_buf = torch.zeros(z0.size, dtype=torch.float32, device="cuda")
    with torch.cuda.stream(torch.cuda.ExternalStream(ctx.stream)):
        dp.sample_cfg_pair(sampler, sch, g, is_cond, v_buf, group)
    got = np.empty_like(z0)
    sampler.download(got.ctypes.data)
    torch.cuda.synchronize()

    # both members of the pair must hold the same latent, bit for bit
    t = torch.from_numpy(got.copy()).cuda()
    other = [torch.empty_like(t) for _ in range(2)]
    dist.all_gather(other, t, group=group)
    assert torch.equal(other[0], other[1]), "pair latents diverged"

    if rank == 0:
        want = fo.OracleModel(W, d).sample_euler_cfg(z0, h, w, cc, cu, g, sch)
        one_gpu = model.sample(z0, h, w, cc, sch, ctx_uncond=cu, guidance=g)
        e_oracle, e_batch2 = rel(got, want), rel(got, one_gpu)
        assert e_oracle < 3e-2, e_oracle
        assert e_batch2 < 5e-3, e_batch2
        print("cfg pair ok: vs oracle %.2e, vs batch-2 on one GPU %.2e" % (e_oracle, e_batch2))
    sampler.close()
    model.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
