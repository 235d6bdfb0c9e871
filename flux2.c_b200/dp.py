"""Multi-GPU host logic: one process per GPU, `torch.distributed` for the plumbing.

The denoising path shards in two ways only (the reference itself is single-device and runs one image at a time):

* independent images (seeds / prompts): every rank holds a full replica and denoises its own share; there is
  no collective on the data path, results are gathered on the host;
* the base model's guidance pair: the conditional and the unconditional pass of one image run on two GPUs and
  exchange ONE velocity per step (a 2-rank sum of `latent_ch * h * w` floats).

Everything here works on any backend (`nccl` on GPUs, `gloo` on CPU for tests).
"""
import torch
import torch.distributed as dist


def images_of_rank(num_images, rank, world):
    """Round-robin assignment: image i goes to rank i % world. Returns the list of image indices of `rank`."""
    return list(range(rank, num_images, world))


def max_over_ranks(value, device="cpu"):
    """Every rank gets the maximum of `value` (a per-rank duration): multi-GPU time is the slowest rank's."""
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def pair_of_rank(rank):
    """Ranks (0,1), (2,3), ... form guidance pairs; the even rank runs the conditional pass. Every GPU is
    equidistant through NVSwitch, so the pairing is arbitrary."""
    return rank // 2, rank % 2 == 0


def pair_groups(world):
    """One process group per pair; every rank must call this (new_group is collective). Returns this rank's group."""
    mine = None
    for p in range(world // 2):
        g = dist.new_group(ranks=[2 * p, 2 * p + 1])
        if dist.get_rank() // 2 == p:
            mine = g
    return mine


def guidance_coefficient(is_conditional, guidance):
    """v = v_u + g (v_c - v_u) = g * v_c + (1 - g) * v_u: each rank pre-scales its own velocity."""
    return float(guidance) if is_conditional else 1.0 - float(guidance)


def combine_pair(scaled_velocity, group=None):
    """In-place sum of the two pre-scaled velocities across the pair. A two-term sum is order-independent, so both
    ranks obtain bit-identical results and their latents never diverge."""
    dist.all_reduce(scaled_velocity, op=dist.ReduceOp.SUM, group=group)
    return scaled_velocity


def sample_cfg_pair(sampler, schedule, guidance, is_conditional, v_buf, group=None):
    """Euler loop of one member of a guidance pair. `sampler` is a batch-1 Sampler with this rank's context
    uploaded; `v_buf` a float32 CUDA tensor of latent size; torch's current stream must be the engine's stream
    (torch.cuda.ExternalStream(ctx.stream)) so that the exchange is ordered with the kernels without host syncs."""
    coef = guidance_coefficient(is_conditional, guidance)
    for i in range(len(schedule) - 1):
        sampler.predict(schedule, i)
        sampler.velocity(v_buf.data_ptr(), coef)
        combine_pair(v_buf, group)
        sampler.apply_velocity(v_buf.data_ptr(), i)
