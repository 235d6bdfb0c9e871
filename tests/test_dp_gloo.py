"""Multi-rank host logic on CPU: world_size 2 (and 4) over gloo, spawned as child processes."""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, os.path.join(%r, "tests"))
    import numpy as np, torch, torch.distributed as dist
    from conftest import load_package
    load_package()
    import flux2_c_b200.dp as dp
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    # 1. data-parallel assignment: every image exactly once
    mine = dp.images_of_rank(11, rank, world)
    got = [None] * world
    dist.all_gather_object(got, mine)
    assert sorted(sum(got, [])) == list(range(11))
    assert max(len(g) for g in got) - min(len(g) for g in got) <= 1
    # 2. timing: max over ranks
    assert dp.max_over_ranks(10.0 + rank) == 10.0 + world - 1
    # 3. guidance pair: the pre-scaled all-reduce equals v_u + g (v_c - v_u), identically on both ranks
    pair, is_cond = dp.pair_of_rank(rank)
    group = dp.pair_groups(world)
    g = 4.0
    rng = np.random.default_rng(100 + pair)
    v_c = rng.standard_normal(4096).astype(np.float32)
    v_u = rng.standard_normal(4096).astype(np.float32)
    mine_v = torch.from_numpy((v_c if is_cond else v_u).copy()) * dp.guidance_coefficient(is_cond, g)
    out = dp.combine_pair(mine_v, group).numpy()
    want = v_u + np.float32(g) * (v_c - v_u)
    assert np.allclose(out, want, rtol=1e-5, atol=1e-5)
    both = [None] * world
    dist.all_gather_object(both, out.tobytes())
    assert both[2 * pair] == both[2 * pair + 1], "pair members must hold bit-identical velocities"
    # 4. a whole Euler loop of the pair with a stand-in sampler keeps the two latents identical
    class FakeSampler:
        def __init__(self, z, bias): self.z, self.bias, self.v = z.clone(), bias, None
        def predict(self, sched, i): self.v = torch.tanh(self.z * (1.0 + 0.1 * i)) + self.bias
        def velocity(self, ptr, scale): buf.copy_(self.v * scale)
        def apply_velocity(self, ptr, i): self.z += (sched[i + 1] - sched[i]) * buf
    z0 = torch.from_numpy(np.random.default_rng(7 + pair).standard_normal(256).astype(np.float32))
    buf = torch.zeros(256)
    sched = [1.0, 0.7, 0.3, 0.0]
    fs = FakeSampler(z0, 0.5 if is_cond else -0.25)
    dp.sample_cfg_pair(fs, sched, g, is_cond, buf, group)
    # serial restatement of the reference's CFG loop (flux_sample.c:485-499)
    z = z0.clone()
    for i in range(3):
        vu = torch.tanh(z * (1.0 + 0.1 * i)) - 0.25
        vc = torch.tanh(z * (1.0 + 0.1 * i)) + 0.5
        z = z + (sched[i + 1] - sched[i]) * (vu + g * (vc - vu))
    assert torch.allclose(fs.z, z, atol=1e-5)
    dist.barrier()
    dist.destroy_process_group()
    print("rank", rank, "ok")
""") % ROOT


@pytest.mark.parametrize("world", [2, 4])
def test_multi_rank_host_logic_gloo(tmp_path, world):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(29500 + world + os.getpid() % 500), str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ok") == world
