"""flux_cuda_group_*: several GPUs of one machine behind the C ABI, driven from one process. On a one-GPU box the
group of one is checked against the single-context path and the pair call must refuse; with two or more GPUs the
guidance pair split over two GPUs is checked against the batch-of-two path on one GPU and against the numpy oracle,
and independent images are spread over the members."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
LATENT_TOL = 3e-2


def rel(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))


def _gpus():
    import torch
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.fixture(scope="module")
def tiny_group(fx):
    import flux2_c_b200.synth as synth
    n = min(_gpus(), 2)
    if n < 1:
        pytest.skip("no GPU")
    d = synth.Dims.tiny()
    W = synth.make_transformer_weights(d, seed=3, sharp=True, std=0.08)
    g = fx.Group(range(n))
    models = [fx.Model.from_tensors(g.context(r), d, W) for r in range(n)]
    g.set_models(models)
    yield synth, d, W, g, models, n
    for m in models:
        m.close()
    g.close()


def test_group_batch_spreads_independent_images(tiny_group, fx):
    synth, d, W, g, models, n = tiny_group
    h, w, ntxt, steps = 6, 4, 24, 3
    sch = fx.official_schedule(steps, h * w)
    z0s = [fx.init_noise(d.latent_ch, h, w, i) for i in range(5)]
    cs = [synth.make_context(10000 + i, ntxt, d.text_dim) for i in range(5)]
    outs = g.sample_batch(z0s, cs, h, w, sch)
    for i in range(5):  # whichever member ran image i, the result is the single-context one, bit for bit
        assert np.array_equal(outs[i], models[0].sample(z0s[i], h, w, cs[i], sch))
    assert not np.array_equal(outs[0], outs[1])
    assert g.sample_batch([], [], h, w, sch) == []
    r1 = [(synth.make_latent(4, d.latent_ch, 2, 4), 10)]
    outs = g.sample_batch(z0s[:2], cs[:2], h, w, sch, refs=r1)
    assert np.array_equal(outs[1], models[0].sample(z0s[1], h, w, cs[1], sch, refs=r1))


def test_group_pair_needs_two_gpus_or_matches_batch_of_two(tiny_group, fx):
    from oracle import flux_oracle as fo
    synth, d, W, g, models, n = tiny_group
    h, w, ntxt, steps, guidance = 6, 6, 48, 5, 4.0
    z0 = fx.init_noise(d.latent_ch, h, w, 7)
    cc = synth.make_context(41, ntxt, d.text_dim)
    cu = synth.make_context(42, ntxt, d.text_dim)
    sch = fx.official_schedule(steps, h * w)
    if n < 2:
        with pytest.raises(fx.FluxCudaError, match="two GPUs"):
            g.sample_cfg_pair(z0, h, w, cc, cu, guidance, sch)
        return
    one_gpu = models[0].sample(z0, h, w, cc, sch, ctx_uncond=cu, guidance=guidance)
    for _ in range(3):  # several images through the same group: the flags only grow, nothing is reset in between
        pair = g.sample_cfg_pair(z0, h, w, cc, cu, guidance, sch)
        # same math; the batch of two rounds g (v_c - v_u) differently, and guidance 4 multiplies the f16 rounding of
        # either pass by up to 7 at every step: 2.6e-3 measured with references, 1.2e-3 at the 512x512 50-step shape
        assert rel(pair, one_gpu) < 5e-3
    want = fo.OracleModel(W, d).sample_euler_cfg(z0, h, w, cc, cu, guidance, sch)
    assert rel(pair, want) < LATENT_TOL
    r1 = [(synth.make_latent(4, d.latent_ch, 3, 4), 10)]
    assert rel(g.sample_cfg_pair(z0, h, w, cc, cu, guidance, sch, refs=r1),
               models[0].sample(z0, h, w, cc, sch, ctx_uncond=cu, guidance=guidance, refs=r1)) < 5e-3
    # guidance 1 needs no partner's half at all, yet takes the same path: (1 - g) = 0 on the unconditional side
    assert rel(g.sample_cfg_pair(z0, h, w, cc, cu, 1.0, sch), models[0].sample(z0, h, w, cc, sch)) < 1e-3


def test_group_rejects_bad_arguments(tiny_group, fx):
    synth, d, W, g, models, n = tiny_group
    with pytest.raises(fx.FluxCudaError):
        fx.Group([0, 0])
    with pytest.raises(fx.FluxCudaError):
        fx.Group([_gpus() + 3])
    other = fx.Context(0)
    try:
        stray = fx.Model.from_tensors(other, d, W)
        with pytest.raises(fx.FluxCudaError, match="not created from the group"):
            g.set_models([stray] * n)
        stray.close()
    finally:
        other.close()
    g.set_models(models)


_SEAM_PAIR_SCRIPT = r"""
import os, sys
import numpy as np
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
from conftest import load_package
fx = load_package()
import flux2_c_b200.synth as synth
from oracle import ref_binding as rb
seam = rb.RefLib("seam")
d = synth.Dims.tiny()
tf = seam.load_transformer(sys.argv[2])
h, w = 6, 4
z = synth.make_latent(1, d.latent_ch, h, w)
c = synth.make_context(2, 24, d.text_dim)
cu = synth.make_context(3, 24, d.text_dim)
sch = fx.official_schedule(4, h * w)
out = tf.sample_euler_cfg(z, h, w, c, cu, 3.0, sch)
plain = tf.sample_euler(z, h, w, c, sch)
np.savez(sys.argv[3], cfg=out, plain=plain)
tf.close()
"""


def test_seam_splits_guided_sampling_over_two_gpus(fx, tmp_path):
    """FLUX_CUDA_DEVICES=0,1 makes the reference's flux_sample_euler_cfg (served by the seam) run its two passes on two
    GPUs; the result must be the one the same call gives on one GPU, and unguided sampling is unaffected."""
    import subprocess
    import sys
    import flux2_c_b200.synth as synth
    from oracle import ref_binding as rb
    if _gpus() < 2:
        pytest.skip("needs 2 GPUs")
    if not rb.available("seam"):
        pytest.skip("oracle/_ref/libflux_seam.so is not built")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    d = synth.Dims.tiny()
    wpath = str(tmp_path / "tiny.safetensors")
    synth.write_safetensors(wpath, synth.make_transformer_weights(d, seed=3, sharp=True, std=0.08))
    outs = {}
    for tag, env in (("one", {}), ("two", {"FLUX_CUDA_DEVICES": "0,1"})):
        out = str(tmp_path / (tag + ".npz"))
        r = subprocess.run([sys.executable, "-c", _SEAM_PAIR_SCRIPT, root, wpath, out], capture_output=True, text=True,
                           env=dict(os.environ, **env), timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
        outs[tag] = np.load(out)
    assert rel(outs["two"]["cfg"], outs["one"]["cfg"]) < 5e-3
    assert np.array_equal(outs["two"]["plain"], outs["one"]["plain"])
