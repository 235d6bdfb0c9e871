"""The reference's own library with its transformer, sampler and text-encoder files replaced by the engine's seam
(oracle/_ref/libflux_seam.so, built by `make -C oracle cli`), called in-process through the very binding the tests
use for the reference build: same symbols, same arguments, malloc-owned results. Checked against the numpy oracle
(tiny DiT) and against the reference's stored output (text encoder at the Qwen3-4B shape, loaded from a two-shard
model directory)."""
import os
import shutil
import tempfile

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
VEL_TOL, LATENT_TOL, TEXT_TOL = 2e-2, 3e-2, 2e-2


def rel(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))


@pytest.fixture(scope="module")
def seam(fx, ctx):
    from oracle import ref_binding as rb
    if not rb.available("seam"):
        pytest.skip("oracle/_ref/libflux_seam.so is not built")
    return rb.RefLib("seam")


@pytest.fixture(scope="module")
def scratch():
    base = "/dev/shm" if os.path.isdir("/dev/shm") and os.access("/dev/shm", os.W_OK) else None
    d = tempfile.mkdtemp(prefix="flux_seam_", dir=base)
    yield d
    shutil.rmtree(d, ignore_errors=True)


def test_seam_transformer_and_samplers_match_oracle(seam, scratch, fx):
    import flux2_c_b200.synth as synth
    from oracle import flux_oracle as fo
    d = synth.Dims.tiny()
    W = synth.make_transformer_weights(d, seed=3, sharp=True, std=0.08)
    path = os.path.join(scratch, "tiny_dit.safetensors")
    synth.write_safetensors(path, W)
    om = fo.OracleModel(W, d)
    tf = seam.load_transformer(path)
    try:
        h, w = 6, 4
        z = synth.make_latent(1, d.latent_ch, h, w)
        c = synth.make_context(2, 24, d.text_dim)
        cu = synth.make_context(3, 24, d.text_dim)
        r1 = synth.make_latent(4, d.latent_ch, 2, 4)
        z_before = z.copy()
        assert rel(tf.forward(z, h, w, c, 0.7), om.forward(z, h, w, c, 0.7)) < VEL_TOL
        assert rel(tf.forward(z, h, w, c, 0.4, refs=[(r1, 10)]), om.forward(z, h, w, c, 0.4, refs=[(r1, 10)])) < VEL_TOL
        sch = fx.official_schedule(4, h * w)
        assert rel(tf.sample_euler(z, h, w, c, sch), om.sample_euler(z, h, w, c, sch)) < LATENT_TOL
        assert rel(tf.sample_euler(z, h, w, c, sch, refs=[(r1, 10)]),
                   om.sample_euler(z, h, w, c, sch, refs=[(r1, 10)])) < LATENT_TOL
        assert rel(tf.sample_euler_cfg(z, h, w, c, cu, 3.0, sch),
                   om.sample_euler_cfg(z, h, w, c, cu, 3.0, sch)) < LATENT_TOL
        assert np.array_equal(z, z_before)  # inputs are borrowed, never modified
    finally:
        tf.close()


def test_seam_text_encoder_loads_shards_and_matches_reference(seam, scratch):
    """qwen3_model_load on a directory with the two shards, qwen3_forward on 64 tokens (40 valid) against the output the
    reference produced from the same tensors. Only layers 0..26 are written here: the output does not depend on the
    rest, and the engine's loader does not ask for them."""
    import flux2_c_b200.synth as synth
    path = os.path.join(GOLDEN, "reference_qwen3.npz")
    if not os.path.exists(path):
        pytest.skip("reference_qwen3.npz missing")
    g = np.load(path)
    d = synth.QwenDims.qwen3_4b()
    mdir = os.path.join(scratch, "text_encoder")
    W = synth.make_qwen_weights(d, seed=0, threads=os.cpu_count(), max_layer=26)
    synth.write_qwen_shards(mdir, W)
    del W
    m = seam.qwen3_load(mdir)
    try:
        shutil.rmtree(mdir, ignore_errors=True)  # weights are resident: the files are not needed any more
        out = seam.qwen3_forward(m, g["ids"], g["mask"])
        assert out.shape == (64, 7680)
        assert rel(out[:, ::4], g["out_sub"]) < TEXT_TOL
    finally:
        seam.L.qwen3_model_free(m)
    with pytest.raises(RuntimeError):
        seam.qwen3_load(os.path.join(scratch, "no_such_dir"))


def test_seam_vae_decode_is_served_by_the_engine(seam, scratch, fx, ctx):
    """flux_vae_load_safetensors / flux_vae_decode as the library's own callers reach them (redirected at link time):
    the image must match the CPU restatement of the reference's decoder, and be the engine's own result bit for bit."""
    import flux2_c_b200.synth as synth
    from oracle.vae_oracle import VaeOracle
    W = synth.make_vae_weights(seed=5, rich=True)
    path = os.path.join(scratch, "vae.safetensors")
    synth.write_safetensors(path, W, dtype="F32")
    vae = seam.load_vae(path)
    try:
        lat = synth.make_latent(11, 128, 6, 5)
        got = seam.vae_decode(vae, lat)
        want, _ = VaeOracle(W).decode(lat)
        mse = float(((got.astype(np.float64) - want.astype(np.float64)) ** 2).mean())
        assert 10.0 * np.log10(255.0 ** 2 / max(mse, 1e-12)) >= 40.0
        direct = fx.Vae.from_tensors(ctx, W)
        assert np.array_equal(direct.decode(lat), got)
        direct.close()
    finally:
        seam.L.flux_vae_free(vae)


def test_seam_vae_encode_is_served_by_the_engine(seam, scratch):
    import flux2_c_b200.synth as synth
    from oracle.vae_oracle import VaeOracle
    W = synth.make_vae_weights(seed=5, rich=True)
    path = os.path.join(scratch, "vae_enc.safetensors")
    synth.write_safetensors(path, W, dtype="F32")
    vae = seam.load_vae(path)
    try:
        img = np.random.default_rng(2).uniform(-1.0, 1.0, (3, 64, 48)).astype(np.float32)
        got = seam.vae_encode(vae, img)
        assert got.shape == (128, 4, 3)
        assert rel(got, VaeOracle(W).encode(img)) < 1e-2
    finally:
        seam.L.flux_vae_free(vae)
