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


# ------------------------------------------------------------------------------------------------ observers, ownership
def _mapped(path):
    with open("/proc/self/maps") as f:
        return any(line.rstrip().endswith(path) for line in f)


def test_seam_callbacks_fire_in_the_reference_order(seam, scratch, fx, capfd):
    """What the reference's CLI installs unless it is told to be quiet (main.c:147-154): the step callback before a
    step, one sub-step event per double block, single block and final layer, the progress callback after the step, the
    step-image callback with a decoded picture after every step but the last (flux_sample.c:229-266,
    flux_transformer.c:3253, 3488, 3566). The observed loop runs step by step; its latent must be the one the
    unobserved loop (a single CUDA-graph replay) produces. With flux_verbose the per-group timing globals are filled."""
    import ctypes
    import flux2_c_b200.synth as synth
    from oracle import ref_binding as rb
    L = seam.L
    d = synth.Dims.tiny()
    W = synth.make_transformer_weights(d, seed=3, sharp=True, std=0.08)
    path = os.path.join(scratch, "tiny_cb.safetensors")
    synth.write_safetensors(path, W)
    vpath = os.path.join(scratch, "vae_cb.safetensors")
    synth.write_safetensors(vpath, synth.make_vae_weights(seed=5, rich=True), dtype="F32")
    tf = seam.load_transformer(path)
    vae = seam.load_vae(vpath)
    events = []
    STEP = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_int)
    SUB = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_int, ctypes.c_int)
    IMG = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_int, ctypes.POINTER(rb.FluxImage))
    step_cb = STEP(lambda s, n: events.append(("step", s, n)))
    sub_cb = SUB(lambda t, i, n: events.append(("sub", t, i, n)))
    prog_cb = STEP(lambda s, n: events.append(("progress", s, n)))
    img_cb = IMG(lambda s, n, im: events.append(("image", s, n, im.contents.width, im.contents.height)))

    def slot(name):
        return ctypes.c_void_p.in_dll(L, name)

    h, w, steps = 4, 3, 3
    z = synth.make_latent(1, d.latent_ch, h, w)
    c = synth.make_context(2, 24, d.text_dim)
    sch = np.ascontiguousarray(fx.official_schedule(steps, h * w), dtype=np.float32)
    fp = ctypes.POINTER(ctypes.c_float)

    def run(progress):
        zz, cc = z.copy(), c.copy()
        p = L.flux_sample_euler(tf.h, None, zz.ctypes.data_as(fp), 1, d.latent_ch, h, w, cc.ctypes.data_as(fp),
                                cc.shape[0], sch.ctypes.data_as(fp), steps, progress)
        return seam._take(p, z.size).reshape(z.shape)

    quiet = run(None)  # nobody observes: one graph replay on the device
    assert events == []
    verbose = ctypes.c_int.in_dll(L, "flux_verbose")
    try:
        slot("flux_step_callback").value = ctypes.cast(step_cb, ctypes.c_void_p).value
        slot("flux_substep_callback").value = ctypes.cast(sub_cb, ctypes.c_void_p).value
        slot("flux_step_image_callback").value = ctypes.cast(img_cb, ctypes.c_void_p).value
        slot("flux_step_image_vae").value = vae
        verbose.value = 1
        observed = run(ctypes.cast(prog_cb, ctypes.c_void_p))
    finally:
        for name in ("flux_step_callback", "flux_substep_callback", "flux_step_image_callback", "flux_step_image_vae"):
            slot(name).value = None
        verbose.value = 0
    want = []
    for s in range(1, steps + 1):
        want.append(("step", s, steps))
        want += [("sub", 0, i, d.n_double) for i in range(d.n_double)]
        want += [("sub", 1, i, d.n_single) for i in range(d.n_single)]
        want.append(("sub", 2, 0, 1))
        want.append(("progress", s, steps))
        if s < steps:
            want.append(("image", s, steps, 16 * w, 16 * h))
    assert events == want
    assert np.array_equal(observed, quiet)
    err = capfd.readouterr().err
    assert "Denoising timing breakdown" in err and "Step 3:" in err and "Double blocks:" in err
    dbl = ctypes.c_double.in_dll(L, "flux_timing_transformer_double").value
    sgl = ctypes.c_double.in_dll(L, "flux_timing_transformer_single").value
    fin = ctypes.c_double.in_dll(L, "flux_timing_transformer_final").value
    tot = ctypes.c_double.in_dll(L, "flux_timing_transformer_total").value
    assert dbl > 0 and sgl > 0 and fin > 0 and dbl + sgl + fin <= tot
    # the single forward fires its sub-step events too (flux_denoise_step, flux.c:1109-1122)
    events.clear()
    try:
        slot("flux_substep_callback").value = ctypes.cast(sub_cb, ctypes.c_void_p).value
        tf.forward(z, h, w, c, 0.5)
    finally:
        slot("flux_substep_callback").value = None
    assert len(events) == d.n_double + d.n_single + 1
    tf.close()
    seam.L.flux_vae_free(vae)


def test_seam_mmap_loader_owns_the_file(seam, scratch, fx):
    """flux_transformer_load_safetensors_mmap takes the open file over and flux_transformer_free closes it
    (flux.c:310-313, flux_transformer.c:4306-4309); the plain loader leaves it to the caller (flux.c:315-316). This is
    the loader the reference's CLI uses by default (main.c:304, 429-432)."""
    import ctypes
    import flux2_c_b200.synth as synth
    L = seam.L
    L.flux_transformer_load_safetensors_mmap.restype = ctypes.c_void_p
    L.flux_transformer_load_safetensors_mmap.argtypes = [ctypes.c_void_p]
    d = synth.Dims.tiny()
    W = synth.make_transformer_weights(d, seed=3, sharp=True, std=0.08)
    path = os.path.join(scratch, "tiny_mmap.safetensors")
    synth.write_safetensors(path, W)
    z = synth.make_latent(1, d.latent_ch, 4, 4)
    c = synth.make_context(2, 16, d.text_dim)

    sf = L.safetensors_open(path.encode())
    assert sf and _mapped(path)
    h = L.flux_transformer_load_safetensors_mmap(sf)
    assert h
    from oracle import ref_binding as rb
    tf = rb.RefTransformer(seam, h)
    v_mmap = tf.forward(z, 4, 4, c, 0.6)
    assert _mapped(path)      # still the transformer's
    tf.close()                # flux_transformer_free
    assert not _mapped(path)  # ... which closed it

    sf = L.safetensors_open(path.encode())
    tf2 = rb.RefTransformer(seam, L.flux_transformer_load_safetensors(sf))
    L.safetensors_close(sf)   # the caller's to close, right after loading; the weights are resident
    assert not _mapped(path)
    assert np.array_equal(tf2.forward(z, 4, 4, c, 0.6), v_mmap)
    tf2.close()
    L.flux_transformer_free(None)  # NULL-safe


def test_seam_unused_sampler_exports_match_reference(seam, scratch, fx):
    """The exports nothing in the reference calls - flux_sample_heun, flux_sample_euler_ancestral,
    flux_generate_latent, flux_sigmoid_schedule, flux_resolution_schedule (flux_sample.c:75-116, 697-821, 891-919) -
    against the reference's own outputs at the klein shape (4 x 4 latent, 32 text tokens)."""
    import flux2_c_b200.synth as synth
    path = os.path.join(GOLDEN, "reference_samplers.npz")
    if not os.path.exists(path):
        pytest.skip("reference_samplers.npz missing")
    g = np.load(path)
    for key in g.files:
        if key.startswith("sigmoid_"):
            _, n, shift = key.split("_")
            assert np.allclose(seam.sigmoid_schedule(int(n), float(shift)), g[key], atol=2e-6), key
        elif key.startswith("resolution_"):
            _, n, hh, ww = key.split("_")
            assert np.allclose(seam.resolution_schedule(int(n), int(hh), int(ww)), g[key], atol=2e-6), key
    d = synth.Dims.klein4b()
    wpath = os.path.join(scratch, "klein_sharp.safetensors")
    synth.write_safetensors(wpath, synth.make_transformer_weights(d, seed=0, sharp=True, threads=os.cpu_count()))
    tf = seam.load_transformer(wpath)
    os.remove(wpath)
    try:
        h = w = 4
        z0 = fx.init_noise(128, h, w, 42)
        c = synth.make_context(1234, 32, d.text_dim)
        sch = g["sched"]
        assert rel(tf.sample_euler(z0, h, w, c, sch), g["euler_final"]) < LATENT_TOL
        assert rel(tf.sample_heun(z0, h, w, c, sch), g["heun_final"]) < LATENT_TOL
        assert rel(tf.sample_euler_ancestral(z0, h, w, c, sch, 0.0, 777), g["ancestral_eta0_final"]) < LATENT_TOL
        got = tf.sample_euler_ancestral(z0, h, w, c, sch, 0.5, 777)
        assert rel(got, g["ancestral_final"]) < LATENT_TOL
        # the injected noise is part of the result: another seed of the library's generator must move it
        assert rel(tf.sample_euler_ancestral(z0, h, w, c, sch, 0.5, 778), g["ancestral_final"]) > 5 * LATENT_TOL
        assert rel(tf.generate_latent(c, 64, 64, 2, 5), g["generate_final"]) < LATENT_TOL
    finally:
        tf.close()
