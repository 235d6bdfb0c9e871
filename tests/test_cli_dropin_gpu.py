"""Drop-in check through the reference's own, unmodified CLI.

oracle/Makefile (`make cli`) links the reference's main.c / flux.c / flux_cli.c / flux_vae.c / ... twice: once as the
plain reference (`flux_ref_cli`, BLAS build) and once with flux_transformer.c + flux_sample.c replaced by the seam
(`flux_cuda_cli`, which calls libflux_cuda.so; flux_qwen3.c is replaced too and the VAE's functions are redirected).
Both are run on the same synthetic model directory, first with external embeddings and noise, then from a text
prompt (tokenizer -> text encoder -> denoising -> VAE -> PNG) and from a prompt plus an input image (img2img: VAE
encoder -> reference tokens); the decoded PNGs must agree to PSNR >= 30 dB.
"""
import os
import subprocess
import zlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")


def read_png_rgb(path):
    """Minimal PNG reader for 8-bit RGB / RGBA, non-interlaced files (what the reference's writer emits)."""
    data = open(path, "rb").read()
    assert data[:8] == b"\x89PNG\r\n\x1a\n"
    pos, idat, w = 8, b"", None
    while pos < len(data):
        n = int.from_bytes(data[pos:pos + 4], "big")
        kind = data[pos + 4:pos + 8]
        body = data[pos + 8:pos + 8 + n]
        if kind == b"IHDR":
            w, h = int.from_bytes(body[:4], "big"), int.from_bytes(body[4:8], "big")
            depth, ctype, interlace = body[8], body[9], body[12]
            assert depth == 8 and ctype in (2, 6) and interlace == 0
            ch = 3 if ctype == 2 else 4
        elif kind == b"IDAT":
            idat += body
        pos += 12 + n
    raw = np.frombuffer(zlib.decompress(idat), dtype=np.uint8).reshape(h, 1 + w * ch)
    out = np.zeros((h, w * ch), dtype=np.int32)
    prev = np.zeros(w * ch, dtype=np.int32)
    for y in range(h):
        f, line = int(raw[y, 0]), raw[y, 1:].astype(np.int32)
        cur = np.zeros(w * ch, dtype=np.int32)
        if f == 0:
            cur = line
        elif f == 2:
            cur = (line + prev) & 255
        else:
            for x in range(w * ch):
                a = cur[x - ch] if x >= ch else 0
                b = prev[x]
                c = prev[x - ch] if x >= ch else 0
                if f == 1:
                    p = a
                elif f == 3:
                    p = (a + b) // 2
                else:
                    pa, pb, pc = abs(b - c), abs(a - c), abs(a + b - 2 * c)
                    p = a if (pa <= pb and pa <= pc) else (b if pb <= pc else c)
                cur[x] = (line[x] + p) & 255
        out[y] = cur
        prev = cur
    return out.reshape(h, w, ch)[:, :, :3].astype(np.float64)


@pytest.fixture(scope="module")
def model_dir(fx, tmp_path_factory):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    if not (os.path.exists(os.path.join(REF, "flux_cuda_cli")) and os.path.exists(os.path.join(REF, "flux_ref_cli"))):
        pytest.skip("oracle/_ref CLIs not built (make -C oracle cli)")
    import shutil
    import flux2_c_b200.synth as synth
    base = "/dev/shm" if os.access("/dev/shm", os.W_OK) else str(tmp_path_factory.mktemp("model"))
    mdir = os.path.join(base, "flux_synth_model_%d" % os.getpid())
    try:
        d = synth.Dims.klein4b()
        synth.write_safetensors(os.path.join(_mk(mdir, "transformer"), "diffusion_pytorch_model.safetensors"),
                                synth.make_transformer_weights(d, seed=0, threads=os.cpu_count()))
        synth.write_safetensors(os.path.join(_mk(mdir, "vae"), "diffusion_pytorch_model.safetensors"),
                                synth.make_vae_weights(), dtype="F32")
        open(os.path.join(mdir, "model_index.json"), "w").write('{"_class_name": "Flux2KleinPipeline", "is_distilled": true}')
        yield synth, d, mdir
    finally:
        shutil.rmtree(mdir, ignore_errors=True)


def _mk(*parts):
    p = os.path.join(*parts)
    os.makedirs(p, exist_ok=True)
    return p


def _run_both(args, tmp_path, tag, cuda_flags=("-q", "--no-mmap"), stderr_of=None):
    # the reference's BLAS build needs the OpenBLAS (and its libgfortran / libquadmath) bundled in the image's wheels
    site = os.path.dirname(os.path.dirname(np.__file__))
    libs = ":".join(os.path.join(site, d) for d in ("opencv_python_headless.libs", "scipy.libs"))
    env = dict(os.environ, OPENBLAS_NUM_THREADS=str(os.cpu_count()),
               LD_LIBRARY_PATH=libs + ":" + os.environ.get("LD_LIBRARY_PATH", ""))
    outs = {}
    for name in ("cuda", "ref"):
        out = str(tmp_path / ("out_%s_%s.png" % (tag, name)))
        flags = list(cuda_flags) if name == "cuda" else ["-q", "--no-mmap"]
        cmd = [os.path.join(REF, "flux_%s_cli" % name)] + args + ["-o", out] + flags
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=1500, env=env)
        assert r.returncode == 0, "%s failed:\n%s\n%s" % (name, r.stdout[-2000:], r.stderr[-2000:])
        if stderr_of is not None:
            stderr_of[name] = r.stderr
        outs[name] = read_png_rgb(out)
    a, b = outs["cuda"], outs["ref"]
    assert a.shape == b.shape == (128, 128, 3)
    assert b.std() > 10
    return 10 * np.log10(255.0 ** 2 / max(((a - b) ** 2).mean(), 1e-12))


def test_reference_cli_runs_on_the_engine(fx, model_dir, tmp_path):
    synth, d, mdir = model_dir
    emb, noise = str(tmp_path / "emb.bin"), str(tmp_path / "noise.bin")
    synth.make_context(1234, 512, d.text_dim).tofile(emb)
    fx.init_noise(128, 8, 8, 42).tofile(noise)
    psnr = _run_both(["-d", mdir, "-e", emb, "-n", noise, "-W", "128", "-H", "128", "-s", "4", "-S", "42"], tmp_path, "emb")
    assert psnr >= 30.0, "PSNR %.1f dB" % psnr


def test_reference_cli_default_call_path(fx, model_dir, tmp_path):
    """The CLI as it runs when nothing is switched off: the memory-mapped loader, whose file the transformer then owns
    (main.c:304, 429-432; flux.c:310-313), and the step / sub-step progress callbacks (main.c:147-154), which make the
    seam run the loop step by step. -v adds the timing breakdown (flux_sample.c:270-287). Same picture as the
    reference's CPU build, and the progress line the callbacks draw: five d, four s (one per five single blocks), F."""
    synth, d, mdir = model_dir
    emb, noise = str(tmp_path / "emb.bin"), str(tmp_path / "noise.bin")
    synth.make_context(1234, 512, d.text_dim).tofile(emb)
    fx.init_noise(128, 8, 8, 42).tofile(noise)
    err = {}
    psnr = _run_both(["-d", mdir, "-e", emb, "-n", noise, "-W", "128", "-H", "128", "-s", "4", "-S", "42"], tmp_path,
                     "default", cuda_flags=("-v",), stderr_of=err)
    assert psnr >= 30.0, "PSNR %.1f dB" % psnr
    log = err["cuda"]
    assert "Denoising (d=double block" in log
    for step in range(1, 5):
        assert "Step %d/4 dddddssssF" % step in log, log[-1500:]
    assert "Denoising timing breakdown" in log and "Single blocks:" in log


def test_reference_cli_debug_py_path(fx, model_dir, tmp_path):
    """`flux --debug-py` (flux_img2img_debug_py, flux.c:1125-1232): noise, reference latent and text embeddings come
    from three files under /tmp, the loop is flux_sample_euler_with_refs with T offset 10, then the VAE."""
    synth, d, mdir = model_dir
    files = {"/tmp/py_noise.bin": fx.init_noise(128, 8, 8, 11),
             "/tmp/py_ref_latent.bin": synth.make_latent(7, 128, 8, 8),
             "/tmp/py_text_emb.bin": synth.make_context(1234, 512, d.text_dim)}
    try:
        for path, arr in files.items():
            arr.astype(np.float32).tofile(path)
        psnr = _run_both(["-d", mdir, "--debug-py", "-W", "128", "-H", "128", "-s", "4"], tmp_path, "debugpy")
    finally:
        for path in files:
            if os.path.exists(path):
                os.remove(path)
    assert psnr >= 30.0, "PSNR %.1f dB" % psnr


def _repl_session(mdir, tmp_path, lines):
    """Drives the engine build of the reference's interactive mode (flux_cli.c) through its standard input and returns
    (stdout, [paths of the images it saved])."""
    site = os.path.dirname(os.path.dirname(np.__file__))
    env = dict(os.environ, HOME=str(tmp_path), TERM="dumb")
    r = subprocess.run([os.path.join(REF, "flux_cuda_cli"), "-d", mdir], input="\n".join(lines) + "\n",
                       capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    paths = [ln.split("Done -> ")[1].split(" (ref")[0] for ln in r.stdout.splitlines() if "Done -> " in ln]
    return r.stdout, paths


def test_reference_cli_from_a_text_prompt(fx, model_dir, tmp_path):
    """`flux -p "..."`: the reference's tokenizer feeds the text encoder, which runs on the GPU in one build and on the
    CPU in the other; a byte-level tokenizer file and seeded Qwen3-4B-shaped weights stand in for the real ones."""
    synth, d, mdir = model_dir
    import shutil
    qd = synth.QwenDims.qwen3_4b()
    try:
        synth.write_tokenizer_json(os.path.join(mdir, "tokenizer", "tokenizer.json"))
        synth.write_qwen_shards(os.path.join(mdir, "text_encoder"), synth.make_qwen_weights(qd, seed=0,
                                                                                            threads=os.cpu_count()))
        psnr = _run_both(["-d", mdir, "-p", "a cat in the rain and the thin man", "-W", "128", "-H", "128", "-s", "4",
                          "-S", "42"], tmp_path, "prompt")
        # img2img: the input image goes through the VAE encoder (GPU in one build, CPU in the other) and enters the
        # denoising loop as reference tokens
        rng = np.random.default_rng(3)
        yy, xx = np.mgrid[0:128, 0:128]
        pic = np.stack([128 + 100 * np.sin(xx / 9.0), 128 + 100 * np.cos(yy / 7.0), 40 + 1.5 * xx], axis=-1)
        pic = np.clip(pic + rng.normal(0, 6, pic.shape), 0, 255).astype(np.uint8)
        ppm = str(tmp_path / "input.ppm")
        with open(ppm, "wb") as f:
            f.write(b"P6\n128 128\n255\n" + pic.tobytes())
        psnr_i2i = _run_both(["-d", mdir, "-p", "the man in the rain", "-i", ppm, "-W", "128", "-H", "128", "-s", "4",
                              "-S", "7"], tmp_path, "img2img")
        # the interactive mode's embedding cache (flux_cli.c:380-400): the second and third time a prompt is entered
        # its embeddings come from the cache (4-bit block quantised, embcache.c:30-120, so slightly different from
        # the encoder's output) and go straight to flux_generate_with_embeddings
        out, imgs = _repl_session(mdir, tmp_path, ["!seed 42", "!size 128x128", "!steps 4",
                                                   "a cat in the rain and the thin man",
                                                   "a cat in the rain and the thin man",
                                                   "a cat in the rain and the thin man", "!quit"])
        assert len(imgs) == 3 and out.count("(using cached embedding)") == 2, out[-1500:]
        first, second, third = (read_png_rgb(p) for p in imgs)
        one_shot = read_png_rgb(str(tmp_path / "out_prompt_cuda.png"))
    finally:
        shutil.rmtree(os.path.join(mdir, "text_encoder"), ignore_errors=True)
    assert psnr >= 30.0, "PSNR %.1f dB" % psnr
    assert psnr_i2i >= 30.0, "img2img PSNR %.1f dB" % psnr_i2i
    assert np.array_equal(first, one_shot)   # the same prompt, seed and size as the `flux -p` run above: same picture
    assert np.array_equal(second, third)     # both from the cached embedding: the engine repeats itself bit for bit
    mse = np.mean((first - second) ** 2)     # the cache is lossy: close, not equal
    assert 10 * np.log10(255.0 ** 2 / max(mse, 1e-12)) >= 30.0
