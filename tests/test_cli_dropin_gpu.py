"""Drop-in check through the reference's own, unmodified CLI.

oracle/Makefile (`make cli`) links the reference's main.c / flux.c / flux_cli.c / flux_vae.c / ... twice: once as the
plain reference (`flux_ref_cli`, BLAS build) and once with flux_transformer.c + flux_sample.c replaced by the seam
(`flux_cuda_cli`, which calls libflux_cuda.so). Both are run on the same synthetic model directory with the same
external embeddings and noise; the decoded PNGs must agree to PSNR >= 30 dB.
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


def test_reference_cli_runs_on_the_engine(fx, tmp_path):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    cuda_cli, ref_cli = os.path.join(REF, "flux_cuda_cli"), os.path.join(REF, "flux_ref_cli")
    if not (os.path.exists(cuda_cli) and os.path.exists(ref_cli)):
        pytest.skip("oracle/_ref CLIs not built (make -C oracle cli)")
    import flux2_c_b200.synth as synth
    base = "/dev/shm" if os.access("/dev/shm", os.W_OK) else str(tmp_path)
    mdir = os.path.join(base, "flux_synth_model_%d" % os.getpid())
    os.makedirs(os.path.join(mdir, "transformer"), exist_ok=True)
    os.makedirs(os.path.join(mdir, "vae"), exist_ok=True)
    tpath = os.path.join(mdir, "transformer", "diffusion_pytorch_model.safetensors")
    vpath = os.path.join(mdir, "vae", "diffusion_pytorch_model.safetensors")
    try:
        d = synth.Dims.klein4b()
        synth.write_safetensors(tpath, synth.make_transformer_weights(d, seed=0, threads=os.cpu_count()))
        synth.write_safetensors(vpath, synth.make_vae_weights(), dtype="F32")
        open(os.path.join(mdir, "model_index.json"), "w").write('{"_class_name": "Flux2KleinPipeline", "is_distilled": true}')
        emb, noise = str(tmp_path / "emb.bin"), str(tmp_path / "noise.bin")
        synth.make_context(1234, 512, d.text_dim).tofile(emb)
        fx.init_noise(128, 8, 8, 42).tofile(noise)
        outs = {}
        # the reference's BLAS build needs the OpenBLAS (and its libgfortran / libquadmath) bundled in the image's wheels
        site = os.path.dirname(os.path.dirname(np.__file__))
        libs = ":".join(os.path.join(site, d) for d in ("opencv_python_headless.libs", "scipy.libs"))
        env = dict(os.environ, OPENBLAS_NUM_THREADS=str(os.cpu_count()),
                   LD_LIBRARY_PATH=libs + ":" + os.environ.get("LD_LIBRARY_PATH", ""))
        for name, exe in (("cuda", cuda_cli), ("ref", ref_cli)):
            out = str(tmp_path / ("out_%s.png" % name))
            cmd = [exe, "-d", mdir, "-e", emb, "-n", noise, "-W", "128", "-H", "128", "-s", "4", "-S", "42", "-o", out,
                   "-q", "--no-mmap"]
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=1500, env=env)
            assert r.returncode == 0, "%s failed:\n%s\n%s" % (name, r.stdout[-2000:], r.stderr[-2000:])
            outs[name] = read_png_rgb(out)
    finally:
        for p in (tpath, vpath, os.path.join(mdir, "model_index.json")):
            if os.path.exists(p):
                os.remove(p)
    a, b = outs["cuda"], outs["ref"]
    assert a.shape == b.shape == (128, 128, 3)
    assert b.std() > 10
    psnr = 10 * np.log10(255.0 ** 2 / max(((a - b) ** 2).mean(), 1e-12))
    assert psnr >= 30.0, "PSNR %.1f dB" % psnr
