"""Fixtures from the REFERENCE implementation (see make_golden.py) that pin the remaining benchmarked configurations.

  python tests/golden/make_golden_pins.py img2img    1024x1024 img2img (8704 tokens) as a 4-step Euler loop
  python tests/golden/make_golden_pins.py qwen3      text encoder at the Qwen3-4B shape, 512 tokens, all valid
  python tests/golden/make_golden_pins.py psnr512    the reference VAE's image of the 512x512 final latent
  python tests/golden/make_golden_pins.py samplers   Heun / ancestral / generate_latent loops and the two unused schedules

Each part writes one .npz next to this file. Every value comes out of the reference build under oracle/_ref
(oracle/ref_binding.py); the inputs are the seeded synthetic tensors of flux2.c_b200/synth.py.
"""
import os
import shutil
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
from conftest import load_package  # noqa: E402

load_package()
import flux2_c_b200.synth as synth  # noqa: E402
from oracle import ref_binding as rb  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
D = synth.Dims.klein4b()


def model(kind, lib):
    path = "/tmp/synth_%s.safetensors" % kind
    if not os.path.exists(path):
        synth.write_safetensors(path, synth.make_transformer_weights(D, seed=0, sharp=kind == "sharp"))
    return lib.load_transformer(path)


def img2img():
    """BASELINE config 4 as a loop: 4096 target + 4096 reference tokens (T offset 10) + 512 text tokens, 4 Euler steps
    on the official schedule. The loop is flux_sample_euler_with_refs' own (flux_sample.c:303-375): v = forward(z, t_i),
    z += dt v. Stored: the velocity of every step (every 2nd latent row / column), the reference's state before steps
    1..3 rounded to f16 (the engine is fed these states, so a step's error is not mixed with drift; the rounding moves
    the input by 5e-4 of its norm, far inside the 2e-2 gate), and the final latent (every 2nd row / column)."""
    lib = rb.RefLib(rb.best_kind())
    tf = model("base", lib)
    h = w = 64
    z = lib.init_noise(128, h, w, 42)
    ref = synth.make_latent(7, 128, 64, 64)
    c = synth.make_context(1234, 512, D.text_dim)
    sch = lib.official_schedule(4, h * w)
    out = {"sched": sch, "ref_build": lib.kind}
    t0 = time.time()
    for i in range(4):
        if i:
            out["z_%d_f16" % i] = z.astype(np.float16)
            z_in = out["z_%d_f16" % i].astype(np.float32)  # the velocity stored is the one of the stored state
        else:
            z_in = z
        v = tf.forward(z_in, h, w, c, float(sch[i]), refs=[(ref, 10)])
        out["v_%d_sub" % i] = v[:, ::2, ::2].copy()
        out["v_%d_rms" % i] = np.float64(np.sqrt((v.astype(np.float64) ** 2).mean()))
        z = z_in + np.float32(sch[i + 1] - sch[i]) * v
        print("img2img step", i, time.time() - t0, flush=True)
    out["final_sub"] = z[:, ::2, ::2].copy()
    out["final_rms"] = np.float64(np.sqrt((z.astype(np.float64) ** 2).mean()))
    tf.close()
    np.savez_compressed(os.path.join(HERE, "reference_img2img_loop.npz"), **out)


def qwen3():
    """qwen3_forward (flux_qwen3.c:1041-1156) on 512 tokens, attention mask all ones: the shape the benchmark's
    prompt-to-image leg runs. Every 4th output column is stored."""
    lib = rb.RefLib(rb.best_kind())
    d = synth.QwenDims.qwen3_4b()
    W = synth.make_qwen_weights(d, seed=0)
    mdir = tempfile.mkdtemp(prefix="qwen_synth_", dir="/tmp")
    try:
        synth.write_qwen_shards(mdir, W)
        del W
        m = lib.qwen3_load(mdir)
    finally:
        shutil.rmtree(mdir, ignore_errors=True)
    ids = np.random.default_rng(512).integers(0, d.vocab, 512).astype(np.int32)
    mask = np.ones(512, dtype=np.int32)
    t0 = time.time()
    out = lib.qwen3_forward(m, ids, mask)
    print("qwen3 forward", time.time() - t0, flush=True)
    lib.L.qwen3_model_free(m)
    np.savez_compressed(os.path.join(HERE, "reference_qwen3_512.npz"), ids=ids, out_sub=out[:, ::4].copy(),
                        out_rms=np.float64(np.sqrt((out.astype(np.float64) ** 2).mean())), ref_build=lib.kind)


def psnr512():
    """flux_vae_decode (flux_vae.c:690-837) of the reference's own final latent of BASELINE config 2 (512x512, the
    'cfg2_final' entry of reference_base.npz) with the plain synthetic VAE weights: the uint8 RGB image."""
    lib = rb.RefLib(rb.best_kind())
    gold = np.load(os.path.join(HERE, "reference_base.npz"))
    vpath = "/tmp/synth_vae_plain.safetensors"
    synth.write_safetensors(vpath, synth.make_vae_weights(), dtype="F32")
    vae = lib.load_vae(vpath)
    t0 = time.time()
    img = lib.vae_decode(vae, gold["cfg2_final"])
    print("vae decode 512", time.time() - t0, "std", img.std(), flush=True)
    lib.L.flux_vae_free(vae)
    np.savez_compressed(os.path.join(HERE, "reference_cfg2_image.npz"), image=img, ref_build=lib.kind)


def samplers():
    """The exports nothing in the reference calls (flux_sample.c:75-116, 697-821, 891-919), at the klein shape on a
    4 x 4 latent with 32 text tokens."""
    lib = rb.RefLib(rb.best_kind())
    out = {"ref_build": lib.kind}
    for n, shift in ((4, 0.0), (10, 1.5), (50, -0.75)):
        out["sigmoid_%d_%g" % (n, shift)] = lib.sigmoid_schedule(n, shift)
    for n, hh, ww in ((4, 256, 256), (8, 512, 512), (20, 1024, 1024), (5, 512, 768)):
        out["resolution_%d_%d_%d" % (n, hh, ww)] = lib.resolution_schedule(n, hh, ww)
    tf = model("sharp", lib)
    h = w = 4
    z0 = lib.init_noise(128, h, w, 42)
    c = synth.make_context(1234, 32, D.text_dim)
    sch = lib.official_schedule(3, h * w)
    out["sched"] = sch
    out["heun_final"] = tf.sample_heun(z0, h, w, c, sch)
    out["ancestral_final"] = tf.sample_euler_ancestral(z0, h, w, c, sch, 0.5, 777)
    out["ancestral_eta0_final"] = tf.sample_euler_ancestral(z0, h, w, c, sch, 0.0, 777)
    out["euler_final"] = tf.sample_euler(z0, h, w, c, sch)
    out["generate_final"] = tf.generate_latent(c, 64, 64, 2, 5)
    tf.close()
    np.savez_compressed(os.path.join(HERE, "reference_samplers.npz"), **out)
    print("samplers written", flush=True)


if __name__ == "__main__":
    for part in sys.argv[1:]:
        {"img2img": img2img, "qwen3": qwen3, "psnr512": psnr512, "samplers": samplers}[part]()
