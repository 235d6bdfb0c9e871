"""Further fixtures from the REFERENCE implementation (see make_golden.py): the two heavier BASELINE shapes.

  guided_256 : 256x256, 512 text tokens, 10 Euler steps with classifier-free guidance 4.0 (the base-model
               configuration at a step count the CPU reference finishes in minutes), "sharp" weights: combined
               velocities along the reference's own trajectory and the final latent.
  img2img_1024 : one forward of the 1024x1024 img2img shape (4096 target + 4096 reference tokens + 512 text
               tokens = 8704), benchmark weights; the velocity is stored subsampled (every 2nd latent row / column).

    python tests/golden/make_golden_extra.py
"""
import os
import sys
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


def main():
    lib = rb.RefLib(rb.best_kind())
    out = {"ref_build": lib.kind}
    t0 = time.time()

    tf = model("sharp", lib)
    h = w = 16
    steps, g = 10, 4.0
    z = lib.init_noise(128, h, w, 42)
    cc = synth.make_context(1234, 512, D.text_dim)
    cu = synth.make_context(4321, 512, D.text_dim)
    sch = lib.official_schedule(steps, h * w)
    vs = []
    for i in range(steps):
        vu = tf.forward(z, h, w, cu, float(sch[i]))
        vc = tf.forward(z, h, w, cc, float(sch[i]))
        v = vu + np.float32(g) * (vc - vu)  # flux_sample.c:495-499
        vs.append(v)
        z = z + np.float32(sch[i + 1] - sch[i]) * v
        print("guided step", i, time.time() - t0, flush=True)
    out["guided_256_sched"] = sch
    out["guided_256_v"] = np.stack(vs)
    out["guided_256_final"] = z
    tf.close()

    tf = model("base", lib)
    h = w = 64
    z = lib.init_noise(128, h, w, 42)
    ref = synth.make_latent(7, 128, 64, 64)
    c = synth.make_context(1234, 512, D.text_dim)
    v = tf.forward(z, h, w, c, 1.0, refs=[(ref, 10)])
    out["img2img_1024_v_sub"] = v[:, ::2, ::2].copy()
    out["img2img_1024_v_rms"] = np.float64(np.sqrt((v.astype(np.float64) ** 2).mean()))
    print("img2img forward", time.time() - t0, flush=True)
    tf.close()
    np.savez_compressed(os.path.join(HERE, "reference_extra.npz"), **out)


def guided_512():
    """BASELINE config 3 in full: benchmark weights, 512x512, 50 Euler steps, guidance 4.0, separate conditional /
    unconditional 512-token contexts. 100 reference forwards (about half an hour on 8 cores). Stored: the final
    latent and, for three probe steps, the reference's state and combined velocity."""
    lib = rb.RefLib(rb.best_kind())
    tf = model("base", lib)
    h = w = 32
    steps, g = 50, 4.0
    z = lib.init_noise(128, h, w, 42)
    cc = synth.make_context(1234, 512, D.text_dim)
    cu = synth.make_context(4321, 512, D.text_dim)
    sch = lib.official_schedule(steps, h * w)
    out = {"sched": sch, "ref_build": lib.kind}
    t0 = time.time()
    for i in range(steps):
        vu = tf.forward(z, h, w, cu, float(sch[i]))
        vc = tf.forward(z, h, w, cc, float(sch[i]))
        v = vu + np.float32(g) * (vc - vu)
        if i in (0, 24, 49):
            out["z_%d" % i] = z.copy()
            out["v_%d" % i] = v.copy()
        z = z + np.float32(sch[i + 1] - sch[i]) * v
        print("guided 512 step", i, time.time() - t0, flush=True)
    out["final"] = z
    tf.close()
    np.savez_compressed(os.path.join(HERE, "reference_guided512.npz"), **out)


def qwen3():
    """Text encoder at the Qwen3-4B shape: 64 tokens (40 valid, 24 padded) through the reference's qwen3_forward;
    every 4th output column is stored."""
    import shutil
    import tempfile
    lib = rb.RefLib(rb.best_kind())
    d = synth.QwenDims.qwen3_4b()
    W = synth.make_qwen_weights(d, seed=0)
    chk = float(np.abs(synth.bf16_bits_to_f32(W["model.layers.0.self_attn.q_norm.weight"]).astype(np.float64)).sum() +
                np.abs(synth.bf16_bits_to_f32(W["model.layers.26.mlp.down_proj.weight"][:64]).astype(np.float64)).sum())
    mdir = tempfile.mkdtemp(prefix="qwen_synth_", dir="/tmp")
    try:
        synth.write_qwen_shards(mdir, W)
        del W
        m = lib.qwen3_load(mdir)
    finally:
        shutil.rmtree(mdir, ignore_errors=True)
    ids = np.random.default_rng(64).integers(0, d.vocab, 64).astype(np.int32)
    mask = np.array([1] * 40 + [0] * 24, dtype=np.int32)
    out = lib.qwen3_forward(m, ids, mask)
    lib.L.qwen3_model_free(m)
    np.savez_compressed(os.path.join(HERE, "reference_qwen3.npz"), ids=ids, mask=mask, out_sub=out[:, ::4].copy(),
                        out_rms=np.float64(np.sqrt((out.astype(np.float64) ** 2).mean())), weights_checksum=chk,
                        ref_build=lib.kind)
    print("qwen3 golden written, rms", float(np.sqrt((out.astype(np.float64) ** 2).mean())))


if __name__ == "__main__":
    if sys.argv[1:] == ["guided512"]:
        guided_512()
    elif sys.argv[1:] == ["qwen3"]:
        qwen3()
    else:
        main()
