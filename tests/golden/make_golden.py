"""Generates tests/golden/*.npz by running the REFERENCE implementation (compiled by oracle/Makefile into
oracle/_ref/) on seeded synthetic inputs. Needs oracle/_ref built from the reference's sources, ~40 GB of RAM and a few
minutes; the fixtures it writes are committed so that the tests need neither.

    python tests/golden/make_golden.py            # both weight sets
    python tests/golden/make_golden.py base|sharp

Inputs are NOT stored: tests regenerate them from the same seeds through flux2.c_b200/synth.py; each
fixture stores a checksum of the inputs it was computed from.
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


def checksum(*arrays):
    return float(sum(np.abs(np.asarray(a, dtype=np.float64)).sum() for a in arrays))


def run(kind):
    sharp = kind == "sharp"
    t0 = time.time()
    W = synth.make_transformer_weights(D, seed=0, sharp=sharp)
    path = "/tmp/synth_%s.safetensors" % kind
    if not os.path.exists(path):
        synth.write_safetensors(path, W)
    wsum = checksum(synth.bf16_bits_to_f32(W["proj_out.weight"]), synth.bf16_bits_to_f32(W["x_embedder.weight"]))
    del W
    lib = rb.RefLib(rb.best_kind())
    tf = lib.load_transformer(path)
    print(kind, "loaded in %.0fs (%s build)" % (time.time() - t0, lib.kind), flush=True)
    out = {"weights_checksum": wsum, "ref_build": lib.kind}

    # A / B: single forwards, small
    z = synth.make_latent(42, 128, 4, 4)
    ctx = synth.make_context(1234, 32, D.text_dim)
    out["A_v"] = tf.forward(z, 4, 4, ctx, 0.7)
    ref_lat = synth.make_latent(7, 128, 2, 3)
    out["B_v"] = tf.forward(z, 4, 4, ctx, 0.4, refs=[(ref_lat, 10)])
    ref_lat2 = synth.make_latent(8, 128, 3, 2)
    out["B2_v"] = tf.forward(z, 4, 4, ctx, 0.4, refs=[(ref_lat, 10), (ref_lat2, 20)])
    out["AB_in"] = checksum(z, ctx, ref_lat, ref_lat2)

    # C / D: 2-step Euler and CFG loops, small
    h, w, ntxt = 6, 4, 48
    z0 = lib.init_noise(128, h, w, 42)
    ctx = synth.make_context(1234, ntxt, D.text_dim)
    ctxu = synth.make_context(4321, ntxt, D.text_dim)
    sch = lib.official_schedule(2, h * w)
    out["C_sched"] = sch
    out["C_z0"] = z0
    v0 = tf.forward(z0, h, w, ctx, float(sch[0]))
    z1 = z0 + np.float32(sch[1] - sch[0]) * v0
    v1 = tf.forward(z1, h, w, ctx, float(sch[1]))
    out["C_v"] = np.stack([v0, v1])
    out["C_final"] = tf.sample_euler(z0, h, w, ctx, sch)
    out["D_final"] = tf.sample_euler_cfg(z0, h, w, ctx, ctxu, 4.0, sch)
    out["C_ref_final"] = tf.sample_euler(z0, h, w, ctx, sch, refs=[(ref_lat, 10)])
    out["CD_in"] = checksum(ctx, ctxu)
    print(kind, "small cases done", time.time() - t0, flush=True)

    # config 1 (256x256, 512 text tokens, 4 steps, noise seed 42): velocities along the reference's own trajectory
    def full_config(tag, h, w, steps):
        z = lib.init_noise(128, h, w, 42)
        ctx = synth.make_context(1234, 512, D.text_dim)
        sch = lib.official_schedule(steps, h * w)
        vs = []
        for i in range(steps):
            v = tf.forward(z, h, w, ctx, float(sch[i]))
            vs.append(v)
            z = z + np.float32(sch[i + 1] - sch[i]) * v
        out[tag + "_sched"] = sch
        out[tag + "_v"] = np.stack(vs)
        out[tag + "_final"] = tf.sample_euler(lib.init_noise(128, h, w, 42), h, w, ctx, sch)
        out[tag + "_final_stepwise"] = z
        print(kind, tag, "done", time.time() - t0, flush=True)

    if sharp:
        z = lib.init_noise(128, 16, 16, 42)
        ctx = synth.make_context(1234, 512, D.text_dim)
        out["cfg1_v0"] = tf.forward(z, 16, 16, ctx, 1.0)
    else:
        full_config("cfg1", 16, 16, 4)
        full_config("cfg2", 32, 32, 4)
    tf.close()
    np.savez_compressed(os.path.join(HERE, "reference_%s.npz" % kind), **out)


def host_fixtures():
    lib = rb.RefLib(rb.best_kind())
    out = {}
    for steps, n in [(4, 256), (4, 1024), (4, 4096), (50, 1024), (2, 16), (4, 4301), (8, 12544)]:
        out["official_%d_%d" % (steps, n)] = lib.official_schedule(steps, n)
    out["linear_7"] = lib.linear_schedule(7)
    out["power_5_2"] = lib.power_schedule(5, 2.0)
    for (h, w, seed) in [(4, 4, 42), (16, 16, 42), (32, 32, 42), (6, 4, 7), (64, 48, 123456789), (112, 112, 1)]:
        n = lib.init_noise(128, h, w, seed)
        out["noise_%d_%d_%d_head" % (h, w, seed)] = n.reshape(-1)[:64].copy()
        out["noise_%d_%d_%d_tail" % (h, w, seed)] = n.reshape(-1)[-64:].copy()
        out["noise_%d_%d_%d_sum" % (h, w, seed)] = np.float64(n.astype(np.float64).sum())
        out["noise_%d_%d_%d_abs" % (h, w, seed)] = np.float64(np.abs(n.astype(np.float64)).sum())
    np.savez_compressed(os.path.join(HERE, "reference_host.npz"), **out)
    x = np.random.default_rng(0).standard_normal((2, 32, 12, 8)).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "reference_patchify.npz"), **{"in": x, "patchified": lib.patchify(x)})


if __name__ == "__main__":
    kinds = sys.argv[1:] or ["host", "base", "sharp"]
    for k in kinds:
        host_fixtures() if k == "host" else run(k)
