#!/usr/bin/env python
"""Benchmark of the B200 denoising engine on the reference's headline workload.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --micro gemm|gemmtable|attn|adaln|qwen3|vae|conv|gn|load|step [...]   # one kernel or stage, small memory

Workload ("step" = one image): FLUX.2-klein-4B-shaped DiT, seeded random bf16 weights N(0, 0.02), 512x512 output
(1024 image tokens + 512 text tokens), batch 1, 4-step Euler loop on the official schedule, guidance 1; image i of
the job has noise seed i and the context of seed 10000 + i. Metric: images/s (whole job). With N > 1 (launched by torchrun, one rank per GPU) every rank holds a
full replica and denoises its own images: independent seeds, no collective on the data path, weak scaling.

The JSON line also carries the end-to-end figure through the library's host-buffer API (`e2e`: uploads and downloads
inside the timed region, pipelined; the one-image-at-a-time figure beside it), the roofline of
the dominant kernel (`roofline`) and the reference's CPU path timed on this machine's host cores
(`cpu_baseline`). `--impl reference` times the reference's own CPU implementation (oracle/_ref, built from the
reference's sources by oracle/Makefile) instead.
"""
import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))

H_LAT, W_LAT, TXT, STEPS_PER_IMAGE = 32, 32, 512, 4
WORKLOAD = "klein4b_512x512_4step_b1"
METRIC = "images_per_sec_512x512_4step"


_OUT = None  # the process's real stdout, once main() has pointed file descriptor 1 at stderr


def emit(obj):
    """Prints the result line. Libraries that write to stdout on their own (NCCL's version banner under NCCL_DEBUG=VERSION)
    have had file descriptor 1 redirected to stderr by main(), so that stdout carries the JSON line and nothing else."""
    out = _OUT if _OUT is not None else sys.stdout
    out.write(json.dumps(obj) + "\n")
    out.flush()


def bench_config(world):
    """The `config` object of the result line; both arms print the same one (the reference's CPU path computes in f32,
    which its `dtype` says)."""
    return {"workload": WORKLOAD, "tokens": H_LAT * W_LAT + TXT, "dit_steps_per_image": STEPS_PER_IMAGE,
            "inputs": "image i: noise seed i, 512-token N(0,1) context of seed 10000 + i; image i on rank i % N",
            "operands": "f16 x f16 (weights converted from bf16 at load), f32 accumulate",
            "parallelism": "replica_dp%d" % world, "l2": "inputs larger than L2: 7.75 GB of weights per DiT step",
            "accumulate": "f32", "residual_stream": "f32"}


def load_package():
    name = "flux2_c_b200"
    if name in sys.modules:
        return sys.modules[name]
    pkg = os.path.join(ROOT, "flux2.c_b200")
    spec = importlib.util.spec_from_file_location(name, os.path.join(pkg, "__init__.py"),
                                                  submodule_search_locations=[pkg])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


def step_flops(n_img, n_txt, d):
    """Algorithmic FLOPs of one DiT forward (2 per MAC; GEMMs + attention), as a dict by kernel class."""
    h, m, C, T = d.hidden, d.mlp, d.latent_ch, d.text_dim
    N = n_img + n_txt
    gemm = d.n_double * N * 2 * (4 * h * h + 3 * h * m) + d.n_single * N * 2 * (h * (3 * h + 2 * m) + (h + m) * h)
    gemm += 2 * n_img * C * h + 2 * n_img * h * C
    attn = (d.n_double + d.n_single) * 4 * N * N * h
    return {"gemm": float(gemm), "attn": float(attn), "ctx_embed_once": float(2 * n_txt * T * h)}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        top = sorted(sm)[len(sm) // 2:]  # samples under load: the upper half (idle samples sit at the low clock)
        return {"sm_mhz": statistics.median(top), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------------- CPU arms
def cpu_port_baseline(synth, weights, dims, z0, ctx, sched):
    """The numpy restatement of the reference's forward, timed on the host cores: ONE DiT forward of the
    512x512 workload (the first of an image's four), images/s = 1 / (4 x that)."""
    sys.path.insert(0, ROOT)
    from oracle import flux_oracle as fo
    om = fo.OracleModel(weights, dims)
    om.preload()  # bf16 -> f32 expansion of the weights is model loading, not the step
    t0 = time.perf_counter()
    om.forward(z0, H_LAT, W_LAT, ctx, float(sched[0]))
    dt = time.perf_counter() - t0
    return {"value": 1.0 / (STEPS_PER_IMAGE * dt), "unit": "images/s", "cores": os.cpu_count(), "kind": "port",
            "sample": "1 of the 4 DiT forwards of one 512x512 image (%.1f s), x4; numpy f32 + its threaded BLAS" % dt,
            "ms_per_dit_step": dt * 1e3}


def cpu_reference_baseline(synth, weights, dims, z0, ctx, sched):
    """The reference's own CPU build (oracle/_ref) timed on the host cores: ONE DiT forward of the 512x512 workload,
    images/s = 1 / (4 x that). Returns None when the build did not travel with the repository."""
    sys.path.insert(0, ROOT)
    from oracle import ref_binding as rb
    kind = rb.best_kind()
    if kind is None:
        return None
    tmpdir = "/dev/shm" if os.path.isdir("/dev/shm") and os.access("/dev/shm", os.W_OK) else tempfile.gettempdir()
    path = os.path.join(tmpdir, "flux_bench_cpu_%d.safetensors" % os.getpid())
    try:
        synth.write_safetensors(path, weights)
        lib = rb.RefLib(kind)
        tf = lib.load_transformer(path)
    finally:
        if os.path.exists(path):
            os.remove(path)
    t0 = time.perf_counter()
    tf.forward(z0, H_LAT, W_LAT, ctx, float(sched[0]))
    dt = time.perf_counter() - t0
    tf.close()
    return {"value": 1.0 / (STEPS_PER_IMAGE * dt), "unit": "images/s", "cores": lib.blas_threads, "kind": "reference",
            "sample": "1 of the 4 DiT forwards of one 512x512 image (%.1f s), x4; the reference's %s build, %d BLAS "
                      "threads" % (dt, kind, lib.blas_threads), "ms_per_dit_step": dt * 1e3}


def run_reference_arm(args):
    """--impl reference: the reference's own CPU code (oracle/_ref) on the same workload, host cores only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    load_package()
    import flux2_c_b200.synth as synth
    sys.path.insert(0, ROOT)
    from oracle import ref_binding as rb
    kind = rb.best_kind()
    if kind is None:
        emit({"impl": "reference", "unavailable": "oracle/_ref was not built (run make -C oracle)"})
        return 0
    dims = synth.Dims.klein4b()
    tmpdir = "/dev/shm" if os.path.isdir("/dev/shm") and os.access("/dev/shm", os.W_OK) else tempfile.gettempdir()
    path = os.path.join(tmpdir, "flux_bench_ref_%d.safetensors" % os.getpid())
    try:
        W = synth.make_transformer_weights(dims, seed=0)
        synth.write_safetensors(path, W)
        del W
        lib = rb.RefLib(kind)
        tf = lib.load_transformer(path)
    finally:
        if os.path.exists(path):
            os.remove(path)
    z0 = lib.init_noise(dims.latent_ch, H_LAT, W_LAT, 42)
    ctx = synth.make_context(1234, TXT, dims.text_dim)
    sched = lib.official_schedule(STEPS_PER_IMAGE, H_LAT * W_LAT)
    # one "step" of this arm = a bounded sample of one image: ONE of its four DiT forwards (the reference's CPU path
    # needs ~20 s per forward on 16 cores, so a whole image per step would not end within minutes). images/s =
    # 1 / (forwards_per_image x the mean forward time); ms_per_step is the time of what a step really ran.
    # CPU code has nothing to warm beyond its first call (page faults, BLAS thread pool): one untimed forward at most,
    # so that the default run stays within minutes; the line reports the warm-up really done.
    warm = min(args.warmup, 1)
    for _ in range(warm):
        tf.forward(z0, H_LAT, W_LAT, ctx, float(sched[0]))
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tf.forward(z0, H_LAT, W_LAT, ctx, float(sched[0]))
    dt = (time.perf_counter() - t0) / args.steps
    value = 1.0 / (STEPS_PER_IMAGE * dt)
    threads = lib.blas_threads
    sample = ("per step: 1 of the 4 DiT forwards of one 512x512 image; images/s = 1 / (4 x ms_per_step) "
              "(%s build, %d BLAS threads)" % (kind, threads))
    line = {"metric": METRIC, "value": value, "unit": "images/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
            "config": bench_config(args.gpus), "forwards_per_step": 1, "forwards_per_image": STEPS_PER_IMAGE,
            "ms_per_image": STEPS_PER_IMAGE * dt * 1e3,
            "cpu_baseline": {"value": value, "unit": "images/s", "cores": threads, "kind": "reference",
                             "sample": sample},
            "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "ms_per_dit_step": dt * 1e3}
    emit(line)
    return 0


# ---------------------------------------------------------------------------------------------- micro benches
def run_micro(args):
    import torch
    fx = load_package()
    ctx = fx.Context(0)
    stream = torch.cuda.ExternalStream(ctx.stream)
    peaks = measured_peaks()
    iters = args.steps

    def timed(fn):
        for _ in range(max(3, args.warmup)):
            fn()
        ctx.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
        ctx.sync()
        return e0.elapsed_time(e1) / iters

    if args.micro == "gemm":
        M, N, K = args.shape
        x = torch.randn(M, K, device="cuda").to(torch.float16)  # f16 operands, as in the engine
        w = (torch.randn(N, K, device="cuda") * 0.02).to(torch.float16)
        out = torch.zeros(M, N, device="cuda", dtype=torch.float16)
        torch.cuda.synchronize()
        epi = fx.EPI_STORE_BF16 | fx.EPI_X_F16 | fx.EPI_OUT_F16
        if args.epi == "qkv":
            # the fused [Q|K|V] projection with per-head RMSNorm and rotation in the epilogue (N = 3 * heads * 128)
            wq = torch.randn(128, device="cuda")
            ang = torch.rand(M, 64, device="cuda") * 6.28
            cos = torch.cos(ang).repeat_interleave(2, dim=1).contiguous()
            sin = torch.sin(ang).repeat_interleave(2, dim=1).contiguous()
            torch.cuda.synchronize()
            ms = timed(lambda: ctx.gemm_qkv_norm_rope(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N // 3, K,
                                                      wq.data_ptr(), wq.data_ptr(), cos.data_ptr(), sin.data_ptr(), M,
                                                      f16=True))
        elif args.epi == "gated":
            # the gated residual update of the f32 stream: out_f32 += gate * acc (read-modify-write epilogue)
            res = torch.randn(M, N, device="cuda")
            gate = torch.randn(N, device="cuda")
            torch.cuda.synchronize()
            ms = timed(lambda: ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), res.data_ptr(), M, N, K,
                                             fx.EPI_GATED_RES_F32 | fx.EPI_X_F16, gate_ptr=gate.data_ptr(),
                                             tile_n=args.tile_n))
        elif args.epi == "f32":
            res = torch.zeros(M, N, device="cuda")
            torch.cuda.synchronize()
            ms = timed(lambda: ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), res.data_ptr(), M, N, K,
                                             fx.EPI_STORE_F32 | fx.EPI_X_F16, tile_n=args.tile_n))
        else:
            ms = timed(lambda: ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, epi,
                                             tile_n=args.tile_n))
        tf = 2.0 * M * N * K / ms / 1e9
        line = {"micro": "gemm", "shape": [M, N, K], "tile_n": args.tile_n, "epilogue": args.epi, "ms": ms,
                "tflops": tf, "frac_of_burst_peak": tf / peaks["bf16"], "peak_source": peaks["source"]}
        if args.trace and args.tile_n == 512:
            # timeline of the first CTA of one more launch, in SM clock cycles since that CTA's entry
            stamps = torch.zeros(8, dtype=torch.int64, device="cuda")
            torch.cuda.synchronize()
            ctx.set_gemm_trace(stamps.data_ptr())
            if args.epi == "gated":
                ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), res.data_ptr(), M, N, K, fx.EPI_GATED_RES_F32 | fx.EPI_X_F16,
                              gate_ptr=gate.data_ptr(), tile_n=512)
            elif args.epi == "f32":
                ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), res.data_ptr(), M, N, K, fx.EPI_STORE_F32 | fx.EPI_X_F16,
                              tile_n=512)
            else:
                ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, epi, tile_n=512)
            ctx.sync()
            ctx.set_gemm_trace(None)
            st = stamps.cpu().tolist()
            names = ["entry", "prologue_done", "first_operands", "last_mma_issued", "first_accumulator_ready",
                     "last_epilogue_done", "before_teardown", "tmem_freed"]
            line["trace_cycles_since_entry"] = {n: int(v - st[0]) for n, v in zip(names, st)}
        emit(line)
    elif args.micro == "gemmtable":
        # The GEMM shapes of the 512x512 configuration (N x K of each projection) at M = 512, 1024 and 1536 rows, timed
        # back to back in one process at burst clocks, with torch.matmul (cuBLAS) on the same operands as the yardstick
        # column. Plain 16-bit store epilogue on both sides.
        shapes = [("double qkv", 9216, 3072), ("double ff in", 18432, 3072), ("single linear1", 27648, 3072),
                  ("single linear2", 3072, 12288), ("out proj", 3072, 3072), ("double ff out", 3072, 9216)]
        rows = []
        epi = fx.EPI_STORE_BF16 | fx.EPI_X_F16 | fx.EPI_OUT_F16
        for name, N, K in shapes:
            for M in (512, 1024, 1536):
                x = torch.randn(M, K, device="cuda").to(torch.float16)
                w = (torch.randn(N, K, device="cuda") * 0.02).to(torch.float16)
                out = torch.zeros(M, N, device="cuda", dtype=torch.float16)
                torch.cuda.synchronize()
                ms = timed(lambda: ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, epi))
                wt = w.t()
                with torch.cuda.stream(stream):
                    ms_lib = timed(lambda: torch.matmul(x, wt, out=out))
                fl = 2.0 * M * N * K
                rows.append({"name": name, "M": M, "N": N, "K": K, "us": round(ms * 1e3, 2),
                             "tflops": round(fl / ms / 1e9, 1), "torch_matmul_us": round(ms_lib * 1e3, 2),
                             "torch_matmul_tflops": round(fl / ms_lib / 1e9, 1)})
                del x, w, out
        emit({"micro": "gemmtable", "rows": rows, "peak_source": peaks["source"]})
    elif args.micro == "attn":
        seq, heads = args.seq, 24
        hid = heads * 128
        qkv = torch.randn(seq, 3 * hid, device="cuda").to(torch.float16)
        out = torch.zeros(seq, hid, device="cuda", dtype=torch.float16)
        torch.cuda.synchronize()
        ms = timed(lambda: ctx.attention(qkv.data_ptr(), 1, seq, 3 * hid, 0, hid, 2 * hid, heads, out.data_ptr(), hid,
                                         f16=True))
        tf = 4.0 * seq * seq * hid / ms / 1e9
        line = {"micro": "attn", "seq": seq, "heads": heads, "ms": ms, "tflops": tf,
                "frac_of_burst_peak": tf / peaks["bf16"], "peak_source": peaks["source"]}
        if args.trace:
            # timeline of CTA (0, 0, 0) of one more launch: 16 SM-clock stamps per key tile, relative to the first
            T = (seq + 127) // 128
            stamps = torch.zeros(16 * T, dtype=torch.int64, device="cuda")
            torch.cuda.synchronize()
            ctx.set_gemm_trace(stamps.data_ptr())
            ctx.attention(qkv.data_ptr(), 1, seq, 3 * hid, 0, hid, 2 * hid, heads, out.data_ptr(), hid, f16=True)
            ctx.sync()
            ctx.set_gemm_trace(None)
            st = stamps.cpu().view(T, 16)
            base = int(st[st > 0].min())
            line["trace_cycles"] = [[int(v - base) if v > 0 else None for v in row] for row in st.tolist()]
        emit(line)
    elif args.micro == "adaln":
        rows, hid = args.rows, 3072
        x = torch.randn(rows, hid, device="cuda")
        sh = torch.randn(hid, device="cuda")
        sc = torch.randn(hid, device="cuda")
        out = torch.zeros(rows, hid, device="cuda", dtype=torch.bfloat16)
        torch.cuda.synchronize()
        ms = timed(lambda: ctx.adaln(x.data_ptr(), out.data_ptr(), rows, hid, sh.data_ptr(), sc.data_ptr()))
        gbs = rows * hid * 6.0 / ms / 1e6
        emit({"micro": "adaln", "rows": rows, "ms": ms, "gbs": gbs, "frac_of_hbm_peak":
                          gbs / peaks["hbm_gbs"], "peak_source": peaks["source"]})
    elif args.micro == "gn":
        # K9: GroupNorm(32) + swish over a channels-last f32 tensor of --size x --size pixels x --shape[1] channels
        # (statistics pass + normalise pass): algorithmic bytes = 2 reads of the f32 input + 1 write of the 16-bit output
        side, C = args.size, args.shape[1]
        x = torch.randn(1, side * side, C, device="cuda") * 2 + 0.5
        g = torch.randn(C, device="cuda")
        b = torch.randn(C, device="cuda")
        out = torch.zeros(1, side * side, C, device="cuda", dtype=torch.float16)
        torch.cuda.synchronize()
        ms = timed(lambda: ctx.group_norm(x.data_ptr(), False, out.data_ptr(), 1, side * side, C, g.data_ptr(),
                                          b.data_ptr(), 1e-4, True))
        algo = side * side * C * (4 + 4 + 2)
        emit({"micro": "gn", "pixels": side * side, "channels": C, "ms": ms, "gbs": algo / ms / 1e6,
                          "frac_of_hbm_peak": algo / ms / 1e6 / peaks["hbm_gbs"], "algorithmic_bytes": algo,
                          "peak_source": peaks["source"]})
    elif args.micro == "step":
        # Every kernel of the denoising loop at its real shape in a process that holds about 1.5 GB on the device (for
        # profiler captures of the small kernels): a model with the klein-4B widths but ONE double-stream and ONE
        # single-stream block, 512x512, 512 text tokens, 4 steps; --guidance 4 runs the guidance pair as a batch of two.
        import numpy as np
        synth = importlib.import_module("flux2_c_b200.synth")
        dims = synth.Dims(n_double=1, n_single=1)
        model = fx.Model.from_tensors(ctx, dims, synth.make_transformer_weights(dims, seed=0, threads=os.cpu_count()))
        guided = args.guidance != 1.0
        sampler = fx.Sampler(model, H_LAT, W_LAT, TXT, batch=2 if guided else 1, max_steps=STEPS_PER_IMAGE)
        z0 = torch.from_numpy(fx.init_noise(dims.latent_ch, H_LAT, W_LAT, 42)).pin_memory()
        cc = torch.from_numpy(synth.make_context(1234, TXT, dims.text_dim)).pin_memory()
        cu = torch.from_numpy(synth.make_context(4321, TXT, dims.text_dim)).pin_memory()
        sched = fx.official_schedule(STEPS_PER_IMAGE, H_LAT * W_LAT)
        sampler.upload(z0.data_ptr(), cc.data_ptr(), cu.data_ptr() if guided else None)
        ms = timed(lambda: sampler.run(sched, guidance=args.guidance))
        out = torch.zeros(z0.numel(), dtype=torch.float32).pin_memory()
        sampler.download(out.data_ptr())
        emit({"micro": "step", "blocks": [1, 1], "guided": guided, "ms_per_image": ms,
              "launches": sampler.last_run()[1], "finite": bool(torch.isfinite(out).all())})
        sampler.close()
        model.close()
    elif args.micro == "load":
        # Load time of the klein-4B-shaped transformer file (7.75 GB, bf16) through the engine's safetensors loader:
        # map, validate, copy, convert bf16 -> f16 and re-lay on the device. The file sits in RAM-backed storage, so
        # this is the loader's own cost, not a disk's.
        synth = importlib.import_module("flux2_c_b200.synth")
        dims = synth.Dims.klein4b()
        shm = "/dev/shm" if os.path.isdir("/dev/shm") and os.access("/dev/shm", os.W_OK) else tempfile.gettempdir()
        path = os.path.join(shm, "flux_bench_load_%d.safetensors" % os.getpid())
        synth.write_safetensors(path, synth.make_transformer_weights(dims, seed=0, threads=os.cpu_count()))
        size = os.path.getsize(path)
        times = []
        try:
            for _ in range(max(2, min(iters, 3))):
                t0 = time.perf_counter()
                model = fx.Model.load_safetensors(ctx, path)
                ctx.sync()
                times.append(time.perf_counter() - t0)
                model.close()
        finally:
            os.remove(path)
        emit({"micro": "load", "file_gb": size / 1e9, "seconds": times, "best_gb_per_s": size / 1e9 / min(times)})
    elif args.micro == "conv":
        # K8 alone: 3x3 convolution, --size x --size pixels, --shape[1] -> --shape[2] channels (shape[0] unused),
        # 16-bit channels-last in, f32 out (the upsampling convolutions of the VAE decoder).
        side, cin, cout = args.size, args.shape[1], args.shape[2]
        x = torch.randn(1, side, side, cin, device="cuda").to(torch.float16)
        w = (torch.randn(cout, 9 * cin, device="cuda") * 0.02).to(torch.float16)
        b = torch.randn(cout, device="cuda")
        out = torch.zeros(side * side, cout, device="cuda")
        torch.cuda.synchronize()
        ms = timed(lambda: ctx.conv3x3(x.data_ptr(), 1, side, side, cin, w.data_ptr(), cout, b.data_ptr(), 1,
                                       out.data_ptr(), cout))
        tf = 2.0 * 9 * cin * cout * side * side / ms / 1e9
        algo = side * side * (cin * 2 + cout * 4) + w.numel() * 2
        emit({"micro": "conv", "pixels": [side, side], "cin": cin, "cout": cout, "ms": ms, "tflops": tf,
                          "frac_of_burst_peak": tf / peaks["bf16"], "algorithmic_bytes": algo,
                          "peak_source": peaks["source"]})
    elif args.micro == "vae":
        # The VAE decoder on a --size x --size image (latent size/16): device time with the latent resident, and the
        # host-buffer call (latent in, uint8 RGB out).
        import numpy as np
        synth = importlib.import_module("flux2_c_b200.synth")
        vae = fx.Vae.from_tensors(ctx, synth.make_vae_weights(seed=5, rich=True))
        hl = args.size // 16
        lat = torch.from_numpy(synth.make_latent(42, 128, hl, hl)).cuda()
        img = np.empty((16 * hl, 16 * hl, 3), dtype=np.uint8)
        torch.cuda.synchronize()
        ms = timed(lambda: vae.decode_device(lat.data_ptr(), hl, hl))
        lat_h = lat.cpu().numpy()
        t0 = time.perf_counter()
        for _ in range(iters):
            vae.decode_ptr(lat_h.ctypes.data, hl, hl, img.ctypes.data)
        e2e = (time.perf_counter() - t0) * 1e3 / iters
        px = [(2 * hl) ** 2 * 4 ** i for i in range(4)]  # pixels per level: 1/8, 1/4, 1/2 and full resolution
        c3 = lambda p, ci, co: 2.0 * 9 * ci * co * p
        flops = (c3(px[0], 32, 512) + 10 * c3(px[0], 512, 512) + 4 * 2.0 * px[0] * 512 * 512 + 4.0 * px[0] * px[0] * 512 +
                 7 * c3(px[1], 512, 512) + c3(px[2], 512, 512) + c3(px[2], 512, 256) + 5 * c3(px[2], 256, 256) +
                 2.0 * px[2] * 512 * 256 + c3(px[3], 256, 256) + c3(px[3], 256, 128) + 5 * c3(px[3], 128, 128) +
                 2.0 * px[3] * 256 * 128 + c3(px[3], 128, 3))
        # the encoder on an image of the same size (host f32 [3, H, W] in, host latent out)
        rgbf = np.random.default_rng(0).uniform(-1.0, 1.0, (3, 16 * hl, 16 * hl)).astype(np.float32)
        for _ in range(2):
            vae.encode(rgbf)
        t0 = time.perf_counter()
        for _ in range(iters):
            vae.encode(rgbf)
        enc_ms = (time.perf_counter() - t0) * 1e3 / iters
        emit({"micro": "vae", "image": [16 * hl, 16 * hl], "ms_device": ms, "ms_e2e": e2e,
                          "encode_ms_e2e": enc_ms,
                          "launches": vae.last_launches(), "conv_tflops": flops / ms / 1e9,
                          "algorithmic_gflop": flops / 1e9, "image_std": float(img.std()),
                          "peak_source": peaks["source"]})
        vae.close()
    elif args.micro == "qwen3":
        # The text encoder at the Qwen3-4B shape (only the 27 layers the output depends on are built), one prompt
        # of --seq tokens through the host-buffer entry point: token ids in, [seq, 7680] f32 embeddings out.
        import numpy as np
        synth = importlib.import_module("flux2_c_b200.synth")
        nl = max(3, args.layers)  # three distinct output layers are read
        d = synth.QwenDims(layers=27) if nl >= 27 else synth.QwenDims(layers=nl, out_layers=(0, nl // 2, nl - 1))
        W = synth.make_qwen_weights(d, seed=0, threads=os.cpu_count())
        B = max(1, args.prompt_batch)
        enc = fx.TextEncoder.from_tensors(ctx, d, W, max_seq=max(512, args.seq) * B)
        del W
        seq = args.seq
        ids = np.random.default_rng(0).integers(0, d.vocab, (B, seq))
        for _ in range(max(3, args.warmup)):
            out = enc.forward_batch(ids, None)
        t0 = time.perf_counter()
        for _ in range(iters):
            out = enc.forward_batch(ids, None)
        ms = (time.perf_counter() - t0) * 1e3 / iters / B
        dev_ms = timed(lambda: enc.forward_batch(ids, None, device=True)) / B
        qd, kd = d.heads * d.head_dim, d.kv_heads * d.head_dim
        per_layer = 2.0 * seq * (d.hidden * (qd + 2 * kd) + qd * d.hidden + 3 * d.hidden * d.inter) + 2.0 * seq * seq * qd
        flops = d.layers * per_layer
        wbytes = d.layers * 2.0 * (d.hidden * (qd + 2 * kd) + qd * d.hidden + 3 * d.hidden * d.inter)
        emit({"micro": "qwen3", "seq": seq, "prompts_per_pass": B, "layers_run": d.layers, "ms_per_prompt_e2e": ms,
                          "ms_per_prompt_device": dev_ms, "model_tflops_device": flops / dev_ms / 1e9,
                          "model_tflops": flops / ms / 1e9, "weight_gb_per_pass": wbytes / 1e9,
                          "weight_stream_ms_at_hbm_peak": wbytes / peaks["hbm_gbs"] / 1e6,
                          "d2h_bytes": int(out.nbytes), "finite": bool(np.isfinite(out).all()),
                          "peak_source": peaks["source"]})
        enc.close()
    return 0


# ---------------------------------------------------------------------------------------------- text encoder leg
SWEEP_IMAGES = 64


def prompt_to_latent_pass(args, fx, synth, ctx, sampler, sched, stream, barrier, all_ranks, rank, world, dist):
    """The throughput-sweep configuration: SWEEP_IMAGES independent images split over the ranks (image i on rank
    i % world), each from its own 512 token ids (seed 20000 + i) and its own noise (seed i). Per image: text-encoder
    forward (Qwen3-4B shape; the 27 layers the output depends on - later layers are neither generated nor run, as in
    the reference's device path), embeddings handed to the sampler on the device, 4 DiT steps, latent read back.
    Host -> device per image: ids + noise. A fixed number of images: strong scaling; the job's time is the slowest
    rank's."""
    import importlib
    import numpy as np
    import torch
    dp = importlib.import_module("flux2_c_b200.dp")
    qd = synth.QwenDims(layers=27)
    dims = synth.Dims.klein4b()
    PB = max(1, args.prompt_batch)  # prompts per encoder pass: the weights are read once for the group

    def all_ok(ok):
        # every rank calls this the same number of times, whether its own part worked or not, so that a failure on
        # one rank ends the leg everywhere instead of leaving the others waiting in a barrier
        if world == 1:
            return ok
        t = torch.tensor([1.0 if ok else 0.0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item() > 0.5)

    enc, err = None, None
    t_setup = time.perf_counter()
    if world == 1:
        enc = fx.TextEncoder.from_tensors(ctx, qd, synth.make_qwen_weights(qd, seed=0, threads=os.cpu_count()),
                                          max_seq=TXT * PB)
    else:
        shm = "/dev/shm" if os.path.isdir("/dev/shm") and os.access("/dev/shm", os.W_OK) else tempfile.gettempdir()
        mdir = os.path.join(shm, "flux_bench_qwen_%s" % os.environ.get("MASTER_PORT", "0"))
        try:
            if rank == 0:
                synth.write_qwen_shards(mdir, synth.make_qwen_weights(qd, seed=0, threads=os.cpu_count()))
        except Exception as e:
            err = e
        wrote = all_ok(err is None)
        try:
            if wrote:
                enc = fx.TextEncoder.load_dir(ctx, mdir, max_seq=TXT * PB)
        except Exception as e:
            err = e
        loaded = all_ok(wrote and enc is not None)
        if rank == 0:
            import shutil
            shutil.rmtree(mdir, ignore_errors=True)
        if not loaded:
            if enc is not None:
                enc.close()
            raise RuntimeError("text encoder set-up failed on some rank: %r" % (err,))
    setup_s = time.perf_counter() - t_setup
    mine = dp.images_of_rank(SWEEP_IMAGES, rank, world)
    n = len(mine)
    ids = np.stack([np.random.default_rng(20000 + i).integers(0, qd.vocab, TXT) for i in mine]).astype(np.int32)
    n_lat = dims.latent_ch * H_LAT * W_LAT
    z = torch.stack([torch.from_numpy(fx.init_noise(dims.latent_ch, H_LAT, W_LAT, i)).reshape(-1)
                     for i in mine]).pin_memory()
    out = torch.zeros(n, n_lat, dtype=torch.float32).pin_memory()
    ctx_bytes = TXT * 3 * qd.hidden * 4

    def run_images(count, per_image):
        """The first `count` of this rank's images: prompts are encoded PB at a time; the embeddings of prompt j of a
        group sit at dev + j * ctx_bytes until the next group is encoded, which the stream orders after the uploads
        that read them."""
        done = 0
        while done < count:
            g = min(PB, count - done)
            dev = enc.forward_batch(ids[done:done + g], None, device=True)
            for j in range(g):
                sampler.upload(z[done + j].data_ptr(), dev + j * ctx_bytes)
                sampler.run(sched)
                per_image(done + j)
            done += g

    def timed(count, per_image):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record()
        run_images(count, per_image)
        with torch.cuda.stream(stream):
            e1.record()
        barrier()
        return all_ranks(e0.elapsed_time(e1))

    to_latent = lambda j: sampler.download(out[j].data_ptr())  # waits for the image
    run_images(min(n, max(3, PB)), to_latent)
    rank_ms = timed(n, to_latent)
    ms = max(rank_ms)
    # the encoder alone, device time per prompt
    reps = max(2, min(10, args.steps))
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record()
    for i in range(reps):
        enc.forward_batch(ids[:min(PB, n)], None, device=True)
    with torch.cuda.stream(stream):
        e1.record()
    barrier()
    enc_ms = max(all_ranks(e0.elapsed_time(e1))) / reps / min(PB, n)
    finite = bool(torch.isfinite(out).all())

    # the same plus the VAE decoder: the latent goes from the sampler to the decoder on the device, the 512x512 RGB
    # image (786 KB) is what returns to the host
    vae = fx.Vae.from_tensors(ctx, synth.make_vae_weights(seed=5, rich=True))
    rgb = torch.zeros(16 * H_LAT * 16 * W_LAT * 3, dtype=torch.uint8).pin_memory()

    to_image = lambda j: vae.decode_ptr(sampler.latent_device(), H_LAT, W_LAT, rgb.data_ptr())  # waits for the image
    run_images(min(n, max(3, PB)), to_image)
    img_rank_ms = timed(n, to_image)
    img_ms = max(img_rank_ms)
    barrier()
    with torch.cuda.stream(stream):
        e0.record()
    for i in range(reps):
        vae.decode_device(sampler.latent_device(), H_LAT, W_LAT)
    with torch.cuda.stream(stream):
        e1.record()
    barrier()
    vae_ms = max(all_ranks(e0.elapsed_time(e1))) / reps
    img_std = float(rgb.float().std())
    vae.close()
    enc.close()
    return {"workload": "%d images over %d GPU(s), image i on rank i %% N; per image: %d token ids (seed 20000 + i) -> "
            "Qwen3-4B-shaped encoder (27 of 36 layers: the ones the output depends on; %d prompts per encoder pass) -> "
            "4 DiT steps at 512x512 from noise seed i -> latent on the host" % (SWEEP_IMAGES, world, TXT, PB),
            "images_total": SWEEP_IMAGES, "scaling": "strong", "value": SWEEP_IMAGES / (ms * 1e-3),
            "unit": "images/s", "ms_per_image": ms / max(1, -(-SWEEP_IMAGES // world)),
            "per_rank_ms": {"min": min(rank_ms), "max": max(rank_ms)},
            "text_encoder_ms_per_prompt": enc_ms, "prompts_per_encoder_pass": PB,
            "h2d_bytes_per_image": int(TXT * 4 + n_lat * 4), "d2h_bytes_per_image": int(n_lat * 4),
            "finite": finite, "encoder_setup_s": setup_s,
            "prompt_to_image": {"workload": "the same, then the VAE decoder on the device; a 512x512 uint8 RGB image "
                                "returns to the host", "value": SWEEP_IMAGES / (img_ms * 1e-3), "unit": "images/s",
                                "ms_per_image": img_ms / max(1, -(-SWEEP_IMAGES // world)),
                                "per_rank_ms": {"min": min(img_rank_ms), "max": max(img_rank_ms)},
                                "vae_decode_ms": vae_ms, "d2h_bytes_per_image": int(rgb.numel()),
                                "image_std": img_std}}


# ---------------------------------------------------------------------------------------------- other configurations
CONFIGS = {
    1: dict(name="klein4b_256x256_4step_b1", h=16, w=16, steps=4, guidance=1.0, ref=None),
    3: dict(name="klein4b_base_512x512_50step_cfg4_pair_as_batch2", h=32, w=32, steps=50, guidance=4.0, ref=None),
    4: dict(name="klein4b_img2img_1024x1024_4step_1ref_8704tok", h=64, w=64, steps=4, guidance=1.0, ref=(64, 64, 10)),
}


def run_config(args):
    """The other single-GPU configurations of the workload list (the default run is configuration 2): images/s with
    the inputs resident, K images back to back, CUDA events on the engine's stream. One JSON line of its own."""
    import numpy as np
    import torch
    import torch.distributed as dist
    fx = load_package()
    import flux2_c_b200.synth as synth
    c = CONFIGS[args.config]
    if args.group:
        return run_config_group(args, fx, synth, c)
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    pair = world == 2 and args.config == 3  # the guidance pair split across two GPUs, one exchange per step
    if world > 1:
        if not pair:
            raise SystemExit("--config under torchrun: only configuration 3 on exactly two ranks (the guidance pair)")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dims = synth.Dims.klein4b()
    ctx = fx.Context(local)
    model = fx.Model.from_tensors(ctx, dims, synth.make_transformer_weights(dims, seed=0,
                                                                            threads=max(1, os.cpu_count() // world)))
    h, w, steps, g = c["h"], c["w"], c["steps"], c["guidance"]
    batch = 2 if g != 1.0 else 1
    refs = [c["ref"]] if c["ref"] else []
    z0 = torch.from_numpy(fx.init_noise(dims.latent_ch, h, w, 42)).pin_memory()
    cc = torch.from_numpy(synth.make_context(1234, TXT, dims.text_dim)).pin_memory()
    cu = torch.from_numpy(synth.make_context(4321, TXT, dims.text_dim)).pin_memory()
    ref_lat = [torch.from_numpy(synth.make_latent(7, dims.latent_ch, r[0], r[1])).pin_memory() for r in refs]
    sched = fx.official_schedule(steps, h * w)
    stream = torch.cuda.ExternalStream(ctx.stream)
    if pair:
        dp = importlib.import_module("flux2_c_b200.dp")
        _, is_cond = dp.pair_of_rank(rank)
        group = dp.pair_groups(world)
        sampler = fx.Sampler(model, h, w, TXT, batch=1, max_steps=steps)
        v_buf = torch.zeros(dims.latent_ch * h * w, dtype=torch.float32, device="cuda")
        mine = cc if is_cond else cu

        def one_image():
            sampler.upload(z0.data_ptr(), mine.data_ptr())
            with torch.cuda.stream(stream):
                dp.sample_cfg_pair(sampler, sched, g, is_cond, v_buf, group)
    else:
        sampler = fx.Sampler(model, h, w, TXT, ref_shapes=refs, batch=batch, max_steps=steps)
        sampler.upload(z0.data_ptr(), cc.data_ptr(), cu.data_ptr() if batch == 2 else None,
                       [t.data_ptr() for t in ref_lat])

        def one_image():
            sampler.run(sched, guidance=g)

    def sync_all():
        if world > 1:
            dist.barrier()
        ctx.sync()
        torch.cuda.synchronize()

    for _ in range(max(1, min(3, args.warmup))):
        one_image()
    sync_all()
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record()
    for _ in range(args.steps):
        one_image()
    with torch.cuda.stream(stream):
        e1.record()
    sync_all()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    clk = clocks.stop() if rank == 0 else None
    out = torch.zeros(dims.latent_ch * h * w, dtype=torch.float32).pin_memory()
    sampler.download(out.data_ptr())
    n_ref = sum(r[0] * r[1] for r in refs)
    N = h * w + n_ref + TXT
    hd, m = dims.hidden, dims.mlp
    lin = dims.n_double * N * 2 * (4 * hd * hd + 3 * hd * m) + dims.n_single * N * 2 * (hd * (3 * hd + 2 * m) + (hd + m) * hd)
    lin += 2 * (h * w + n_ref) * dims.latent_ch * hd + 2 * h * w * hd * dims.latent_ch
    attn = (dims.n_double + dims.n_single) * 4 * N * N * hd
    flops = batch * steps * (lin + attn) + batch * 2 * TXT * dims.text_dim * hd
    if pair:
        c = dict(c, name="klein4b_base_512x512_50step_cfg4_pair_split_across_2_gpus")
    if rank == 0:
        emit({"config": args.config, "workload": c["name"], "value": 1e3 / ms, "unit": "images/s",
                          "n_gpus": world, "ms_per_image": ms, "ms_per_dit_step": ms / steps,
                          "dit_steps_per_image": steps, "batch": batch, "tokens": N, "model_tflops": flops / ms / 1e9,
                          "attention_share_of_flops": batch * steps * attn / flops, "images_timed": args.steps,
                          "finite": bool(torch.isfinite(out).all()), "clocks": clk, "dtype": "f16", "data": "synthetic"})
    sampler.close()
    model.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def run_config_group(args, fx, synth, c):
    """--config 3 --group: the guidance pair split over GPUs 0 and 1 through the C ABI's own group calls
    (flux_cuda_group_sample_cfg_pair: one process, one internal host thread per GPU, peer-memory exchange), timed as a
    host call with host buffers in and the latent out, against the same image as a batch of two on GPU 0."""
    import numpy as np
    import torch
    if args.config != 3 or torch.cuda.device_count() < 2:
        raise SystemExit("--group: configuration 3 on a box with at least two GPUs")
    dims = synth.Dims.klein4b()
    W = synth.make_transformer_weights(dims, seed=0, threads=os.cpu_count())
    g = fx.Group([0, 1])
    models = [fx.Model.from_tensors(g.context(r), dims, W) for r in range(2)]
    del W
    g.set_models(models)
    h, w, steps, guidance = c["h"], c["w"], c["steps"], c["guidance"]
    z0 = fx.init_noise(dims.latent_ch, h, w, 42)
    cc = synth.make_context(1234, TXT, dims.text_dim)
    cu = synth.make_context(4321, TXT, dims.text_dim)
    sched = fx.official_schedule(steps, h * w)
    pair = g.sample_cfg_pair(z0, h, w, cc, cu, guidance, sched)  # warm-up, and the result to compare
    t0 = time.perf_counter()
    for _ in range(args.steps):
        pair = g.sample_cfg_pair(z0, h, w, cc, cu, guidance, sched)
    pair_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    one = models[0].sample(z0, h, w, cc, sched, ctx_uncond=cu, guidance=guidance)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one = models[0].sample(z0, h, w, cc, sched, ctx_uncond=cu, guidance=guidance)
    one_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    err = float(np.linalg.norm(pair.astype(np.float64) - one) / np.linalg.norm(one.astype(np.float64)))
    emit({"config": 3, "workload": "klein4b_base_512x512_50step_cfg4_pair_split_across_2_gpus_c_abi_group",
          "value": 1e3 / pair_ms, "unit": "images/s", "n_gpus": 2, "ms_per_image": pair_ms,
          "ms_per_dit_step": pair_ms / steps, "one_gpu_batch_of_two_ms_per_image": one_ms,
          "speedup_over_one_gpu": one_ms / pair_ms, "rel_l2_against_one_gpu": err, "images_timed": args.steps,
          "timing": "host wall clock around the call: host buffers in, latent out", "dtype": "f16",
          "data": "synthetic"})
    for m in models:
        m.close()
    g.close()
    return 0


# ---------------------------------------------------------------------------------------------- main arm
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: the engine has no CPU path")

    fx = load_package()
    import flux2_c_b200.synth as synth
    dims = synth.Dims.klein4b()
    ctx = fx.Context(local)
    if args.half != "f16":
        ctx.set_half_format(args.half)  # before the model is loaded: the weights are stored in this format

    # ---- model: rank 0 generates the seeded weights once; other ranks read the same file through the loader
    # (all of this is set-up, outside every timed region; its duration is reported as setup_s)
    t_setup = time.perf_counter()
    W = None
    if world == 1:
        W = synth.make_transformer_weights(dims, seed=0, threads=os.cpu_count())
        t_weights = time.perf_counter() - t_setup
        model = fx.Model.from_tensors(ctx, dims, W)
    else:
        shm = "/dev/shm" if os.path.isdir("/dev/shm") and os.access("/dev/shm", os.W_OK) else tempfile.gettempdir()
        path = os.path.join(shm, "flux_bench_%s.safetensors" % os.environ.get("MASTER_PORT", "0"))
        if rank == 0:
            synth.write_safetensors(path, synth.make_transformer_weights(dims, seed=0, threads=os.cpu_count()))
        dist.barrier()
        t_weights = time.perf_counter() - t_setup
        model = fx.Model.load_safetensors(ctx, path)
        dist.barrier()
        if rank == 0:
            os.remove(path)
    t_load = time.perf_counter() - t_setup - t_weights

    # ---- inputs: `steps` images per rank (weak scaling). Image i of the job has noise seed i and the context of
    # seed 10000 + i and runs on rank i % world. Pinned host copies for the end-to-end region, device copies for the
    # device-resident one.
    dp = importlib.import_module("flux2_c_b200.dp")
    mine = dp.images_of_rank(args.steps * world, rank, world)
    n_lat = dims.latent_ch * H_LAT * W_LAT
    z_host = torch.stack([torch.from_numpy(fx.init_noise(dims.latent_ch, H_LAT, W_LAT, i)).reshape(-1)
                          for i in mine]).pin_memory()
    c_host = torch.stack([torch.from_numpy(synth.make_context(10000 + i, TXT, dims.text_dim)).reshape(-1)
                          for i in mine]).pin_memory()
    z_dev, c_dev = z_host.cuda(), c_host.cuda()
    out = torch.zeros(len(mine), n_lat, dtype=torch.float32).pin_memory()
    sched = fx.official_schedule(STEPS_PER_IMAGE, H_LAT * W_LAT)
    sampler = fx.Sampler(model, H_LAT, W_LAT, TXT, batch=1, max_steps=STEPS_PER_IMAGE)
    stream = torch.cuda.ExternalStream(ctx.stream)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        ctx.sync()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def all_ranks(ms):
        if world == 1:
            return [ms]
        t = torch.tensor([ms], device="cuda")
        got = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(got, t)
        return [float(x.item()) for x in got]

    def resident(j):  # inputs of image j are already in HBM: a device-to-device copy into the sampler's buffers
        sampler.upload(z_dev[j].data_ptr(), c_dev[j].data_ptr())
        sampler.run(sched)

    def end_to_end(j):  # pinned host inputs in, latent out on the host; download waits for the image
        sampler.upload(z_host[j].data_ptr(), c_host[j].data_ptr())
        sampler.run(sched)
        sampler.download(out[j].data_ptr())

    if args.ncu_range:
        # one warm image, then exactly one image between cudaProfilerStart/Stop (ncu --profile-from-start off)
        resident(0)
        ctx.sync()
        torch.cuda.profiler.start()
        resident(0)
        ctx.sync()
        torch.cuda.profiler.stop()
        emit({"ncu_range": "one image", "launches": sampler.last_run()[1]})
        return 0

    # ---- device-resident timing: inputs already in HBM, K images back to back
    K = len(mine)
    for w_i in range(max(3, args.warmup)):
        resident(w_i % K)
    barrier()
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record()
        for j in range(K):
            resident(j)
        e1.record()
    barrier()
    my_ms = e0.elapsed_time(e1)
    rank_ms = all_ranks(my_ms)
    ms_total = max(rank_ms)
    launches = sampler.last_run()[1] * K

    # ---- end to end through the host-buffer API: H2D of the inputs and D2H of the latent inside the region.
    # (a) one image at a time: upload, run, download, and the host waits for the image before it queues the next;
    for j in range(2):
        end_to_end(j % K)
    barrier()
    with torch.cuda.stream(stream):
        e0.record()
    for j in range(K):
        end_to_end(j)
    with torch.cuda.stream(stream):
        e1.record()
    barrier()
    e2e_serial_ms = max_over_ranks(max(e0.elapsed_time(e1), 0.0))

    # (b) pipelined, the way a host generates many images: the inputs of image j + 1 cross PCIe on the library's copy
    # stream while image j is computed, the latent's device -> host copy is queued behind the run, one wait at the end.
    def pipelined():
        sampler.stage_inputs(z_host[0].data_ptr(), c_host[0].data_ptr())
        for j in range(K):
            sampler.run(sched)  # picks up the staged inputs of image j
            if j + 1 < K:
                sampler.stage_inputs(z_host[j + 1].data_ptr(), c_host[j + 1].data_ptr())
            sampler.download_async(out[j].data_ptr())
        ctx.sync()

    pipelined()
    out.zero_()
    barrier()
    t0 = time.perf_counter()
    with torch.cuda.stream(stream):
        e0.record()
    pipelined()
    with torch.cuda.stream(stream):
        e1.record()
    barrier()
    e2e_ms = max_over_ranks(max(e0.elapsed_time(e1), 0.0))
    e2e_wall_ms = max_over_ranks((time.perf_counter() - t0) * 1e3)
    clk = clocks.stop() if rank == 0 else None
    finite = bool(torch.isfinite(out).all()) and float(out.std()) > 0.0
    distinct = K < 2 or not torch.equal(out[0], out[1])  # different seeds must give different images
    saturated = ctx.saturated_stores()
    z0, cemb = z_host[0], c_host[0]
    sampler.upload(z_dev[0].data_ptr(), c_dev[0].data_ptr())

    # ---- roofline of the dominant kernel (the tcgen05 GEMM): per-class CUDA-event times of the same loop
    fl = step_flops(H_LAT * W_LAT, TXT, dims)
    prof = None
    try:
        # several images back to back so that the profiled one runs at the same sustained (power-capped) clocks
        # as the timed region; the event pairs of the last image are the ones read
        sampler.set_profiling(True)
        for _ in range(max(3, min(args.steps, 6))):
            sampler.run(sched)
        ctx.sync()
        prof = sampler.profile()
        if args.dump_launches:
            with open(args.dump_launches, "w") as f:
                json.dump(sampler.profile_launches(), f)
        sampler.set_profiling(False)
    except AttributeError:
        pass
    peaks = measured_peaks()
    roof = None
    roof_all = None
    if prof and prof["gemm"]["ms"] > 0:
        gemm_flops = STEPS_PER_IMAGE * fl["gemm"] + fl["ctx_embed_once"]
        ach = gemm_flops / (prof["gemm"]["ms"] * 1e-3) / 1e12
        roof_all = {"bound": "tensor", "kernel": "all GEMM launches of one image (gemm2_bf16_tn_kernel; "
                    "gemm_bf16_tn_kernel<128> for proj_out)", "achieved": ach, "peak": peaks["bf16_sustained"],
                    "unit": "TFLOP/s", "frac": ach / peaks["bf16_sustained"], "launches_per_image": prof["gemm"]["n"],
                    "per_class_ms_per_image": {k: v["ms"] for k, v in prof.items()}}
        # the dominant kernel + shape: the single-stream linear1 GEMM [N x 3072] . [3072 x 27648] (80 launches per
        # image, 55 % of the FLOPs). GEMM launch order inside an image: 1 context embed, then per DiT step
        # 1 x_embed, 4 per double block, (linear1, linear2) per single block, 1 proj_out.
        gl = [ms for ms, cls in sampler.profile_launches() if cls == 0]
        per_step = 2 + 4 * dims.n_double + 2 * dims.n_single
        lin1 = []
        for st in range(STEPS_PER_IMAGE):
            base = 1 + st * per_step + 1 + 4 * dims.n_double
            lin1 += [gl[base + 2 * j] for j in range(dims.n_single)] if len(gl) >= 1 + STEPS_PER_IMAGE * per_step else []
        if lin1:
            n_tok = H_LAT * W_LAT + TXT
            f1 = 2.0 * n_tok * dims.hidden * (3 * dims.hidden + 2 * dims.mlp)
            ms1 = sum(lin1) / len(lin1)
            a1 = f1 / (ms1 * 1e-3) / 1e12
            roof = {"bound": "tensor", "kernel": "gemm2_bf16_tn_kernel (f16 operands, CTA pairs) on the single-stream linear1 shape "
                    "[%d x %d] . [%d x %d]" % (n_tok, dims.hidden, dims.hidden, 3 * dims.hidden + 2 * dims.mlp),
                    "achieved": a1, "peak": peaks["bf16_sustained"], "unit": "TFLOP/s",
                    "frac": a1 / peaks["bf16_sustained"],
                    # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this very shape under ncu: a
                    # figure quoted from the committed capture, not measured by this run; algorithmic bytes 264.2 MB
                    "traffic": 243.6e6, "traffic_source": "profiles/gemm2_bf16_tn_1536x27648x3072.md (ncu, one launch)",
                    "launches": len(lin1), "avg_launch_ms": ms1,
                    "flops_per_launch": f1, "peak_source": peaks["source"] + " (sustained cuBLAS bf16)",
                    "frac_of_burst_peak": a1 / peaks["bf16"]}
    images = args.steps * world
    value = images / (ms_total * 1e-3)
    line = {
        "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_total / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": args.half, "data": "synthetic",
        "config": bench_config(world),
        "ms_per_dit_step": ms_total / args.steps / STEPS_PER_IMAGE,
        "model_tflops": (STEPS_PER_IMAGE * (fl["gemm"] + fl["attn"]) + fl["ctx_embed_once"]) * args.steps /
                        (ms_total * 1e-3) / 1e12,
        "e2e": {"value": images / (e2e_ms * 1e-3), "unit": "images/s", "h2d_bytes_per_step": int(z0.numel() * 4 +
                cemb.numel() * 4), "d2h_bytes_per_step": int(n_lat * 4), "wall_ms_per_step":
                e2e_wall_ms / args.steps, "mode": "pipelined: inputs of the next image staged on a copy stream, "
                "latent downloads queued, one wait at the end", "one_image_at_a_time": images / (e2e_serial_ms * 1e-3)},
        "gpu_launches": int(launches), "finite": finite, "distinct_images": distinct,
        "saturated_f16_stores": int(saturated), "clocks": clk, "roofline": roof or roof_all,
        "roofline_all_gemm": roof_all,
        "per_rank_ms_per_step": {"min": min(rank_ms) / args.steps, "max": max(rank_ms) / args.steps},
        "setup_s": {"weights_generated_and_written": t_weights, "model_load": t_load},
        "prompt_to_latent": None, "leg_timeout": False,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            zc = z0.numpy().reshape(dims.latent_ch, H_LAT, W_LAT)
            cc = cemb.numpy().reshape(TXT, dims.text_dim)
            base = cpu_reference_baseline(synth, W, dims, zc, cc, sched)
            line["cpu_baseline"] = base if base is not None else cpu_port_baseline(synth, W, dims, zc, cc, sched)
        except Exception as e:  # the baseline must never take the GPU numbers down with it
            line["cpu_baseline"] = {"error": repr(e)}

    # ---- the throughput-sweep configuration, last: every image has its own prompt, encoded by the Qwen3-4B-shaped
    # text encoder on the same GPU right before its denoising loop; the embeddings never leave the device. It is an
    # extra leg: if it raises, or does not come back within its time limit, the line above is printed without it.
    if not args.no_text_encoder:
        def give_up():
            # the headline numbers above were measured before this leg started: print them, say that the leg did not
            # come back, and end the process with a failure status so that the stall shows in the run's record
            if rank == 0:
                line["prompt_to_latent"] = {"error": "did not finish within %d s" % args.leg_timeout}
                line["leg_timeout"] = True
                emit(line)
            os._exit(3)

        watchdog = threading.Timer(args.leg_timeout, give_up)
        watchdog.daemon = True
        watchdog.start()
        try:
            line["prompt_to_latent"] = prompt_to_latent_pass(args, fx, synth, ctx, sampler, sched, stream, barrier,
                                                             all_ranks, rank, world, dist if world > 1 else None)
        except Exception as e:
            line["prompt_to_latent"] = {"error": repr(e)}
        watchdog.cancel()
    if rank == 0:
        emit(line)
    sampler.close()
    model.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--micro", default=None, choices=["gemm", "gemmtable", "attn", "adaln", "qwen3", "vae", "conv", "gn", "load", "step"])
    ap.add_argument("--half", default="f16", choices=["f16", "bf16"],
                    help="16-bit storage format of weights and activations (f32 accumulation either way)")
    ap.add_argument("--shape", type=int, nargs=3, default=[1536, 27648, 3072])
    ap.add_argument("--tile-n", type=int, default=0, help="GEMM tile width: 128, 256, or 512 = CTA pairs")
    ap.add_argument("--epi", default="store", choices=["store", "qkv", "gated", "f32"], help="epilogue of --micro gemm")
    ap.add_argument("--trace", action="store_true", help="--micro gemm --tile-n 512: timeline of the first CTA")
    ap.add_argument("--seq", type=int, default=1536)
    ap.add_argument("--guidance", type=float, default=1.0, help="--micro step: 4 runs the guidance pair (batch of two)")
    ap.add_argument("--layers", type=int, default=27, help="--micro qwen3: encoder layers to build and run")
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--size", type=int, default=512, help="image side for --micro vae")
    ap.add_argument("--config", type=int, default=2, help="1, 3 or 4: another configuration of the workload list")
    ap.add_argument("--group", action="store_true", help="--config 3: the pair through flux_cuda_group_* in one process")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-text-encoder", action="store_true", help="skip the prompt -> latent leg")
    ap.add_argument("--prompt-batch", type=int, default=4, help="prompts encoded per text-encoder pass")
    ap.add_argument("--leg-timeout", type=int, default=300, help="seconds the prompt -> image leg may take")
    ap.add_argument("--dump-launches", default=None, help="write [ms, class] of every launch of one image to this file")
    ap.add_argument("--ncu-range", action="store_true", help="profile exactly one image (for ncu launch lists)")
    args = ap.parse_args()
    global _OUT
    sys.stdout.flush()
    _OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if args.impl == "reference":
        if args.steps == 10:
            args.steps, args.warmup = 2, 1
        return run_reference_arm(args)
    if args.micro:
        return run_micro(args)
    if args.config in CONFIGS:
        return run_config(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
