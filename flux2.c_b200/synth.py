"""Seeded synthetic workloads in the reference's on-disk and in-memory formats.

No model weights, prompts or images can be downloaded where this runs, so every test and
benchmark uses klein-4B-*shaped* random tensors: bf16 weights N(0, 0.02^2) laid out and named as
the reference's loader expects (flux_transformer.c:4452-4602), bf16-representable N(0,1) text
context, N(0,1) reference latents. The generator is numpy's Philox, keyed per tensor, so a tensor's
values depend only on (seed, tensor index) and tensors can be produced in parallel and in any
order; results are identical on any machine with the same numpy.
"""
import json
import struct
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class Dims:
    hidden: int = 3072
    heads: int = 24
    head_dim: int = 128
    mlp: int = 9216
    n_double: int = 5
    n_single: int = 20
    text_dim: int = 7680
    latent_ch: int = 128
    time_dim: int = 256
    rope_theta: float = 2000.0
    axis_dim: int = 32

    @staticmethod
    def klein4b():
        """The shape the reference hard-codes (flux_transformer.c:4418-4434)."""
        return Dims()

    @staticmethod
    def tiny():
        """Same structure at a size a CPU test evaluates in milliseconds."""
        return Dims(hidden=256, heads=2, head_dim=128, mlp=768, n_double=1, n_single=2, text_dim=192)


def bf16_round(x):
    """f32 array -> f32 array holding the nearest-even bf16 value of each element."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u + (0x7FFF + ((u >> 16) & 1))) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32)


def f32_to_bf16_bits(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def transformer_tensor_specs(d: Dims):
    """Ordered (name, shape, kind) of every tensor of the DiT; kind 'qknorm' marks the per-head RMSNorm weights."""
    h, m = d.hidden, d.mlp
    specs = [
        ("x_embedder.weight", (h, d.latent_ch), "w"),
        ("context_embedder.weight", (h, d.text_dim), "w"),
        ("time_guidance_embed.timestep_embedder.linear_1.weight", (h, d.time_dim), "w"),
        ("time_guidance_embed.timestep_embedder.linear_2.weight", (h, h), "w"),
        ("double_stream_modulation_img.linear.weight", (6 * h, h), "w"),
        ("double_stream_modulation_txt.linear.weight", (6 * h, h), "w"),
        ("single_stream_modulation.linear.weight", (3 * h, h), "w"),
        ("norm_out.linear.weight", (2 * h, h), "w"),
        ("proj_out.weight", (d.latent_ch, h), "w"),
    ]
    for i in range(d.n_double):
        p = "transformer_blocks.%d." % i
        for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
            specs.append((p + "attn.%s.weight" % n, (d.head_dim,), "qknorm"))
        for n in ("to_q", "to_k", "to_v", "to_out.0", "add_q_proj", "add_k_proj", "add_v_proj", "to_add_out"):
            specs.append((p + "attn.%s.weight" % n, (h, h), "w"))
        specs.append((p + "ff.linear_in.weight", (2 * m, h), "w"))
        specs.append((p + "ff.linear_out.weight", (h, m), "w"))
        specs.append((p + "ff_context.linear_in.weight", (2 * m, h), "w"))
        specs.append((p + "ff_context.linear_out.weight", (h, m), "w"))
    for j in range(d.n_single):
        p = "single_transformer_blocks.%d." % j
        specs.append((p + "attn.norm_q.weight", (d.head_dim,), "qknorm"))
        specs.append((p + "attn.norm_k.weight", (d.head_dim,), "qknorm"))
        specs.append((p + "attn.to_qkv_mlp_proj.weight", (3 * h + 2 * m, h), "w"))
        specs.append((p + "attn.to_out.weight", (h, h + m), "w"))
    return specs


def _gen_tensor(seed, index, shape, std):
    n = int(np.prod(shape))
    rng = np.random.Generator(np.random.Philox(key=[np.uint64(seed), np.uint64(index)]))
    out = np.empty(n, dtype=np.uint16)
    chunk = 1 << 24
    for s in range(0, n, chunk):
        e = min(n, s + chunk)
        v = rng.standard_normal(e - s, dtype=np.float32)
        v *= np.float32(std)
        out[s:e] = f32_to_bf16_bits(v)
    return out.reshape(shape)


def make_transformer_weights(d: Dims, seed=0, sharp=False, std=0.02, threads=None):
    """dict name -> uint16 array of bf16 bit patterns.

    sharp=False is the benchmark's init (every element N(0, std^2), QK-norm vectors included, which
    makes attention logits ~1e-4 and softmax uniform). sharp=True sets the QK-norm vectors to 1.0 so
    that attention is position- and content-sensitive; parity tests use it to catch RoPE / scale /
    key-order mistakes the benchmark init cannot see.
    """
    specs = transformer_tensor_specs(d)
    one = np.uint16(0x3F80)  # bf16(1.0)

    def job(arg):
        idx, (name, shape, kind) = arg
        if kind == "qknorm" and sharp:
            return name, np.full(shape, one, dtype=np.uint16)
        return name, _gen_tensor(seed, idx, shape, std)

    with ThreadPoolExecutor(max_workers=threads or 8) as ex:
        return dict(ex.map(job, list(enumerate(specs))))


def make_context(seed, txt_seq=512, text_dim=7680):
    """f32 [txt_seq, text_dim], N(0,1) rounded to bf16-representable values."""
    rng = np.random.Generator(np.random.Philox(key=[np.uint64(seed), np.uint64(0xC0)]))
    return bf16_round(rng.standard_normal((txt_seq, text_dim), dtype=np.float32))


def make_latent(seed, ch, h, w):
    """f32 [ch, h, w] N(0,1): stand-in for noise or a VAE-encoded reference image."""
    rng = np.random.Generator(np.random.Philox(key=[np.uint64(seed), np.uint64(0x1A)]))
    return rng.standard_normal((ch, h, w), dtype=np.float32)


def write_safetensors(path, tensors, dtype="BF16"):
    """Writes name -> array (uint16 bf16 bits for BF16, float32 for F32) in safetensors layout:
    8-byte little-endian header length, JSON header, raw little-endian data (flux_safetensors.c:155-292)."""
    header = {}
    off = 0
    for name, arr in tensors.items():
        nbytes = arr.size * arr.itemsize
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for arr in tensors.values():
            f.write(np.ascontiguousarray(arr).tobytes() if arr.size < (1 << 20) else memoryview(np.ascontiguousarray(arr)))
    return off + 8 + len(hj)
