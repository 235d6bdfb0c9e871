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


def vae_tensor_specs():
    """(name, shape, kind) of the 250 tensors the reference's VAE loader reads (flux_vae.c:1150-1354):
    kind 'w' = conv/linear weight, 'one' = norm scale, 'zero' = bias / running mean."""
    specs = []

    def conv(name, cout, cin, k):
        specs.append((name + ".weight", (cout, cin, k, k), "w"))
        specs.append((name + ".bias", (cout,), "zero"))

    def norm(name, ch):
        specs.append((name + ".weight", (ch,), "one"))
        specs.append((name + ".bias", (ch,), "zero"))

    def resblock(prefix, cin, cout):
        norm(prefix + ".norm1", cin)
        conv(prefix + ".conv1", cout, cin, 3)
        norm(prefix + ".norm2", cout)
        conv(prefix + ".conv2", cout, cout, 3)
        if cin != cout:
            conv(prefix + ".conv_shortcut", cout, cin, 1)

    def attn(prefix, ch):
        norm(prefix + ".group_norm", ch)
        for n in ("to_q", "to_k", "to_v", "to_out.0"):
            specs.append((prefix + ".%s.weight" % n, (ch, ch), "w"))
            specs.append((prefix + ".%s.bias" % n, (ch,), "zero"))

    base, mult = 128, (1, 2, 4, 4)
    conv("encoder.conv_in", base, 3, 3)
    for lvl in range(4):
        ch = base * mult[lvl]
        prev = base if lvl == 0 else base * mult[lvl - 1]
        for r in range(2):
            resblock("encoder.down_blocks.%d.resnets.%d" % (lvl, r), prev if (r == 0 and lvl > 0) else ch, ch)
        if lvl < 3:
            conv("encoder.down_blocks.%d.downsamplers.0.conv" % lvl, ch, ch, 3)
    mid = base * mult[3]
    for side in ("encoder", "decoder"):
        resblock(side + ".mid_block.resnets.0", mid, mid)
        attn(side + ".mid_block.attentions.0", mid)
        resblock(side + ".mid_block.resnets.1", mid, mid)
    norm("encoder.conv_norm_out", mid)
    conv("encoder.conv_out", 64, mid, 3)
    conv("quant_conv", 64, 64, 1)
    conv("post_quant_conv", 32, 32, 1)
    conv("decoder.conv_in", mid, 32, 3)
    for lvl in range(3, -1, -1):
        ch = base * mult[lvl]
        prev = mid if lvl == 3 else base * mult[lvl + 1]
        for r in range(3):
            resblock("decoder.up_blocks.%d.resnets.%d" % (3 - lvl, r), prev if r == 0 else ch, ch)
    for i in range(3):
        ch = base * mult[3 - i]
        conv("decoder.up_blocks.%d.upsamplers.0.conv" % i, ch, ch, 3)
    norm("decoder.conv_norm_out", base)
    conv("decoder.conv_out", 3, base, 3)
    specs.append(("bn.running_mean", (128,), "zero"))
    specs.append(("bn.running_var", (128,), "one"))
    return specs


def make_vae_weights(seed=0, std=0.02, rich=False):
    """dict name -> float32 array: conv/linear weights N(0, std^2), norm scales 1, biases and running mean 0,
    running variance 1 (the set the decoded-image PSNR check of the denoising path uses).
    rich=True is the set for the VAE's own parity tests: every bias N(0, 0.1^2), norm scales 1 + N(0, 0.2^2),
    running mean N(0, 0.5^2), running variance uniform(0.5, 2), attention q/k projections ten times larger, so
    that biases, affine terms, de-normalisation and a non-uniform softmax all show in the output."""
    out = {}
    for idx, (name, shape, kind) in enumerate(vae_tensor_specs()):
        rng = np.random.Generator(np.random.Philox(key=[np.uint64(seed), np.uint64(0x7A0000 + idx)]))
        if kind == "w":
            scale = std * (10.0 if rich and (".to_q." in name or ".to_k." in name) else 1.0)
            out[name] = (rng.standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(np.float32)
        elif not rich:
            out[name] = np.full(shape, 1.0 if kind == "one" else 0.0, dtype=np.float32)
        elif name == "bn.running_var":
            out[name] = rng.uniform(0.5, 2.0, shape).astype(np.float32)
        elif name == "bn.running_mean":
            out[name] = (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.5)).astype(np.float32)
        elif kind == "one":
            out[name] = (1.0 + rng.standard_normal(shape, dtype=np.float32) * np.float32(0.2)).astype(np.float32)
        else:
            out[name] = (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.1)).astype(np.float32)
    return out


@dataclass(frozen=True)
class QwenDims:
    """Qwen3 text encoder shape (flux_qwen3.h:21-40)."""
    hidden: int = 2560
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    inter: int = 9728
    layers: int = 36
    vocab: int = 151936
    rope_theta: float = 1000000.0
    out_layers: tuple = (8, 17, 26)  # hidden states after these layers are concatenated

    @staticmethod
    def qwen3_4b():
        return QwenDims()

    @staticmethod
    def tiny():
        return QwenDims(hidden=256, heads=4, kv_heads=2, head_dim=128, inter=512, layers=4, vocab=1000,
                        out_layers=(0, 1, 3))


def qwen_tensor_specs(d: QwenDims):
    """Ordered (name, shape, kind) of the text encoder's tensors (flux_qwen3.c:1216-1251, 1360, 1375)."""
    specs = [("model.embed_tokens.weight", (d.vocab, d.hidden), "w"), ("model.norm.weight", (d.hidden,), "norm")]
    for l in range(d.layers):
        p = "model.layers.%d." % l
        specs += [
            (p + "input_layernorm.weight", (d.hidden,), "norm"),
            (p + "post_attention_layernorm.weight", (d.hidden,), "norm"),
            (p + "self_attn.q_proj.weight", (d.heads * d.head_dim, d.hidden), "w"),
            (p + "self_attn.k_proj.weight", (d.kv_heads * d.head_dim, d.hidden), "w"),
            (p + "self_attn.v_proj.weight", (d.kv_heads * d.head_dim, d.hidden), "w"),
            (p + "self_attn.o_proj.weight", (d.hidden, d.heads * d.head_dim), "w"),
            (p + "self_attn.q_norm.weight", (d.head_dim,), "norm"),
            (p + "self_attn.k_norm.weight", (d.head_dim,), "norm"),
            (p + "mlp.gate_proj.weight", (d.inter, d.hidden), "w"),
            (p + "mlp.up_proj.weight", (d.inter, d.hidden), "w"),
            (p + "mlp.down_proj.weight", (d.hidden, d.inter), "w"),
        ]
    return specs


def make_qwen_weights(d: QwenDims, seed=0, std=0.02, sharp=True, threads=None, max_layer=None):
    """dict name -> uint16 bf16 bits. Linear / embedding weights N(0, std^2). With sharp=True the RMSNorm and
    per-head q/k norm vectors are 1 + N(0, 0.1^2) (a plain N(0, 0.02) init would scale every normalised activation
    by ~0.02 and make attention uniform, hiding RoPE / mask / GQA mistakes); sharp=False draws them like the rest."""
    specs = qwen_tensor_specs(d)

    def wanted(name):  # max_layer: only the embedding and layers 0..max_layer (same values as in the full set)
        if max_layer is None or not name.startswith("model.layers."):
            return True
        return int(name.split(".")[2]) <= max_layer

    def job(arg):
        idx, (name, shape, kind) = arg
        if kind == "norm" and sharp:
            rng = np.random.Generator(np.random.Philox(key=[np.uint64(seed), np.uint64(0x51000000 + idx)]))
            return name, f32_to_bf16_bits(1.0 + 0.1 * rng.standard_normal(shape, dtype=np.float32))
        return name, _gen_tensor(seed, 0x51000000 + idx, shape, std if kind == "w" else std)

    with ThreadPoolExecutor(max_workers=threads or 8) as ex:
        return dict(ex.map(job, [(i, sp) for i, sp in enumerate(specs) if wanted(sp[0])]))


def write_qwen_shards(model_dir, tensors):
    """The two-file layout the reference loader insists on (flux_qwen3.c:1341-1356): both files must exist; a tensor
    may live in either."""
    import os
    os.makedirs(model_dir, exist_ok=True)
    names = list(tensors)
    half = len(names) // 2
    write_safetensors(os.path.join(model_dir, "model-00001-of-00002.safetensors"), {n: tensors[n] for n in names[:half]})
    write_safetensors(os.path.join(model_dir, "model-00002-of-00002.safetensors"), {n: tensors[n] for n in names[half:]})


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


def write_tokenizer_json(path):
    """A minimal byte-level BPE tokenizer file in the layout the reference's loader reads (flux_qwen3_tokenizer.c:
    317-600): "model": {"vocab": {token: id}, "merges": [[left, right], ...]}. The vocabulary is the 256 byte symbols
    of the GPT-2 byte-to-unicode table (ids 0..255) plus a few merged pairs, so any prompt tokenizes; the chat
    template's special tokens have fixed ids inside the loader (flux_qwen3_tokenizer.c:25-29) and need no entry."""
    import os
    bs = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    sym = {b: chr(c) for b, c in zip(bs, cs)}
    vocab = {sym[b]: b for b in range(256)}
    merges = []
    for left, right in (("t", "h"), ("a", "n"), (sym[32], "a"), ("i", "n"), ("th", "e"), (sym[32], "c")):
        merges.append([left, right])
        vocab[left + right] = len(vocab)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "w", encoding="utf-8") as f:
        json.dump({"version": "1.0", "added_tokens": [], "model": {"type": "BPE", "vocab": vocab, "merges": merges}}, f,
                  ensure_ascii=False)
