"""Synthetic-workload generator: bf16 rounding, tensor inventory, safetensors layout."""
import json
import struct

import numpy as np


def test_bf16_rounding_is_nearest_even(fx):
    import flux2_c_b200.synth as synth
    import torch
    x = np.random.default_rng(0).standard_normal(10000).astype(np.float32) * 3
    want = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    assert np.array_equal(synth.bf16_round(x), want)
    assert np.array_equal(synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(x)), want)


def test_klein_inventory_matches_the_reference_loader(fx):
    import flux2_c_b200.synth as synth
    specs = synth.transformer_tensor_specs(synth.Dims.klein4b())
    assert len(specs) == 169
    assert sum(int(np.prod(s)) for _, s, _ in specs) == 3875544576
    assert sum(1 for _, _, k in specs if k == "qknorm") == 60


def test_weights_are_deterministic_and_scaled(fx):
    import flux2_c_b200.synth as synth
    d = synth.Dims.tiny()
    a = synth.make_transformer_weights(d, seed=0)
    b = synth.make_transformer_weights(d, seed=0, threads=2)
    c = synth.make_transformer_weights(d, seed=1)
    assert all(np.array_equal(a[k], b[k]) for k in a)
    assert not np.array_equal(a["proj_out.weight"], c["proj_out.weight"])
    w = synth.bf16_bits_to_f32(a["single_transformer_blocks.0.attn.to_qkv_mlp_proj.weight"])
    assert abs(w.std() - 0.02) < 5e-4 and abs(w.mean()) < 5e-4
    s = synth.make_transformer_weights(d, seed=0, sharp=True)
    assert np.all(synth.bf16_bits_to_f32(s["transformer_blocks.0.attn.norm_q.weight"]) == 1.0)


def test_safetensors_layout(fx, tmp_path):
    import flux2_c_b200.synth as synth
    W = synth.make_transformer_weights(synth.Dims.tiny(), seed=0)
    path = str(tmp_path / "t.safetensors")
    total = synth.write_safetensors(path, W)
    raw = open(path, "rb").read()
    assert len(raw) == total
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    assert set(header) == set(W)
    for name, meta in header.items():
        b, e = meta["data_offsets"]
        assert meta["dtype"] == "BF16" and list(W[name].shape) == meta["shape"]
        got = np.frombuffer(raw[8 + hlen + b:8 + hlen + e], dtype=np.uint16).reshape(meta["shape"])
        assert np.array_equal(got, W[name])


def test_synthetic_tokenizer_file_is_read_by_the_reference_tokenizer(fx, tmp_path):
    """The byte-level tokenizer.json written for the prompt-driven CLI test must load in the reference's own loader and
    tokenize a prompt into the chat template (special ids are constants of the loader, flux_qwen3_tokenizer.c:25-29)."""
    import ctypes
    import pytest
    import flux2_c_b200.synth as synth
    from oracle import ref_binding as rb
    kind = rb.best_kind()
    if kind is None:
        pytest.skip("the reference build (oracle/_ref) is not present")
    path = str(tmp_path / "tokenizer" / "tokenizer.json")
    synth.write_tokenizer_json(path)
    L = rb.RefLib(kind).L
    L.qwen3_tokenizer_load.restype = ctypes.c_void_p
    L.qwen3_tokenizer_load.argtypes = [ctypes.c_char_p]
    L.qwen3_tokenize_chat.restype = ctypes.POINTER(ctypes.c_int)
    L.qwen3_tokenize_chat.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_int), ctypes.c_int]
    tok = L.qwen3_tokenizer_load(path.encode())
    assert tok
    n = ctypes.c_int()
    ids = L.qwen3_tokenize_chat(tok, b"a cat in the rain", ctypes.byref(n), 512)
    got = [ids[i] for i in range(n.value)]
    assert got[0] == 151644 and 151645 in got and 151667 in got and 151668 in got
    body = got[got.index(10) + 1:got.index(151645)]  # between "user\\n" and <|im_end|>
    assert len(body) >= 8 and all(0 <= t < 262 for t in body)
    assert 260 in body  # the merged pair "the" exists in the vocabulary and is used
